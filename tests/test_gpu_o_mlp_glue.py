"""The memory-bound steps either side of the MLP's linears: the weight quantiser's global maximum and the two global-scale
conventions, SwiGLU (BF16 out), SwiGLU fused with the FP4 activation quantiser, and the down projection consuming that
result without quantising again."""
import numpy as np
import pytest

from gpu_util import bits_from_dev, to_dev

pytestmark = pytest.mark.gpu


def test_global_absmax_and_scale_conventions(cuda, atlas, oracle):
    from atlas_b200 import synth
    for n in (1, 7, 4096 * 33 + 5):
        x = synth.f32_to_bf16_bits(synth.normal(n, n, 3.0))
        xd = to_dev(cuda, x)
        out = cuda.zeros(1, dtype=cuda.float32, device="cuda")
        atlas.nvfp4_global_absmax(xd, out, n)
        want = oracle.lib().orc_nvfp4_global_absmax(x.ctypes.data, n)
        assert float(out.item()) == want == float(np.abs(oracle.bf16_to_f32(x)).max())
        assert atlas.scale2_from_absmax(want) == np.float32(want) / np.float32(6.0 * 448.0)
    # an odd address takes the scalar loop
    x = synth.f32_to_bf16_bits(synth.normal(9, 1001))
    xd = to_dev(cuda, np.concatenate([[0], x]).astype(np.uint16))
    out = cuda.zeros(1, dtype=cuda.float32, device="cuda")
    atlas.nvfp4_global_absmax(xd.data_ptr() + 2, out, 1001)
    assert float(out.item()) == float(np.abs(oracle.bf16_to_f32(x)).max())
    # ModelOpt stores the multiplier, compressed-tensors its reciprocal; zero stays zero
    assert atlas.combined_global_scale(0.125, False) == 0.125
    assert atlas.combined_global_scale(8.0, True) == 0.125
    assert atlas.combined_global_scale(0.0, True) == 0.0


@pytest.mark.parametrize("limit", [0.0, 10.0])
def test_silu_mul(cuda, atlas, oracle, limit):
    from atlas_b200 import synth
    M, K, stride = 37, 4864, 4864 + 24
    g = synth.f32_to_bf16_bits(synth.normal(1, M * stride, 4.0)).reshape(M, stride)
    u = synth.f32_to_bf16_bits(synth.normal(2, M * stride, 6.0)).reshape(M, stride)
    out = cuda.full((M, K + 8), 0x7FC0, dtype=cuda.int16, device="cuda")
    atlas.silu_mul(to_dev(cuda, g), to_dev(cuda, u), out, M, K, gate_scale=0.5, up_scale=2.0, swiglu_limit=limit,
                   in_row_stride=stride, out_row_stride=K + 8)
    cuda.cuda.synchronize()
    got = bits_from_dev(out)
    assert (got[:, K:] == 0x7FC0).all()
    want = oracle.silu_mul(np.ascontiguousarray(g[:, :K]), np.ascontiguousarray(u[:, :K]), 0.5, 2.0, limit)
    want_bits = synth.f32_to_bf16_bits(want)
    # the fast exponential differs from expf in the last bits: almost always the same BF16, never more than one ulp away
    d = np.abs(got[:, :K].astype(np.int32) - want_bits.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 2e-3
    if limit:
        assert np.abs(oracle.bf16_to_f32(got[:, :K])).max() <= 100.0      # |g| <= 10 from above, |u| <= 10


def test_silu_mul_quant_matches_the_quantiser_on_fp32_values(cuda, atlas, oracle):
    from atlas_b200 import synth
    M, K = 29, 4096
    g = synth.f32_to_bf16_bits(synth.normal(3, M * K, 3.0)).reshape(M, K)
    u = synth.f32_to_bf16_bits(synth.normal(4, M * K, 3.0)).reshape(M, K)
    u[5] = 0                                                              # an all-zero row: zero scale bytes, zero codes
    nbytes = atlas.act_fp4_ws_bytes(M, K)
    ws = cuda.full((nbytes,), 0xA5, dtype=cuda.uint8, device="cuda")
    atlas.silu_mul_quant_nvfp4(to_dev(cuda, g), to_dev(cuda, u), ws, nbytes, M, K, swiglu_limit=10.0)
    cuda.cuda.synchronize()
    raw = ws.cpu().numpy()
    off = (M * (K // 2) + 255) // 256 * 256
    packed, scales = raw[:M * K // 2].reshape(M, K // 2), raw[off:off + M * K // 16].reshape(M, K // 16)
    v = oracle.silu_mul(g, u, 1.0, 1.0, 10.0)
    want_p, want_s = oracle.quantize_f32_to_nvfp4_scale1(v)
    assert not scales[5].any() and not packed[5].any()
    # identical except where the fast exponential moves a value across a bin edge or the group maximum across a scale step
    assert (scales != want_s).mean() < 1e-3 and (packed != want_p).mean() < 2e-3
    got_f = oracle.dequant_nvfp4_to_f32(packed, scales, 1.0, M, K)
    step = np.repeat(oracle.e4m3_decode_array(scales) if hasattr(oracle, "e4m3_decode_array") else
                     np.array([oracle.lib().orc_e4m3_decode(int(b)) for b in scales.reshape(-1)], dtype=np.float32).reshape(scales.shape), 16, axis=1)
    assert (np.abs(got_f - v) <= 1.01 * step).all()                        # within one code step (largest step is 2 x scale; |v| <= 6 x scale)


def test_down_projection_consumes_the_fused_activations(cuda, atlas, oracle):
    """ACT_FP4 | ACT_FP4_READY: the call takes the quantised activations already in `ws` — same bits as quantising them itself —
    and the chain gate/up -> fused SwiGLU+quantise -> down agrees with the chain through a BF16 intermediate."""
    from atlas_b200 import synth, tp as tpmod
    M, inter, hidden = 96, 1024, 512
    case = synth.make_case("down", M=M, K=inter, N=hidden, ranks=[16, 8], max_rank=16, none_frac=0.2, scale2=0.02, b_std=0.1, seed=8)
    g = synth.f32_to_bf16_bits(synth.normal(5, M * inter, 2.0)).reshape(M, inter)
    u = synth.f32_to_bf16_bits(synth.normal(6, M * inter, 2.0)).reshape(M, inter)
    gd, ud = to_dev(cuda, g), to_dev(cuda, u)
    sh = tpmod.DeviceShard(cuda, atlas, case, 1, 0)
    # through BF16: h = SwiGLU(g, u) becomes the call's x, the call quantises it
    atlas.silu_mul(gd, ud, sh.x, M, inter)
    y_a = cuda.empty((M, hidden), dtype=cuda.bfloat16, device="cuda")
    d = sh.desc(y_a, extra_flags=atlas.FLAG_ACT_FP4 | atlas.FLAG_FORCE_TCGEN05)
    atlas.nvfp4_lora_linear(d)
    # the same call again with READY: the quantiser is skipped, ws is reused as it stands
    y_b = cuda.empty((M, hidden), dtype=cuda.bfloat16, device="cuda")
    d_ready = sh.desc(y_b, extra_flags=atlas.FLAG_ACT_FP4 | atlas.FLAG_ACT_FP4_READY | atlas.FLAG_FORCE_TCGEN05)
    sh.x.zero_()                                                          # proves the base product no longer reads x ...
    atlas.silu_mul(gd, ud, sh.x, M, inter)                                # ... (the LoRA shrink still does: put it back)
    atlas.nvfp4_lora_linear(d_ready)
    cuda.cuda.synchronize()
    assert np.array_equal(bits_from_dev(y_a.view(cuda.int16)), bits_from_dev(y_b.view(cuda.int16)))
    # fused: activations quantised from the FP32 product, no BF16 h for the base product
    atlas.silu_mul_quant_nvfp4(gd, ud, sh._ws, atlas.act_fp4_ws_bytes(M, inter), M, inter)
    y_c = cuda.empty((M, hidden), dtype=cuda.bfloat16, device="cuda")
    atlas.nvfp4_lora_linear(sh.desc(y_c, extra_flags=atlas.FLAG_ACT_FP4 | atlas.FLAG_ACT_FP4_READY | atlas.FLAG_FORCE_TCGEN05))
    cuda.cuda.synchronize()
    a, c = oracle.bf16_to_f32(bits_from_dev(y_a.view(cuda.int16))), oracle.bf16_to_f32(bits_from_dev(y_c.view(cuda.int16)))
    # Quantising the FP32 product instead of its BF16 rounding (which moves a value by up to 2^-9 of itself) flips the
    # code of the roughly 1 % of values that sit that close to a bin edge, each by a whole step (a quarter to a third of
    # the value): an L2 difference of sqrt(0.01) x 0.3 = 3 % between the two activation tensors and hence between the
    # outputs, far inside the quantisation noise of the mode itself.  (What the fused kernel writes is pinned code by
    # code in test_silu_mul_quant_matches_the_quantiser_on_fp32_values.)
    assert np.abs(a - c).max() <= 0.15 * np.abs(a).max() and np.mean(np.abs(a - c)) <= 5e-2 * np.abs(a).mean()
    assert atlas.device_status() == 0
