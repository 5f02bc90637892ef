"""The FP4-activation (W4A4) mode of the fused layer: block-scaled FP4 x FP4 MMA against the oracle's act_fp4 mode.

The mode mirrors the reference's opt-in W4A4 arm (crates/spark-model/src/layers/ops/gemm_fp4.rs:20-107): x is
quantised to NVFP4 with a tensor scale of one by the quantiser of kernels/gb10/common/quantize_bf16_to_nvfp4.cu,
the base product runs on the quantised values, the LoRA term on the exact ones."""
import numpy as np
import pytest

from gpu_util import DeviceCase, assert_close, ideal

pytestmark = pytest.mark.gpu


def _a4(atlas):
    return atlas.FLAG_FORCE_TCGEN05 | atlas.FLAG_ACT_FP4


def _ws_parts(dc, M, K):
    ws = dc.ws.cpu().numpy()
    codes_bytes = (M * (K // 2) + 255) // 256 * 256
    return ws[:M * (K // 2)].reshape(M, K // 2), ws[codes_bytes:codes_bytes + M * (K // 16)].reshape(M, K // 16)


@pytest.mark.parametrize("M,stride", [(48, None), (256, 1032)])
def test_activation_quantiser_is_bit_exact(cuda, atlas, oracle, M, stride):
    from atlas_b200 import synth
    K, N = 512, 128
    case = synth.make_case("aq", M=M, K=K, N=N, ranks=[8], max_rank=8, seed=5 + M)
    case.x[0, :16] = 0                                   # an all-zero group: scale byte 0, codes 0
    case.x[1, 16:32] = oracle.f32_to_bf16(np.full(16, 3000.0, np.float32))   # scale saturates at 448
    dc = DeviceCase(cuda, atlas, case, x_row_stride=stride)
    _, variant = dc.run(lora=False, flags=_a4(atlas))
    assert variant == atlas.VARIANT_TCGEN05
    codes, scales = _ws_parts(dc, M, K)
    want_codes, want_scales = oracle.quantize_bf16_to_nvfp4(case.x, 1.0, M, K)
    assert np.array_equal(scales, want_scales.reshape(M, K // 16))
    assert np.array_equal(codes, want_codes.reshape(M, K // 2))


@pytest.mark.parametrize("M", [256, 128, 64, 16])
def test_decode_through_the_block_scaled_mma_is_bit_exact(cuda, atlas, oracle, M):
    """One activation of +-6 per token (quantises to code 6/14 with scale byte 1.0, i.e. exactly): y[m, f] =
    +-6 w[f, k_m], a single product, so the tensor core's E2M1 x UE4M3 decode, the nibble order and the placement
    of every scale byte (normal and subnormal) are compared bit for bit with the oracle's decode."""
    from atlas_b200 import synth
    K, N = 512, 256
    packed, scales = synth.make_nvfp4_weight(77, N, K)
    scales[:, 0] = np.arange(N, dtype=np.uint8) % 0x7F
    scales[:, 17] = (np.arange(N, dtype=np.uint8) * 5 + 3) % 0x7F
    packed[0, :8] = np.arange(8, dtype=np.uint8) | ((np.arange(8, dtype=np.uint8) + 8) << 4)
    k_of = (np.arange(M) * 37 + 5) % K
    sign = np.where(np.arange(M) % 2 == 0, 6.0, -6.0).astype(np.float32)
    x = np.zeros((M, K), dtype=np.float32)
    x[np.arange(M), k_of] = sign
    case = synth.Case("onehot4", M, K, N, 8, 1, oracle.f32_to_bf16(x), np.full(M, -1, np.int32), [None],
                      packed=packed, scales=scales, scale2=1.0)
    y, variant = DeviceCase(cuda, atlas, case).run(lora=False, flags=_a4(atlas))
    assert variant == atlas.VARIANT_TCGEN05
    w = oracle.dequant_nvfp4_to_f32(packed, scales, 1.0, N, K)            # [N, K]
    want = oracle.f32_to_bf16(np.ascontiguousarray(w[:, k_of].T * sign[:, None]))
    want = np.where(want == 0x8000, 0, want)                              # a sum of signed zeros is +0
    assert np.array_equal(np.where(y == 0x8000, 0, y), want)
    assert atlas.device_status() == 0


@pytest.mark.parametrize("M,K,N", [(16, 256, 128), (40, 512, 200), (64, 1024, 384), (100, 768, 256),
                                   (256, 512, 128), (300, 256, 264), (1, 256, 128), (200, 2560, 512)])
def test_base_linear(cuda, atlas, oracle, M, K, N):
    from atlas_b200 import synth
    case = synth.make_case("base4", M=M, K=K, N=N, ranks=[8], max_rank=8, scale2=0.02, seed=M + K)
    dc = DeviceCase(cuda, atlas, case, out_row_stride=N + 8)
    y, variant = dc.run(lora=False, flags=_a4(atlas))
    assert variant == atlas.VARIANT_TCGEN05
    want = ideal(oracle, case, lora=False, act_fp4=True)
    assert_close(oracle, y[:, :N], want, "base, FP4 activations")
    assert (y[:, N:] == 0x7FC0).all()
    # the mode is really in effect: the exact-activation result differs visibly from it
    exact = ideal(oracle, case, lora=False)
    assert np.abs(exact - want).mean() > 10 * np.abs(oracle.bf16_to_f32(y[:, :N]) - want).mean()
    assert atlas.device_status() == 0


@pytest.mark.parametrize("M,K,N,ranks,max_rank", [
    (64, 512, 256, [8, 16, 32, 64] * 8, 64),
    (300, 512, 384, [32] * 16, 32),
    (130, 256, 200, [8, 24], 24),
])
def test_fused_lora(cuda, atlas, oracle, M, K, N, ranks, max_rank):
    from atlas_b200 import synth
    case = synth.make_case("fused4", M=M, K=K, N=N, ranks=ranks, max_rank=max_rank, max_loras=len(ranks) + 3,
                           none_frac=0.15, scale2=0.02, b_std=0.1, seed=M + N)
    dc = DeviceCase(cuda, atlas, case)
    y, variant = dc.run(flags=_a4(atlas))
    assert variant == atlas.VARIANT_TCGEN05
    want = ideal(oracle, case, act_fp4=True)
    assert_close(oracle, y, want, "fused, FP4 activations")
    yb, _ = dc.run(lora=False, flags=_a4(atlas))
    none = case.seq_slot < 0
    assert none.any() and np.array_equal(y[none], yb[none])            # routing is exact
    base = ideal(oracle, case, lora=False, act_fp4=True)
    got = oracle.bf16_to_f32(y)
    num = ((got - base)[~none] * (want - base)[~none]).sum()
    den = np.linalg.norm((got - base)[~none]) * np.linalg.norm((want - base)[~none])
    assert num / den > 0.99
    assert atlas.device_status() == 0


def test_argument_errors(cuda, atlas, oracle):
    from atlas_b200 import synth
    case = synth.make_case("err4", M=32, K=512, N=128, ranks=[8], max_rank=8, seed=3)
    dc = DeviceCase(cuda, atlas, case)
    y = cuda.zeros((32, 128), dtype=cuda.int16, device="cuda")
    kw = dict(x=dc.x, m=32, k=512, n=128, y=y, w_packed=dc.packed, w_scale=dc.scales, scale2=1.0)
    ws = cuda.zeros(atlas.act_fp4_ws_bytes(32, 512), dtype=cuda.uint8, device="cuda")
    with pytest.raises(atlas.AtlasError) as e:
        atlas.nvfp4_lora_linear(atlas.make_linear_desc(flags=atlas.FLAG_ACT_FP4, **kw))
    assert e.value.status == -4                                          # no scratch
    with pytest.raises(atlas.AtlasError) as e:
        atlas.nvfp4_lora_linear(atlas.make_linear_desc(flags=atlas.FLAG_ACT_FP4, ws=ws, ws_bytes=ws.numel() - 1, **kw))
    assert e.value.status == -2                                          # scratch too small
    with pytest.raises(atlas.AtlasError) as e:
        atlas.nvfp4_lora_linear(atlas.make_linear_desc(flags=atlas.FLAG_ACT_FP4 | atlas.FLAG_FORCE_SIMT, ws=ws,
                                                       ws_bytes=ws.numel(), **kw))
    assert e.value.status == -1                                          # no CUDA-core form of this mode
    kw["k"] = 496                                                         # not a shape the tensor-core path takes
    with pytest.raises(atlas.AtlasError) as e:
        atlas.nvfp4_lora_linear(atlas.make_linear_desc(flags=atlas.FLAG_ACT_FP4, ws=ws, ws_bytes=ws.numel(), **kw))
    assert e.value.status == -1
    cuda.cuda.synchronize()


def test_signed_weight_scale_is_reported(cuda, atlas, oracle):
    """The tensor core reads unsigned scale bytes; a sign bit is dropped and the status word says so."""
    from atlas_b200 import synth
    case = synth.make_case("neg4", M=16, K=256, N=128, ranks=[8], max_rank=8, scale2=0.02, seed=9)
    case.scales[5, 3] |= 0x80
    dc = DeviceCase(cuda, atlas, case)
    y, _ = dc.run(lora=False, flags=_a4(atlas))
    assert atlas.device_status() == 2
    case.scales[5, 3] &= 0x7F
    assert_close(oracle, y, ideal(oracle, case, lora=False, act_fp4=True), "sign dropped")
    assert atlas.device_status() == 0

