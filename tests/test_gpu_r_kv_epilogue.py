"""The K/V consumer of the fused QKV projection (per-head RMS norm with (1 + w), rotary embedding, one rounding, paged
cache write; V copied into its paged cache): bit for bit against the reference's own kernel
(kernels/gb10/common/fused_k_norm_rope_cache.cu, compiled unchanged for sm_100a) on a contiguous K, the same bits when K
and V are read in place from a strided fused QKV buffer, and against the CPU oracle to the last BF16 bit or one next to
it (the oracle's 1/sqrtf, sinf and cosf are the host library's, the device's are its own)."""
import numpy as np
import pytest

from gpu_util import RefModule, bits_from_dev, to_dev

pytestmark = pytest.mark.gpu

FILL = 0x7FC0


def _inputs(oracle, tokens, kv_heads, head_dim, seed):
    rng = np.random.default_rng(seed)
    k = oracle.f32_to_bf16((rng.standard_normal((tokens, kv_heads * head_dim)) * rng.uniform(0.1, 18.0, (tokens, 1))).astype(np.float32))
    v = oracle.f32_to_bf16(rng.standard_normal((tokens, kv_heads * head_dim)).astype(np.float32))
    w = oracle.f32_to_bf16((rng.standard_normal(head_dim) * 0.1).astype(np.float32))
    pos = rng.integers(0, 131072, tokens).astype(np.uint32)
    n_slots = tokens + 37
    slots = rng.permutation(n_slots)[:tokens].astype(np.int64)
    slots[rng.random(tokens) < 0.1] = -1                        # padding tokens
    return k, v, w, pos, slots, n_slots


@pytest.mark.parametrize("head_dim,rotary_dim", [(128, 64), (128, 128), (256, 64), (64, 0)])
def test_k_norm_rope_cache_write(cuda, atlas, oracle, head_dim, rotary_dim):
    torch = cuda
    tokens, kv_heads, block_size, eps, theta = 301, 4, 16, 1e-6, 1.0e7
    k, v, w, pos, slots, n_slots = _inputs(oracle, tokens, kv_heads, head_dim, head_dim + rotary_dim)
    n_blocks = (n_slots + block_size - 1) // block_size
    width = kv_heads * head_dim
    kd, vd, wd = to_dev(torch, k), to_dev(torch, v), to_dev(torch, w)
    posd, slotd = to_dev(torch, pos), torch.from_numpy(slots).cuda()

    def cache():
        return torch.full((n_blocks, block_size, kv_heads, head_dim), np.int16(np.uint16(FILL).view(np.int16)), dtype=torch.int16, device="cuda")

    # this library, K and V contiguous
    kc, vc = cache(), cache()
    atlas.kv_norm_rope_cache_write(kd, vd, width, wd, posd, slotd, kc, vc, tokens, kv_heads, head_dim, rotary_dim, block_size, eps, theta)
    torch.cuda.synchronize()
    got_k, got_v = bits_from_dev(kc), bits_from_dev(vc)
    live = slots >= 0
    blk, off = slots[live] // block_size, slots[live] % block_size
    assert np.array_equal(got_v[blk, off].reshape(-1, width), v[live])                 # V: a plain copy
    untouched = np.ones((n_blocks, block_size), dtype=bool)
    untouched[blk, off] = False
    assert (got_k[untouched] == FILL).all() and (got_v[untouched] == FILL).all()       # nothing else written

    # the reference's kernel on the same contiguous K (rotary_dim = 0 is not a case it is launched with)
    if rotary_dim:
        ref = RefModule("fused_k_norm_rope_cache")
        kc_ref = cache()
        ref.launch("fused_k_norm_rope_cache_write_bf16", (tokens, kv_heads, 1), (head_dim, 1, 1),
                   [kd.data_ptr(), wd.data_ptr(), posd.data_ptr(), kc_ref.data_ptr(), slotd.data_ptr(),
                    ("u32", kv_heads), ("u32", head_dim), ("u32", rotary_dim), ("u32", block_size), float(eps), float(theta)])
        torch.cuda.synchronize()
        assert np.array_equal(got_k, bits_from_dev(kc_ref))                            # same bits as the reference

    # K and V read in place from a fused QKV buffer: [tokens, q | k | v | pad]
    q_w, pad = 3 * width, 24
    stride = q_w + 2 * width + pad
    qkv = torch.zeros((tokens, stride), dtype=torch.int16, device="cuda")
    qkv[:, q_w:q_w + width].copy_(kd)
    qkv[:, q_w + width:q_w + 2 * width].copy_(vd)
    kc2, vc2 = cache(), cache()
    atlas.kv_norm_rope_cache_write(qkv.data_ptr() + q_w * 2, qkv.data_ptr() + (q_w + width) * 2, stride, wd, posd, slotd, kc2, vc2,
                                   tokens, kv_heads, head_dim, rotary_dim, block_size, eps, theta)
    torch.cuda.synchronize()
    assert np.array_equal(bits_from_dev(kc2), got_k) and np.array_equal(bits_from_dev(vc2), got_v)

    # the CPU oracle: equal, or next to it in the last BF16 bit
    want = np.full((n_blocks, block_size, kv_heads, head_dim), FILL, dtype=np.uint16)
    oracle.k_norm_rope_cache_write(k, width, w, pos, slots, want, kv_heads, head_dim, rotary_dim, block_size, eps, theta)
    a, b = got_k[blk, off].astype(np.int32), want[blk, off].astype(np.int32)
    assert np.abs(a - b).max() <= 1
    assert (a != b).mean() < 0.02


def test_shapes_the_kernel_does_not_take_are_refused(cuda, atlas):
    torch = cuda
    z = torch.zeros(4096, dtype=torch.int16, device="cuda")
    pos = torch.zeros(4, dtype=torch.int32, device="cuda")
    slot = torch.zeros(4, dtype=torch.int64, device="cuda")
    for head_dim, rotary in ((48, 0), (128, 32), (512, 64), (128, 192)):
        with pytest.raises(atlas.AtlasError) as e:
            atlas.kv_norm_rope_cache_write(z, None, 1024, z, pos, slot, z, None, 4, 1, head_dim, rotary, 16, 1e-6, 1e4)
        assert e.value.status == -1


@pytest.mark.parametrize("head_dim,rotary_dim,offset_one,factor", [(128, 64, True, 1.0), (128, 128, False, 1.18), (256, 64, True, 1.0), (64, 32, True, 0.9), (192, 64, True, 1.0), (64, 64, False, 1.0)])
def test_decode_qkv_norm_rope_cache_write(cuda, atlas, oracle, head_dim, rotary_dim, offset_one, factor):
    """Q in place, K into the paged cache, V copied — against the reference's fused decode kernel
    (kernels/gb10/common/fused_verify_elemwise.cu) bit for bit, in place on a strided fused QKV buffer, and against the
    oracle."""
    torch = cuda
    tokens, q_heads, kv_heads, block_size, eps = 37, 6, 2, 16, 1e-6
    k, v, wk, pos, slots, n_slots = _inputs(oracle, tokens, kv_heads, head_dim, 7 * head_dim + rotary_dim)
    rng = np.random.default_rng(head_dim)
    q = oracle.f32_to_bf16((rng.standard_normal((tokens, q_heads * head_dim)) * 4).astype(np.float32))
    wq = oracle.f32_to_bf16((rng.standard_normal(head_dim) * (0.1 if offset_one else 1.0)).astype(np.float32))
    if not offset_one:
        wk = oracle.f32_to_bf16((rng.standard_normal(head_dim) + 1.0).astype(np.float32))
    inv_freq = (1.0e6 ** (-2.0 * np.arange(rotary_dim // 2) / rotary_dim)).astype(np.float32)
    n_blocks = (n_slots + block_size - 1) // block_size
    qw, kw = q_heads * head_dim, kv_heads * head_dim
    wqd, wkd, posd, slotd, fd = to_dev(torch, wq), to_dev(torch, wk), to_dev(torch, pos), torch.from_numpy(slots).cuda(), torch.from_numpy(inv_freq).cuda()

    def cache():
        return torch.full((n_blocks, block_size, kv_heads, head_dim), np.int16(np.uint16(FILL).view(np.int16)), dtype=torch.int16, device="cuda")

    # the reference's kernel, contiguous q / k / v
    ref = RefModule("fused_verify_elemwise")
    q_ref, kd, vd = to_dev(torch, q), to_dev(torch, k), to_dev(torch, v)
    kc_ref, vc_ref = cache(), cache()
    ref.launch("fused_qkv_norm_rope_cache_write_bf16", (q_heads + 2 * kv_heads, tokens, 1), (head_dim, 1, 1),
               [q_ref.data_ptr(), kd.data_ptr(), vd.data_ptr(), wqd.data_ptr(), wkd.data_ptr(), posd.data_ptr(), fd.data_ptr(),
                kc_ref.data_ptr(), vc_ref.data_ptr(), slotd.data_ptr(), ("u32", q_heads), ("u32", kv_heads), ("u32", head_dim),
                ("u32", rotary_dim), ("u32", block_size), float(eps), float(factor), ("u32", 1 if offset_one else 0)])
    torch.cuda.synchronize()

    # this library, in place on the fused buffer [tokens, q | k | v | pad]
    stride = qw + 2 * kw + 40
    qkv = torch.zeros((tokens, stride), dtype=torch.int16, device="cuda")
    qkv[:, :qw].copy_(to_dev(torch, q)); qkv[:, qw:qw + kw].copy_(kd); qkv[:, qw + kw:qw + 2 * kw].copy_(vd)
    kc, vc = cache(), cache()
    atlas.qkv_norm_rope_cache_write(qkv.data_ptr(), qkv.data_ptr() + qw * 2, qkv.data_ptr() + (qw + kw) * 2, stride, stride, wqd, wkd, posd, fd,
                                    slotd, kc, vc, tokens, q_heads, kv_heads, head_dim, rotary_dim, block_size, eps, factor, offset_one)
    torch.cuda.synchronize()
    got = bits_from_dev(qkv)
    assert np.array_equal(got[:, :qw], bits_from_dev(q_ref))                            # Q: same bits as the reference
    assert np.array_equal(bits_from_dev(kc), bits_from_dev(kc_ref))                     # K cache: same bits
    assert np.array_equal(bits_from_dev(vc), bits_from_dev(vc_ref))
    assert np.array_equal(got[:, qw:qw + 2 * kw], np.concatenate([k, v], axis=1))       # K and V inputs untouched
    assert (got[:, qw + 2 * kw:] == 0).all()

    # the oracle: equal, or a BF16 step or two away where its host-library rsqrt / sin / cos round the other way
    q_o = q.copy()
    kc_o = np.full((n_blocks, block_size, kv_heads, head_dim), FILL, dtype=np.uint16)
    vc_o = kc_o.copy()
    oracle.qkv_norm_rope_cache_write(q_o, qw, k, v, kw, wq, wk, pos, inv_freq, slots, kc_o, vc_o, q_heads, kv_heads, head_dim, rotary_dim,
                                     block_size, eps, factor, offset_one)
    assert np.array_equal(vc_o, bits_from_dev(vc))
    for a, b in ((got[:, :qw], q_o), (bits_from_dev(kc), kc_o)):
        fa, fb = oracle.bf16_to_f32(np.ascontiguousarray(a)), oracle.bf16_to_f32(np.ascontiguousarray(b))
        live = np.isfinite(fb)
        assert np.array_equal(np.isfinite(fa), live)
        assert np.abs(fa[live] - fb[live]).max() <= 2.0 ** -6 * np.abs(fb[live]).max()
        assert (a != b).mean() < 0.02


def test_k_norm_mrope_cache_write(cuda, atlas, oracle):
    """Three position streams (MRoPE): rotary pair p takes the temporal, height or width position for p mod 3 = 0, 1, 2 —
    bit for bit the reference's `fused_k_norm_rope_mrope_cache_write_bf16`; with equal streams, the scalar-position result."""
    torch = cuda
    tokens, kv_heads, head_dim, rotary_dim, block_size, eps, theta = 203, 2, 128, 64, 16, 1e-6, 1.0e7
    k, v, w, pos, slots, n_slots = _inputs(oracle, tokens, kv_heads, head_dim, 99)
    rng = np.random.default_rng(3)
    pos_h, pos_w = rng.integers(0, 4096, tokens).astype(np.uint32), rng.integers(0, 4096, tokens).astype(np.uint32)
    n_blocks = (n_slots + block_size - 1) // block_size
    width = kv_heads * head_dim
    kd, wd, slotd = to_dev(torch, k), to_dev(torch, w), torch.from_numpy(slots).cuda()
    pt, ph, pw = to_dev(torch, pos), to_dev(torch, pos_h), to_dev(torch, pos_w)

    def cache():
        return torch.full((n_blocks, block_size, kv_heads, head_dim), np.int16(np.uint16(FILL).view(np.int16)), dtype=torch.int16, device="cuda")
    kc, kc_ref, kc_same, kc_scalar = cache(), cache(), cache(), cache()
    atlas.kv_norm_rope_cache_write(kd, None, width, wd, pt, slotd, kc, None, tokens, kv_heads, head_dim, rotary_dim, block_size, eps, theta,
                                   positions_h=ph, positions_w=pw)
    RefModule("fused_k_norm_rope_cache").launch(
        "fused_k_norm_rope_mrope_cache_write_bf16", (tokens, kv_heads, 1), (head_dim, 1, 1),
        [kd.data_ptr(), wd.data_ptr(), pt.data_ptr(), ph.data_ptr(), pw.data_ptr(), kc_ref.data_ptr(), slotd.data_ptr(),
         ("u32", kv_heads), ("u32", head_dim), ("u32", rotary_dim), ("u32", block_size), float(eps), float(theta)])
    atlas.kv_norm_rope_cache_write(kd, None, width, wd, pt, slotd, kc_same, None, tokens, kv_heads, head_dim, rotary_dim, block_size, eps, theta,
                                   positions_h=pt, positions_w=pt)
    atlas.kv_norm_rope_cache_write(kd, None, width, wd, pt, slotd, kc_scalar, None, tokens, kv_heads, head_dim, rotary_dim, block_size, eps, theta)
    torch.cuda.synchronize()
    assert np.array_equal(bits_from_dev(kc), bits_from_dev(kc_ref))
    assert np.array_equal(bits_from_dev(kc_same), bits_from_dev(kc_scalar))
    assert not np.array_equal(bits_from_dev(kc), bits_from_dev(kc_scalar))


def test_k_norm_rope_cache_write_fp8(cuda, atlas, oracle):
    """The K side into an E4M3 paged cache: bit for bit the reference's `fused_k_norm_rope_cache_write_fp8`, values beyond the
    format's range saturating at +-448."""
    torch = cuda
    tokens, kv_heads, head_dim, rotary_dim, block_size, eps, theta, inv_scale = 157, 2, 128, 64, 16, 1e-6, 1.0e6, 200.0
    k, v, w, pos, slots, n_slots = _inputs(oracle, tokens, kv_heads, head_dim, 5)
    n_blocks = (n_slots + block_size - 1) // block_size
    width = kv_heads * head_dim
    kd, wd, posd, slotd = to_dev(torch, k), to_dev(torch, w), to_dev(torch, pos), torch.from_numpy(slots).cuda()
    c8, c8_ref = [torch.full((n_blocks, block_size, kv_heads, head_dim), 0x55, dtype=torch.uint8, device="cuda") for _ in range(2)]
    atlas.k_norm_rope_cache_write_fp8(kd, width, wd, posd, slotd, c8, tokens, kv_heads, head_dim, rotary_dim, block_size, eps, theta, inv_scale)
    RefModule("fused_k_norm_rope_cache").launch(
        "fused_k_norm_rope_cache_write_fp8", (tokens, kv_heads, 1), (head_dim, 1, 1),
        [kd.data_ptr(), wd.data_ptr(), posd.data_ptr(), c8_ref.data_ptr(), slotd.data_ptr(), ("u32", kv_heads), ("u32", head_dim),
         ("u32", rotary_dim), ("u32", block_size), float(eps), float(theta), float(inv_scale)])
    torch.cuda.synchronize()
    got, ref = c8.cpu().numpy(), c8_ref.cpu().numpy()
    assert np.array_equal(got, ref)
    live = slots >= 0
    written = got[slots[live] // block_size, slots[live] % block_size]
    assert ((written & 0x7F) == 0x7E).any()                 # normed magnitudes reach 3-4, times 200: some saturate at 448
    assert not ((written & 0x7F) == 0x7F).any()             # and none becomes the NaN byte
