"""The oracle against every golden value the reference's own sources and tests hold for this path."""
import json
import math
import os
import struct

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _bits(f):
    return struct.unpack("<I", struct.pack("<f", f))[0]


def test_e2m1_table_matches_reference_source(oracle):
    gold = [float(v) for v in json.load(open(os.path.join(GOLD, "e2m1_lut.json")))]
    got = oracle.e2m1_decode_table()
    for i in range(16):
        assert _bits(float(got[i])) == _bits(gold[i]), i       # bit compare keeps -0.0
    # spark-model/examples/w4a16_bf16_microtest.rs:320
    assert got[7] == 6.0
    # spark-runtime/src/cutlass/tests/mod.rs:156-161
    assert list(got[:8]) == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def test_e4m3_table_matches_reference_source(oracle):
    gold = [float(v) for v in json.load(open(os.path.join(GOLD, "e4m3_lut.json")))]
    got = oracle.e4m3_decode_table()
    for i in range(256):
        assert _bits(float(got[i])) == _bits(gold[i]), hex(i)
    assert got[0x7F] == 0.0 and got[0xFF] == 0.0           # NaN byte decodes to zero
    assert got[0x7E] == 448.0
    # e4m3 byte of 1.0 decodes to 1.0 (w4a16_bf16_microtest.rs:321)
    assert got[oracle.lib().orc_e4m3_encode(1.0)] == 1.0


def test_e4m3_encode_roundtrip_and_saturation(oracle):
    L = oracle.lib()
    tab = oracle.e4m3_decode_table()
    for b in range(0x7F):                                   # every finite positive byte is a fixed point
        assert L.orc_e4m3_encode(float(tab[b])) == b
    assert L.orc_e4m3_encode(1e9) == 0x7E                   # saturate at 448
    assert L.orc_e4m3_encode(0.0) == 0
    assert L.orc_e4m3_encode(2.0 ** -12) == 0               # below half the smallest subnormal
    # half-up mantissa rounding with carry: 1.9375 = 1 + 7.5/8 -> 2.0
    assert tab[L.orc_e4m3_encode(1.9375)] == 2.0


def test_e2m1_quantiser_bins(oracle):
    L = oracle.lib()
    # kernels/gb10/common/quantize_bf16_to_nvfp4.cu:109-124: ties go to the smaller magnitude
    edges = [(0.25, 0), (0.2500001, 1), (0.75, 1), (0.76, 2), (1.25, 2), (1.26, 3), (1.75, 3), (1.76, 4),
             (2.5, 4), (2.51, 5), (3.5, 5), (3.51, 6), (5.0, 6), (5.01, 7), (100.0, 7)]
    for v, idx in edges:
        assert L.orc_e2m1_quantize(v) == idx
        assert L.orc_e2m1_quantize(-v) == (8 | idx)
    assert L.orc_e2m1_quantize(0.0) == 0


def test_bf16_rne(oracle):
    L = oracle.lib()
    assert L.orc_f32_to_bf16(1.0) == 0x3F80
    # 1 + 2^-8 is exactly half way between 0x3F80 and 0x3F81: ties to even
    assert L.orc_f32_to_bf16(1.00390625) == 0x3F80
    assert L.orc_f32_to_bf16(1.01171875) == 0x3F82         # 1 + 3*2^-8: tie, rounds to even 0x3F82
    assert L.orc_f32_to_bf16(struct.unpack("<f", struct.pack("<I", 0x3F808001))[0]) == 0x3F81
    nan = L.orc_f32_to_bf16(float("nan"))
    assert (nan & 0x7F80) == 0x7F80 and (nan & 0x0040)
    rng = np.random.default_rng(0)
    a = rng.standard_normal(4096).astype(np.float32)
    vec = oracle.f32_to_bf16(a)
    for i in range(0, 4096, 97):
        assert vec[i] == L.orc_f32_to_bf16(float(a[i]))
    # agrees with torch's conversion (the reference states its helper matches __float2bfloat16)
    import torch
    tb = torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(vec, tb)


def test_splitmix64_and_uniform(oracle):
    import ctypes as C
    L = oracle.lib()
    s = C.c_uint64(0)
    # published SplitMix64 outputs for seed 0
    assert L.orc_splitmix64_next(C.byref(s)) == 0xE220A8397B1DCDAF
    assert L.orc_splitmix64_next(C.byref(s)) == 0x6E789E6AA1B965F4
    s = C.c_uint64(0x51A7)
    u = [L.orc_rng_uniform(C.byref(s), -1.0, 1.0) for _ in range(1000)]
    assert all(-1.0 <= v < 1.0 for v in u) and abs(sum(u) / 1000) < 0.1
    from atlas_b200 import synth
    z = synth.splitmix64(0, 2)
    assert int(z[0]) == 0xE220A8397B1DCDAF and int(z[1]) == 0x6E789E6AA1B965F4


def test_build_seq_slot_vectors(oracle):
    # spark-model/src/lora/slot_math_tests.rs:116-158
    assert oracle.build_seq_slot_host([1, -1, 0], 4, 2) == [1, 2, 0, -1]
    assert oracle.build_seq_slot_host([-1, -1, -1, -1], 4, 0) == [0, 0, 0, 0]
    assert oracle.build_seq_slot_host([3, 1], 2, 0) == [3, 1]
    for count in (1, 4, 32):
        assert oracle.build_seq_slot_host([3] * count, count, 7) == [3] * count
        assert oracle.build_seq_slot_host([-1] * count, count, 5) == [5] * count
        assert oracle.build_seq_slot_host([0] * count, count, 2) == [0] * count


def test_routed_prefill_slot_of(oracle):
    L = oracle.lib()
    assert L.orc_routed_prefill_slot_of(1, 0, 4) == 1
    assert L.orc_routed_prefill_slot_of(-1, 0, 4) == -1     # defers to active -> None
    assert L.orc_routed_prefill_slot_of(0, 0, 4) == -1      # names the active slot -> None
    assert L.orc_routed_prefill_slot_of(9, 0, 4) == -1      # out of range -> None


def test_peft_scaling(oracle):
    L = oracle.lib()
    # atlas-core/src/config/parsers/lora_tests.rs:27-43
    assert L.orc_peft_scaling(32.0, 16, 0) == 2.0
    assert L.orc_peft_scaling(32.0, 16, 1) == 8.0
    # spark-model/src/lora/slot_math_tests.rs:87-113
    assert L.orc_peft_scaling(16.0, 8, 0) == np.float32(16.0 / 8.0)
    assert L.orc_peft_scaling(16.0, 4, 1) == np.float32(16.0 / math.sqrt(4.0))


def _factory_cfg(oracle):
    # the reference's test config (atlas-core/src/config/factory.rs:12-43): 48 layers, every 4th full attention
    return oracle.ModelDims(2048, 5120, 16, 2, 256, 1, 12)


def test_pool_slot_bytes_golden(oracle):
    import ctypes as C
    L = oracle.lib()
    cfg = _factory_cfg(oracle)
    assert L.orc_pool_slot_bytes(C.byref(cfg), 16) == 16_515_072       # slot_math_tests.rs:25-34
    # offsets walk fills exactly one slot (slot_math_tests.rs:37-63)
    off = 0
    for layer in range(12):
        for m in range(7):
            o, i = C.c_size_t(), C.c_size_t()
            L.orc_module_dims(C.byref(cfg), m, C.byref(o), C.byref(i))
            a, b = C.c_size_t(), C.c_size_t()
            assert L.orc_module_slot_offsets(C.byref(cfg), 16, layer, m, C.byref(a), C.byref(b)) == 1
            assert (a.value, b.value) == (off, off + 16 * i.value * 2)
            off = b.value + o.value * 16 * 2
    assert off == 16_515_072
    a, b = C.c_size_t(), C.c_size_t()
    assert L.orc_module_slot_offsets(C.byref(cfg), 16, 12, 0, C.byref(a), C.byref(b)) == 0


def test_nvfp4_dequant_and_quantise_roundtrip(oracle):
    from atlas_b200 import synth
    N, K = 8, 64
    packed, scales = synth.make_nvfp4_weight(3, N, K)
    w = oracle.dequant_nvfp4_to_f32(packed, scales, 1.0, N, K)
    e2 = oracle.e2m1_decode_table()
    e4 = oracle.e4m3_decode_table()
    # element (n, k): low nibble of byte k/2 for even k
    for n, k in [(0, 0), (0, 1), (3, 17), (7, 63), (5, 32)]:
        byte = packed[n, k // 2]
        nib = (byte >> 4) if (k & 1) else (byte & 0xF)
        assert w[n, k] == e2[nib] * e4[scales[n, k // 16]]
    wb = oracle.dequant_nvfp4_to_bf16(packed, scales, 1.0, N, K)
    assert np.array_equal(oracle.bf16_to_f32(wb), w)                   # E2M1 x E4M3 is exact in BF16
    # quantising an exactly representable tensor with the same scale2 reproduces values
    p2, s2 = oracle.quantize_bf16_to_nvfp4(wb, 1.0, N, K)
    w2 = oracle.dequant_nvfp4_to_f32(p2, s2, 1.0, N, K)
    err = np.abs(w2 - w).max() / max(np.abs(w).max(), 1e-9)
    assert err < 0.3


def test_peft_delta_fixture(oracle):
    """delta = scaling * B @ A of the reference's own adapter fixture, via one-hot activations."""
    g = np.load(os.path.join(GOLD, "peft_delta_k_proj.npz"))
    a_bits, b_bits, scaling, r = g["a_bits"], g["b_bits"], float(g["scaling"]), int(g["r"])
    assert scaling == oracle.lib().orc_peft_scaling(float(g["alpha"]), r, int(g["use_rslora"])) == 2.0
    K, N = a_bits.shape[1], b_bits.shape[0]
    max_rank = 16
    pool = oracle.HostPool(K, N, max_rank, 2)
    pool.pack(1, a_bits, b_bits, scaling)
    ncol = g["delta_cols32"].shape[1]
    x = np.zeros((ncol, K), dtype=np.float32)
    x[np.arange(ncol), np.arange(ncol)] = 1.0
    xb = oracle.f32_to_bf16(x)
    w0 = np.zeros((N, K), dtype=np.uint16)
    y = oracle.fused_linear_f32(xb, ncol, N, K, w_bf16=w0, seq_slot=[1] * ncol, pool=pool)
    np.testing.assert_allclose(y.T, g["delta_cols32"], rtol=1e-5, atol=1e-7)


def test_staged_matches_fp32_ideal_within_tolerance(oracle):
    from atlas_b200 import synth
    case = synth.make_case("t", M=12, K=256, N=96, ranks=[8, 16, 4], max_rank=16, none_frac=0.25, scale2=0.01, b_std=0.3, seed=5)
    pool = oracle.HostPool(case.K, case.N, case.max_rank, case.max_loras)
    for s, ad in enumerate(case.adapters):
        if ad:
            pool.pack(s, ad.a, ad.b, ad.scale)
    ideal = oracle.fused_linear_f32(case.x, case.M, case.N, case.K, packed=case.packed, scales=case.scales,
                                    scale2=case.scale2, seq_slot=case.seq_slot, pool=pool)
    y, xa = oracle.reference_sequence(case.x, case.M, case.N, case.K, packed=case.packed, scales=case.scales,
                                      scale2=case.scale2, seq_slot=case.seq_slot, pool=pool)
    yf = oracle.bf16_to_f32(y)
    assert np.all(np.abs(yf - ideal) <= 1e-2 + 2e-2 * np.abs(ideal))
    # un-adapted rows: xa untouched (zero) and output equals the base product alone
    base = oracle.fused_linear_f32(case.x, case.M, case.N, case.K, packed=case.packed, scales=case.scales, scale2=case.scale2)
    for m in range(case.M):
        if case.seq_slot[m] < 0:
            assert not xa[m].any()
            assert np.all(np.abs(yf[m] - base[m]) <= 1e-2 + 2e-2 * np.abs(base[m]))
        else:
            r = case.adapters[case.seq_slot[m]].rank
            assert not xa[m, r:].any()                                  # pad ranks come out zero
    assert np.abs(ideal - base).max() > 0.05                           # the LoRA term is visible in this case


def test_k_norm_rope_cache_write_against_a_float64_formula(oracle):
    """The oracle's K epilogue (RMS norm with (1 + w), rotary pairs (d, d + rotary_dim/2), paged write) against the textbook
    formula in float64: within a BF16 rounding of it, skipped tokens untouched, slots mapped to [block, offset]."""
    rng = np.random.default_rng(5)
    tokens, kv_heads, hd, rot, bs, eps, theta = 9, 2, 128, 64, 4, 1e-6, 1.0e6
    k = oracle.f32_to_bf16(rng.standard_normal((tokens, kv_heads * hd)).astype(np.float32) * 3)
    w = oracle.f32_to_bf16((rng.standard_normal(hd) * 0.1).astype(np.float32))
    pos = rng.integers(0, 5000, tokens).astype(np.uint32)
    slots = np.array([5, 0, -1, 11, 2, 7, -1, 9, 3], dtype=np.int64)
    cache = np.full((3, bs, kv_heads, hd), 0x7FC0, dtype=np.uint16)
    oracle.k_norm_rope_cache_write(k, kv_heads * hd, w, pos, slots, cache, kv_heads, hd, rot, bs, eps, theta)
    kf, wf = oracle.bf16_to_f32(k).astype(np.float64).reshape(tokens, kv_heads, hd), oracle.bf16_to_f32(w).astype(np.float64)
    for t in range(tokens):
        if slots[t] < 0:
            continue
        x = kf[t]
        n = x / np.sqrt((x * x).mean(axis=1, keepdims=True) + eps) * (1.0 + wf)
        out = n.copy()
        half = rot // 2
        ang = pos[t] * theta ** (-2.0 * np.arange(half) / rot)
        out[:, :half] = n[:, :half] * np.cos(ang) - n[:, half:rot] * np.sin(ang)
        out[:, half:rot] = n[:, half:rot] * np.cos(ang) + n[:, :half] * np.sin(ang)
        got = oracle.bf16_to_f32(cache[slots[t] // bs, slots[t] % bs]).astype(np.float64)
        assert np.abs(got - out).max() <= 2.0 ** -7 * np.abs(out).max() + 1e-3
    written = {(int(s) // bs, int(s) % bs) for s in slots if s >= 0}
    for b in range(3):
        for o in range(bs):
            if (b, o) not in written:
                assert (cache[b, o] == 0x7FC0).all()


def test_decode_qkv_epilogue_against_a_float64_formula(oracle):
    """The oracle's decode-path QKV consumer: Q in place, K into the paged cache (normed head rounded to BF16, then rotated
    by position * inv_freq with scaled cosine / sine), V copied — within BF16 roundings of the float64 formula."""
    rng = np.random.default_rng(11)
    tokens, nq, nkv, hd, rot, bs, eps, factor = 5, 3, 2, 64, 32, 4, 1e-6, 1.1
    q = oracle.f32_to_bf16(rng.standard_normal((tokens, nq * hd)).astype(np.float32) * 2)
    k = oracle.f32_to_bf16(rng.standard_normal((tokens, nkv * hd)).astype(np.float32) * 5)
    v = oracle.f32_to_bf16(rng.standard_normal((tokens, nkv * hd)).astype(np.float32))
    wq = oracle.f32_to_bf16((rng.standard_normal(hd) * 0.1).astype(np.float32))
    wk = oracle.f32_to_bf16((rng.standard_normal(hd) * 0.1).astype(np.float32))
    pos = np.array([0, 7, 100, 4095, 31], dtype=np.uint32)
    inv_freq = (1.0e4 ** (-2.0 * np.arange(rot // 2) / rot)).astype(np.float32)
    slots = np.array([2, -1, 0, 5, 7], dtype=np.int64)
    kc = np.full((2, bs, nkv, hd), 0x7FC0, dtype=np.uint16)
    vc = kc.copy()
    q_out = q.copy()
    oracle.qkv_norm_rope_cache_write(q_out, nq * hd, k, v, nkv * hd, wq, wk, pos, inv_freq, slots, kc, vc, nq, nkv, hd, rot, bs, eps, factor, True)

    def chain(x, w, p):
        x = x.astype(np.float64)
        n = x / np.sqrt((x * x).mean() + eps) * (1.0 + w.astype(np.float64))
        out = n.copy()
        h = rot // 2
        ang = p * inv_freq.astype(np.float64)
        c, s = np.cos(ang) * factor, np.sin(ang) * factor
        out[:h] = n[:h] * c - n[h:rot] * s
        out[h:rot] = n[h:rot] * c + n[:h] * s
        return out
    qf, kf = oracle.bf16_to_f32(q).reshape(tokens, nq, hd), oracle.bf16_to_f32(k).reshape(tokens, nkv, hd)
    wqf, wkf = oracle.bf16_to_f32(wq), oracle.bf16_to_f32(wk)
    got_q = oracle.bf16_to_f32(q_out).reshape(tokens, nq, hd)
    for t in range(tokens):
        for h in range(nq):
            want = chain(qf[t, h], wqf, float(pos[t]))
            assert np.abs(got_q[t, h] - want).max() <= 2.0 ** -6 * np.abs(want).max() + 1e-3
        if slots[t] < 0:
            continue
        b, o = slots[t] // bs, slots[t] % bs
        assert np.array_equal(vc[b, o].reshape(-1), v[t])
        for h in range(nkv):
            want = chain(kf[t, h], wkf, float(pos[t]))
            assert np.abs(oracle.bf16_to_f32(kc[b, o, h]) - want).max() <= 2.0 ** -6 * np.abs(want).max() + 1e-3
    assert (kc[0, 1] == 0x7FC0).all() and (vc[0, 3] == 0x7FC0).all()          # slots nobody mapped stay as they were
