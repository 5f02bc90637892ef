"""The reference's own CUDA kernels (compiled unchanged for sm_100a under oracle/_ref) run on this GPU,
against the oracle — this pins the oracle to outputs of the reference itself — and against this
library's replacements for them."""
import numpy as np
import pytest

from gpu_util import ATOL, RTOL, DeviceCase, RefModule, assert_close, bits_from_dev, device_pool, host_pool, ideal, ref_available, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _reference_cubins():
    """These tests are the pin of the oracle to the reference's own kernels: without the compiled kernels they fail, they
    do not skip.  The cubins are built by `make -C oracle REF=<checkout>` (or build() with the checkout beside the
    repository) and travel with the working tree."""
    if not ref_available():
        pytest.fail("oracle/_ref/*.cubin are missing: build them from a checkout of the reference (make -C oracle REF=...)")


def u32(v):
    return ("u32", v)


def test_reference_dequant_equals_oracle(cuda, oracle):
    torch = cuda
    from atlas_b200 import synth
    N, K = 128, 512
    packed, scales = synth.make_nvfp4_weight(21, N, K)
    scales[0, :] = np.arange(32, dtype=np.uint8)                       # subnormal scale bytes too
    out = torch.zeros((N, K), dtype=torch.int16, device="cuda")
    dp, ds = to_dev(torch, packed), to_dev(torch, scales)
    RefModule("dequant_nvfp4_bf16").launch("dequant_nvfp4_to_bf16", (N, 1, 1), (256, 1, 1),
                                           [dp.data_ptr(), ds.data_ptr(), out.data_ptr(), 0.5, u32(N), u32(K)])
    torch.cuda.synchronize()
    assert np.array_equal(bits_from_dev(out), oracle.dequant_nvfp4_to_bf16(packed, scales, 0.5, N, K))


def test_reference_bgmv_equals_oracle_and_library(cuda, atlas, oracle):
    torch = cuda
    from atlas_b200 import synth
    M, K, N, max_rank = 24, 1024, 512, 16
    case = synth.make_case("ref", M=M, K=K, N=N, ranks=[8, 16, 4], max_rank=max_rank, max_loras=4,
                           none_frac=0.2, b_std=0.3, seed=9)
    pool = device_pool(torch, atlas, case)
    base = oracle.f32_to_bf16(np.random.default_rng(2).standard_normal((M, N)).astype(np.float32))
    x, slot = to_dev(torch, case.x), to_dev(torch, case.seq_slot)
    out_ref, xa_ref = to_dev(torch, base), torch.zeros((M, max_rank), dtype=torch.int16, device="cuda")
    mod = RefModule("lora_bgmv")
    mod.launch("lora_bgmv_shrink", ((max_rank + 3) // 4, M, 1), (256, 1, 1),
               [x.data_ptr(), slot.data_ptr(), pool.a_table.data_ptr(), xa_ref.data_ptr(), u32(M), u32(max_rank), u32(K), u32(K)])
    mod.launch("lora_bgmv_expand_fold", ((N + 3) // 4, M, 1), (256, 1, 1),
               [xa_ref.data_ptr(), slot.data_ptr(), pool.b_table.data_ptr(), pool.scale_table.data_ptr(),
                out_ref.data_ptr(), u32(M), u32(N), u32(max_rank), u32(N)])
    torch.cuda.synchronize()
    want = base.copy()
    want_xa = oracle.lora_bgmv_staged(case.x, case.seq_slot, host_pool(oracle, case), want, M)
    ref_out, ref_xa = bits_from_dev(out_ref), bits_from_dev(xa_ref)
    routed = case.seq_slot >= 0
    assert np.array_equal(ref_out[~routed], base[~routed])
    # same rounding boundaries, different FP32 summation order: equal up to the last BF16 bit
    assert_close(oracle, ref_xa, oracle.bf16_to_f32(want_xa), "reference xa vs oracle")
    assert_close(oracle, ref_out, oracle.bf16_to_f32(want), "reference out vs oracle")
    same = (ref_out == want).mean()
    assert same > 0.95, f"only {same:.3f} of outputs bit-identical to the oracle"
    # this library's replacement against the reference kernel
    out_lib, xa_lib = to_dev(torch, base), torch.zeros((M, max_rank), dtype=torch.int16, device="cuda")
    atlas.apply_lora_bgmv(pool.route(), x, out_lib, slot, M, K, N, xa_lib)
    torch.cuda.synchronize()
    assert_close(oracle, bits_from_dev(out_lib), oracle.bf16_to_f32(ref_out), "library vs reference kernel")
    assert (bits_from_dev(out_lib) == ref_out).mean() > 0.95


def test_reference_w4a16_gemm_equals_oracle_and_library(cuda, atlas, oracle):
    torch = cuda
    from atlas_b200 import synth
    M, K, N = 48, 512, 256
    case = synth.make_case("ref", M=M, K=K, N=N, ranks=[8], max_rank=8, scale2=0.01, seed=4)
    x, dp, ds = to_dev(torch, case.x), to_dev(torch, case.packed), to_dev(torch, case.scales)
    c_ref = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    RefModule("w4a16_gemm").launch("w4a16_gemm", ((N + 63) // 64, (M + 63) // 64, 1), (128, 1, 1),
                                   [x.data_ptr(), dp.data_ptr(), ds.data_ptr(), 0.01, c_ref.data_ptr(), u32(M), u32(N), u32(K)])
    torch.cuda.synchronize()
    want = oracle.w4a16_gemm_bf16w(case.x, case.packed, case.scales, float(np.float32(0.01)), M, N, K)
    assert_close(oracle, bits_from_dev(c_ref), oracle.bf16_to_f32(want), "reference gemm vs oracle")
    c_lib = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    atlas.w4a16_gemm(x, dp, ds, float(np.float32(0.01)), c_lib, M, N, K)
    torch.cuda.synchronize()
    assert_close(oracle, bits_from_dev(c_lib), oracle.bf16_to_f32(bits_from_dev(c_ref)), "library vs reference gemm")


def test_reference_launch_sequence_on_configuration_1(cuda, atlas, oracle, capsys):
    """The reference's own three launches for this layer (w4a16_gemm, lora_bgmv_shrink, lora_bgmv_expand_fold), compiled
    unchanged for sm_100a, at the size of benchmark configuration 1: same result as this library's reference-rounding
    mode, and how long the sequence takes on this GPU next to the fused call (printed; run with -s to read it)."""
    torch = cuda
    from atlas_b200 import synth
    case = synth.baseline_config(1)
    M, K, N, max_rank = case.M, case.K, case.N, case.max_rank
    dc = DeviceCase(torch, atlas, case)
    pool = dc.pool
    gemm, bgmv = RefModule("w4a16_gemm"), RefModule("lora_bgmv")
    out_ref = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    xa_ref = torch.zeros((M, max_rank), dtype=torch.int16, device="cuda")

    def reference_sequence():
        gemm.launch("w4a16_gemm", ((N + 63) // 64, (M + 63) // 64, 1), (128, 1, 1),
                    [dc.x.data_ptr(), dc.packed.data_ptr(), dc.scales.data_ptr(), float(case.scale2), out_ref.data_ptr(),
                     u32(M), u32(N), u32(K)], stream=torch.cuda.current_stream().cuda_stream)
        bgmv.launch("lora_bgmv_shrink", ((max_rank + 3) // 4, M, 1), (256, 1, 1),
                    [dc.x.data_ptr(), dc.seq_slot.data_ptr(), pool.a_table.data_ptr(), xa_ref.data_ptr(),
                     u32(M), u32(max_rank), u32(K), u32(K)], stream=torch.cuda.current_stream().cuda_stream)
        bgmv.launch("lora_bgmv_expand_fold", ((N + 3) // 4, M, 1), (256, 1, 1),
                    [xa_ref.data_ptr(), dc.seq_slot.data_ptr(), pool.b_table.data_ptr(), pool.scale_table.data_ptr(),
                     out_ref.data_ptr(), u32(M), u32(N), u32(max_rank), u32(N)], stream=torch.cuda.current_stream().cuda_stream)

    reference_sequence()
    torch.cuda.synchronize()
    y_staged, _ = dc.run(flags=atlas.FLAG_STAGED_LORA)                   # this library, the reference's rounding boundaries
    ref = bits_from_dev(out_ref)
    assert_close(oracle, y_staged, oracle.bf16_to_f32(ref), "library (reference rounding) vs reference kernels")
    y_fused, variant = dc.run(lora_ws=True)
    assert variant == atlas.VARIANT_TCGEN05
    none = case.seq_slot < 0
    got, want = oracle.bf16_to_f32(y_fused), oracle.bf16_to_f32(ref)
    assert_close(oracle, y_fused[none], want[none], "fused vs reference kernels, adapter-less rows")
    # Adapted rows: the reference rounds the base result and the delta to BF16 before it folds them, the fused kernel
    # rounds once.  So the path's rtol / atol hold up to one BF16 ulp (2^-8) of each of the two terms — which matters
    # only where base and delta cancel.  The terms themselves come from the oracle's FP32 ideal on a row sample.
    rows = np.flatnonzero(~none)[::3].astype(np.uint32)
    base_f = ideal(oracle, case, rows=rows, lora=False)
    full_f = ideal(oracle, case, rows=rows)
    lim = ATOL + RTOL * np.abs(want[rows]) + 2.0 ** -8 * (np.abs(base_f) + np.abs(full_f - base_f))
    assert (np.abs(got[rows] - want[rows]) <= lim).all()
    assert (np.abs(got[rows] - full_f) <= ATOL + RTOL * np.abs(full_f)).all()          # and the fused result is inside the plain tolerance of the ideal

    def timed(fn, n=20):
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in ev:
            flush.fill_(1)
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return float(np.median([a.elapsed_time(b) for a, b in ev])) * 1e3

    y = torch.empty((M, N), dtype=torch.int16, device="cuda")
    ws_bytes = atlas.lora_ws_bytes(M, case.max_loras, max_rank)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    d = atlas.make_linear_desc(x=dc.x, m=M, k=K, n=N, y=y, w_packed=dc.packed, w_scale=dc.scales, scale2=case.scale2,
                               seq_slot=dc.seq_slot, route=pool.route(True, True), lora_t=dc.lora_t, ws=ws, ws_bytes=ws_bytes)
    t_ref = timed(reference_sequence)
    t_lib = timed(lambda: atlas.nvfp4_lora_linear(d))
    with capsys.disabled():
        print(f"\n[configuration 1 on this GPU] reference kernels (3 launches): {t_ref:.1f} us; fused call: {t_lib:.1f} us; "
              f"ratio {t_ref / t_lib:.1f}x")
    assert atlas.device_status() == 0


def test_reference_dense_gemv_and_the_dense_tensor_core_base(cuda, atlas, oracle, capsys):
    """Benchmark configuration 0's base (dense BF16 weight, K = N = 4096): the reference's `dense_gemv_bf16`, one launch per
    token row, against the oracle and against this library's tensor-core dense kernel on the same 16 rows; times printed."""
    torch = cuda
    from atlas_b200 import synth
    case = synth.baseline_config(0)
    M, K, N = case.M, case.K, case.N
    dc = DeviceCase(torch, atlas, case)
    gemv = RefModule("dense_gemv_bf16")
    out_ref = torch.zeros((M, N), dtype=torch.int16, device="cuda")

    def reference_rows():
        for r in range(M):
            gemv.launch("dense_gemv_bf16", ((N + 3) // 4, 1, 1), (256, 1, 1),
                        [dc.x.data_ptr() + r * K * 2, dc.w_bf16.data_ptr(), out_ref.data_ptr() + r * N * 2, u32(N), u32(K)],
                        stream=torch.cuda.current_stream().cuda_stream)
    reference_rows()
    torch.cuda.synchronize()
    want = ideal(oracle, case, lora=False)
    assert_close(oracle, bits_from_dev(out_ref), want, "reference dense gemv vs oracle")
    y, variant = dc.run(lora=False)
    assert variant == atlas.VARIANT_TCGEN05 and atlas.last_launch_shape()["k_split"] >= 2
    assert_close(oracle, y, want, "dense tensor-core base vs oracle")
    assert_close(oracle, y, oracle.bf16_to_f32(bits_from_dev(out_ref)), "dense tensor-core base vs reference gemv")

    def timed(fn, n=20):
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in ev:
            flush.fill_(1)
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return float(np.median([a.elapsed_time(b) for a, b in ev])) * 1e3
    yb = torch.empty((M, N), dtype=torch.int16, device="cuda")
    d = atlas.make_linear_desc(x=dc.x, m=M, k=K, n=N, y=yb, w_bf16=dc.w_bf16)
    t_ref, t_lib = timed(reference_rows), timed(lambda: atlas.nvfp4_lora_linear(d))
    with capsys.disabled():
        print(f"\n[configuration 0 base on this GPU] reference dense_gemv_bf16 x {M} rows: {t_ref:.1f} us; dense tensor-core kernel: "
              f"{t_lib:.1f} us ({N * K * 2 / t_lib / 1e3:.0f} GB/s of weights)")
    assert atlas.device_status() == 0
