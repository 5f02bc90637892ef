"""The CUDA-core path of the fused layer (any shape, dense-BF16 base, reference rounding mode)."""
import numpy as np
import pytest

from gpu_util import ATOL, RTOL, DeviceCase, assert_close, ideal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N,ranks,max_rank", [
    (5, 48, 70, [4, 8], 8),
    (16, 512, 192, [16] * 4, 16),
    (70, 272, 130, [8, 16, 32], 32),
])
def test_simt_nvfp4_fused(cuda, atlas, oracle, M, K, N, ranks, max_rank):
    from atlas_b200 import synth
    case = synth.make_case("simt", M=M, K=K, N=N, ranks=ranks, max_rank=max_rank, none_frac=0.2,
                           scale2=0.02, b_std=0.3, seed=K)
    dc = DeviceCase(cuda, atlas, case, out_row_stride=N + 6)
    y, variant = dc.run(flags=atlas.FLAG_FORCE_SIMT)
    assert variant == atlas.VARIANT_SIMT
    # This path keeps the reference's rounding boundaries (base -> BF16, xa -> BF16, delta -> BF16, fold -> BF16,
    # kernels/gb10/common/lora_bgmv.cu:121-125, :214-223), so where base and delta cancel the result carries the
    # BF16 rounding of the larger term: allow one BF16 ulp (2^-8) of |base| and of |delta| beyond the path's rtol / atol.
    want, want_base = ideal(oracle, case), ideal(oracle, case, lora=False)
    got = oracle.bf16_to_f32(np.ascontiguousarray(y[:, :N]))
    lim = ATOL + RTOL * np.abs(want) + 2.0 ** -8 * (np.abs(want_base) + np.abs(want - want_base))
    assert np.isfinite(got).all() and (np.abs(got - want) <= lim).all(), "fused"
    assert (y[:, N:] == 0x7FC0).all()                       # padding columns of the output are untouched
    yb, _ = dc.run(lora=False, flags=atlas.FLAG_FORCE_SIMT)
    assert_close(oracle, yb[:, :N], want_base, "base")
    none = case.seq_slot < 0
    assert np.array_equal(y[none], yb[none])                # un-adapted rows are the base result, bit for bit
    assert atlas.device_status() == 0


def test_config0_dense_bf16_base(cuda, atlas, oracle):
    """Benchmark configuration 0: M=16, K=N=4096, BF16 base, 4 adapters of rank 16, alpha 32.  The base runs on the tensor
    cores (split K inside clusters), the LoRA term keeps the reference's staging; the CUDA-core form gives the same
    result within the tolerance."""
    from atlas_b200 import synth
    case = synth.baseline_config(0)
    dc = DeviceCase(cuda, atlas, case)
    y, variant = dc.run()
    assert variant == atlas.VARIANT_TCGEN05
    assert_close(oracle, y, ideal(oracle, case), "config0")
    want_seq, _ = oracle.reference_sequence(case.x, case.M, case.N, case.K, w_bf16=case.w_bf16,
                                            seq_slot=case.seq_slot, pool=__import__("gpu_util").host_pool(oracle, case))
    assert_close(oracle, y, oracle.bf16_to_f32(want_seq), "config0 vs reference launch sequence")
    y_simt, variant = dc.run(flags=atlas.FLAG_FORCE_SIMT)
    assert variant == atlas.VARIANT_SIMT
    assert_close(oracle, y_simt, oracle.bf16_to_f32(y), "CUDA-core form vs tensor-core form")
    assert atlas.device_status() == 0


@pytest.mark.parametrize("M,K,N", [(1, 256, 200), (16, 4096, 512), (100, 320, 384), (300, 1024, 1000), (37, 64, 128)])
def test_dense_bf16_tensor_core_base_shapes(cuda, atlas, oracle, M, K, N):
    """Dense BF16 weights at ragged shapes: token tiles of 16..128, feature tiles past N, one K block, split K."""
    from atlas_b200 import synth
    case = synth.make_case("dense", M=M, K=K, N=N, ranks=[8, 16], max_rank=16, base="bf16", none_frac=0.3, b_std=0.1, seed=M + N)
    dc = DeviceCase(cuda, atlas, case, out_row_stride=N + 4)
    yb, variant = dc.run(lora=False)
    assert variant == atlas.VARIANT_TCGEN05
    assert_close(oracle, yb[:, :N], ideal(oracle, case, lora=False), "dense base")
    assert (yb[:, N:] == 0x7FC0).all()
    y, _ = dc.run()
    want, want_base = ideal(oracle, case), ideal(oracle, case, lora=False)
    got = oracle.bf16_to_f32(np.ascontiguousarray(y[:, :N]))
    lim = ATOL + RTOL * np.abs(want) + 2.0 ** -8 * (np.abs(want_base) + np.abs(want - want_base))     # staged LoRA roundings
    assert np.isfinite(got).all() and (np.abs(got - want) <= lim).all()
    none = case.seq_slot < 0
    assert np.array_equal(y[none], yb[none])
    assert atlas.device_status() == 0
