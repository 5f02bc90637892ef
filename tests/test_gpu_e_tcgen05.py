"""The tcgen05 path of the fused layer against the FP32-accumulated oracle."""
import numpy as np
import pytest

from gpu_util import DeviceCase, assert_close, ideal

pytestmark = pytest.mark.gpu


def _tc(atlas):
    return atlas.FLAG_FORCE_TCGEN05


def test_decode_through_the_mma_is_bit_exact(cuda, atlas, oracle):
    """One-hot activations: y[m, f] = w[f, m] exactly, so the in-kernel E2M1 x E4M3 expansion is
    compared bit for bit with the oracle's decode (all 16 codes, normal and subnormal scale bytes)."""
    from atlas_b200 import synth
    K, N = 256, 256
    packed, scales = synth.make_nvfp4_weight(31, N, K)
    scales[:, 0] = np.arange(N, dtype=np.uint8) % 0x7F               # every finite scale byte incl. subnormals
    packed[0, :8] = np.arange(8, dtype=np.uint8) | ((np.arange(8, dtype=np.uint8) + 8) << 4)
    x = np.zeros((K, K), dtype=np.float32)
    x[np.arange(K), np.arange(K)] = 1.0
    case = synth.Case("onehot", K, K, N, 8, 1, oracle.f32_to_bf16(x), np.full(K, -1, np.int32), [None],
                      packed=packed, scales=scales, scale2=1.0)
    y, variant = DeviceCase(cuda, atlas, case).run(lora=False, flags=_tc(atlas))
    assert variant == atlas.VARIANT_TCGEN05
    want = oracle.dequant_nvfp4_to_bf16(packed, scales, 1.0, N, K).T     # [K, N]
    # a sum of signed zeros is +0: a weight of -0.0 legitimately comes out as +0.0
    want = np.where(want == 0x8000, 0, want)
    assert np.array_equal(y, want)
    assert atlas.device_status() == 0


@pytest.mark.parametrize("M,K,N", [(16, 256, 128), (40, 512, 200), (64, 1024, 384), (100, 768, 256),
                                   (256, 512, 128), (300, 256, 264), (1, 256, 128)])
def test_base_linear(cuda, atlas, oracle, M, K, N):
    from atlas_b200 import synth
    case = synth.make_case("base", M=M, K=K, N=N, ranks=[8], max_rank=8, scale2=0.02, seed=M + K)
    dc = DeviceCase(cuda, atlas, case, out_row_stride=N + 8)
    y, variant = dc.run(lora=False, flags=_tc(atlas))
    assert variant == atlas.VARIANT_TCGEN05
    assert_close(oracle, y[:, :N], ideal(oracle, case, lora=False), "base")
    assert (y[:, N:] == 0x7FC0).all()
    assert atlas.device_status() == 0


@pytest.mark.parametrize("M,K,N,ranks,max_rank,with_ranks", [
    (16, 256, 128, [16] * 4, 16, True),
    (64, 512, 256, [8, 16, 32, 64] * 8, 64, True),      # heterogeneous ranks, many adapters per tile
    (64, 512, 256, [8, 16, 32, 64] * 8, 64, False),     # contraction over max_rank (no rank table)
    (300, 512, 384, [32] * 16, 32, True),                # two token tiles, the second one partial
    (130, 256, 200, [8, 24], 24, True),                  # max_rank not a multiple of 16, N not of 128
])
def test_fused_lora(cuda, atlas, oracle, M, K, N, ranks, max_rank, with_ranks):
    from atlas_b200 import synth
    case = synth.make_case("fused", M=M, K=K, N=N, ranks=ranks, max_rank=max_rank, max_loras=len(ranks) + 3,
                           none_frac=0.15, scale2=0.02, b_std=0.1, seed=M + N)
    dc = DeviceCase(cuda, atlas, case)
    y, variant = dc.run(with_ranks=with_ranks, flags=_tc(atlas))
    assert variant == atlas.VARIANT_TCGEN05
    want = ideal(oracle, case, use_ranks=with_ranks)
    assert_close(oracle, y, want, "fused")
    # B_s through the address tables (no strided pool declared) must give the same bits as B_s by TMA
    y_tab, _ = dc.run(with_ranks=with_ranks, flags=_tc(atlas), strided=False)
    assert np.array_equal(y_tab, y)
    yb, _ = dc.run(lora=False, flags=_tc(atlas))
    none = case.seq_slot < 0
    assert none.any() and np.array_equal(y[none], yb[none])            # routing is exact
    # the LoRA term is visible at this scale, and the device result tracks it
    base = ideal(oracle, case, lora=False)
    assert np.abs(want - base)[~none].mean() > 0.05
    got = oracle.bf16_to_f32(y)
    num = ((got - base)[~none] * (want - base)[~none]).sum()
    den = np.linalg.norm((got - base)[~none]) * np.linalg.norm((want - base)[~none])
    assert num / den > 0.99
    assert atlas.device_status() == 0


def test_token_permutation_is_bit_exact(cuda, atlas, oracle):
    from atlas_b200 import synth
    import copy
    case = synth.make_case("perm", M=96, K=512, N=256, ranks=[16] * 6, max_rank=16, none_frac=0.2, scale2=0.02, b_std=0.3, seed=2)
    y, _ = DeviceCase(cuda, atlas, case).run(flags=_tc(atlas))
    perm = np.random.default_rng(0).permutation(case.M)
    c2 = copy.copy(case)
    c2.x, c2.seq_slot = case.x[perm].copy(), case.seq_slot[perm].copy()
    y2, _ = DeviceCase(cuda, atlas, c2).run(flags=_tc(atlas))
    assert np.array_equal(y2, y[perm])


def test_bad_slot_is_recorded_not_fatal(cuda, atlas, oracle):
    from atlas_b200 import synth
    case = synth.make_case("bad", M=16, K=256, N=128, ranks=[8, 8], max_rank=8, max_loras=4, ids="distinct", scale2=0.02, seed=6)
    case.seq_slot[3] = 77                   # beyond the tables
    case.seq_slot[4] = 2                    # resident slot with null entries
    dc = DeviceCase(cuda, atlas, case)
    y, _ = dc.run(flags=_tc(atlas))
    yb, _ = dc.run(lora=False, flags=_tc(atlas))
    assert np.array_equal(y[3], yb[3]) and np.array_equal(y[4], yb[4])
    assert atlas.device_status() == 1
    want = ideal(oracle, case)
    assert_close(oracle, y, want, "fused with bad slots")


def test_auto_dispatch_and_fallback(cuda, atlas, oracle):
    from atlas_b200 import synth
    ok = synth.make_case("d", M=8, K=256, N=128, ranks=[8], max_rank=8, scale2=0.02, seed=1)
    _, v = DeviceCase(cuda, atlas, ok).run()
    assert v == atlas.VARIANT_TCGEN05
    odd = synth.make_case("d", M=8, K=272, N=128, ranks=[8], max_rank=8, scale2=0.02, seed=1)   # K % 256 != 0
    dc = DeviceCase(cuda, atlas, odd)
    y, v = dc.run()
    assert v == atlas.VARIANT_SIMT
    assert_close(oracle, y, ideal(oracle, odd), "fallback")
    with pytest.raises(atlas.AtlasError):
        dc.run(flags=atlas.FLAG_FORCE_TCGEN05)


def test_config1_full_size_sampled(cuda, atlas, oracle):
    """Benchmark configuration 1 at full size (M=256, K=5120, N=17408, 16 adapters of rank 32):
    a random sample of outputs against the oracle, and exact routing on the adapter-less rows."""
    from atlas_b200 import synth
    case = synth.baseline_config(1)
    dc = DeviceCase(cuda, atlas, case)
    y, variant = dc.run()
    assert variant == atlas.VARIANT_TCGEN05
    rng = np.random.default_rng(0)
    rows = np.sort(rng.choice(case.M, 24, replace=False)).astype(np.uint32)
    cols = np.sort(rng.choice(case.N, 96, replace=False)).astype(np.uint32)
    assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, case, rows=rows, cols=cols), "config1 sample")
    yb, _ = dc.run(lora=False)
    none = case.seq_slot < 0
    assert np.array_equal(y[none], yb[none])
    assert atlas.device_status() == 0
