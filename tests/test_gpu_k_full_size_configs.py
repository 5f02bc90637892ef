"""The benchmark configurations at full size, sampled against the oracle (the oracle finishes a sample of outputs in
seconds; the whole tensors are covered by size-independent properties: exact routing of adapter-less rows, agreement of
launch shapes that contract in the same order, every element written)."""
import numpy as np
import pytest

from gpu_util import DeviceCase, assert_close, ideal

pytestmark = pytest.mark.gpu


def _sample(case, n_rows, n_cols, seed):
    rng = np.random.default_rng(seed)
    rows = np.sort(rng.choice(case.M, min(n_rows, case.M), replace=False)).astype(np.uint32)
    cols = np.sort(rng.choice(case.N, n_cols, replace=False)).astype(np.uint32)
    return rows, cols


@pytest.mark.parametrize("fp4", [False, True])
def test_config2_decode_batch(cuda, atlas, oracle, fp4):
    """64 tokens, each its own adapter of rank 8..64 out of 64, fused-QKV width 6144: split K, tiles from the shrink."""
    from atlas_b200 import synth
    case = synth.baseline_config(2)
    dc = DeviceCase(cuda, atlas, case)
    mode = atlas.FLAG_ACT_FP4 if fp4 else 0
    y, variant = dc.run(flags=mode, lora_ws=True)
    assert variant == atlas.VARIANT_TCGEN05
    shape = atlas.last_launch_shape()
    assert shape["token_tile"] == 64 and shape["k_split"] >= 2 and shape["lora_tiles_from_shrink"]
    rows, cols = _sample(case, 64, 64, 2)
    assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, case, rows=rows, cols=cols, act_fp4=fp4), "config2 sample")
    # without the rank table every adapter contracts over max_rank (zero padding): same values up to summation order
    y_pad, _ = dc.run(flags=mode, with_ranks=False, lora_ws=True)
    a, b = oracle.bf16_to_f32(y), oracle.bf16_to_f32(y_pad)
    assert np.abs(a - b).max() <= 2e-2 * np.abs(a).max()
    assert atlas.device_status() == 0


def test_config4_wide_mlp_many_adapters(cuda, atlas, oracle):
    """512 tokens, 128 adapters of rank 16 with Zipf ids, a quarter of the rows adapter-less, N = 28672."""
    from atlas_b200 import synth
    case = synth.baseline_config(4)
    dc = DeviceCase(cuda, atlas, case)
    y, variant = dc.run(lora_ws=True)
    assert variant == atlas.VARIANT_TCGEN05
    rows, cols = _sample(case, 64, 64, 4)
    assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, case, rows=rows, cols=cols), "config4 sample")
    assert np.isfinite(oracle.bf16_to_f32(y)).all()                    # every element of the pre-filled buffer was written
    y_build, _ = dc.run()                                               # tiles built in the kernel from lora_t: same bits
    assert np.array_equal(y_build, y)
    yb, _ = dc.run(lora=False)
    none = case.seq_slot < 0
    assert none.sum() > 64 and np.array_equal(y[none], yb[none])
    assert atlas.device_status() == 0


@pytest.mark.parametrize("fp4", [False, True])
def test_config3_prefill_segments(cuda, atlas, oracle, fp4):
    """8192 tokens in 32 contiguous segments, 8 adapters of rank 64, K = 4096, N = 14336."""
    from atlas_b200 import synth
    case = synth.baseline_config(3)
    dc = DeviceCase(cuda, atlas, case)
    y, variant = dc.run(lora_ws=True, flags=atlas.FLAG_ACT_FP4 if fp4 else 0)
    assert variant == atlas.VARIANT_TCGEN05
    # rows on both sides of every segment boundary, plus a random sample
    cuts = np.flatnonzero(np.diff(case.seq_slot) != 0)
    rows = np.unique(np.concatenate([cuts[:12], cuts[:12] + 1, _sample(case, 48, 1, 3)[0]])).astype(np.uint32)
    cols = _sample(case, 1, 64, 5)[1]
    assert rows.size * cols.size >= 4096
    assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, case, rows=rows, cols=cols, act_fp4=fp4), "config3 sample")
    assert np.isfinite(oracle.bf16_to_f32(y)).all()
    assert atlas.device_status() == 0
