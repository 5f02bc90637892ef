"""Two-CTA MMAs (token tiles of 128 and 256) against the single-CTA form of the same kernel and the oracle.

Both forms contract K in the same order with the same operands, so their outputs are compared bit for bit;
the oracle comparison is the usual tolerance."""
import numpy as np
import pytest

from gpu_util import DeviceCase, assert_close, ideal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("act_fp4", [False, True])
@pytest.mark.parametrize("M,K,N,ranks,max_rank", [
    (128, 512, 256, [16] * 6, 16),                   # one pair, token tile 128
    (256, 1024, 384, [32] * 16, 32),                 # odd number of feature tiles: the last pair is half empty
    (300, 512, 640, [8, 16, 32, 64] * 4, 64),        # two token tiles, the second partial
    (100, 768, 200, [8, 24], 24),                    # N not a multiple of 128, max_rank not of 16
])
def test_pair_matches_single_cta_and_oracle(cuda, atlas, oracle, M, K, N, ranks, max_rank, act_fp4):
    from atlas_b200 import synth
    case = synth.make_case("pair", M=M, K=K, N=N, ranks=ranks, max_rank=max_rank, max_loras=len(ranks) + 2,
                           none_frac=0.2, scale2=0.02, b_std=0.1, seed=M + N + K)
    dc = DeviceCase(cuda, atlas, case)
    mode = atlas.FLAG_FORCE_TCGEN05 | (atlas.FLAG_ACT_FP4 if act_fp4 else 0)
    y_pair, variant = dc.run(flags=mode)
    assert variant == atlas.VARIANT_TCGEN05
    assert atlas.device_status() == 0
    y_single, _ = dc.run(flags=mode | atlas.FLAG_NO_CTA_PAIR)
    assert atlas.device_status() == 0
    assert_close(oracle, y_pair, ideal(oracle, case, act_fp4=act_fp4), "pair")
    assert np.array_equal(y_pair, y_single)
    # B_s through the address tables instead of the strided pool
    y_tab, _ = dc.run(flags=mode, strided=False)
    assert np.array_equal(y_tab, y_pair)
    # base only
    yb_pair, _ = dc.run(lora=False, flags=mode)
    yb_single, _ = dc.run(lora=False, flags=mode | atlas.FLAG_NO_CTA_PAIR)
    assert np.array_equal(yb_pair, yb_single)
    none = case.seq_slot < 0
    assert none.any() and np.array_equal(y_pair[none], yb_pair[none])
    assert atlas.device_status() == 0
