"""Split K: several CTAs per output tile (few tiles for the SMs at hand), partial tiles summed over distributed
shared memory, against the one-CTA-per-tile form and the oracle."""
import numpy as np
import pytest

from gpu_util import DeviceCase, assert_close, ideal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["", "fp4", "single", "no_ws"])
@pytest.mark.parametrize("M,K,N,ranks,max_rank", [
    (64, 4096, 256, [8, 16, 32, 64] * 16, 64),       # decode-like: 8-way split, token tile 64, 160 LoRA granules
    (48, 768, 384, [16] * 5, 16),                    # 3 raw stages over 3 CTAs
    (256, 2048, 512, [32] * 16, 32),                 # token tile 256: pairs x 4-way split
    (130, 1280, 200, [8, 24], 24),                   # two token tiles of 128... ragged N, odd max_rank
    (16, 512, 128, [16] * 4, 16),                    # smallest tile
])
def test_split_matches_unsplit_and_oracle(cuda, atlas, oracle, M, K, N, ranks, max_rank, mode):
    from atlas_b200 import synth
    case = synth.make_case("ksplit", M=M, K=K, N=N, ranks=ranks, max_rank=max_rank, max_loras=len(ranks) + 1,
                           ids="distinct" if M == 64 else "uniform", none_frac=0.1, scale2=0.02, b_std=0.1, seed=M + K)
    dc = DeviceCase(cuda, atlas, case)
    fp4 = mode == "fp4"
    flags = atlas.FLAG_FORCE_TCGEN05 | (atlas.FLAG_ACT_FP4 if fp4 else 0) | (atlas.FLAG_NO_CTA_PAIR if mode == "single" else 0)
    ws = mode != "no_ws"
    y_split, variant = dc.run(flags=flags, lora_ws=ws)
    assert variant == atlas.VARIANT_TCGEN05
    assert atlas.device_status() == 0
    shape = atlas.last_launch_shape()
    assert shape["k_split"] > 1 and shape["lora_tiles_from_shrink"] == ws and not (shape["cta_pair"] and mode == "single")
    y_one, _ = dc.run(flags=flags | atlas.FLAG_NO_K_SPLIT, lora_ws=ws)
    assert atlas.last_launch_shape()["k_split"] == 1
    want = ideal(oracle, case, act_fp4=fp4)
    assert_close(oracle, y_split, want, "split")
    assert_close(oracle, y_one, want, "one CTA per tile")
    # the two differ only in the order of FP32 additions
    a, b = oracle.bf16_to_f32(y_split), oracle.bf16_to_f32(y_one)
    assert np.abs(a - b).max() <= 2e-2 * np.abs(b).max()
    # rows without an adapter equal the base-only result of the same form, bit for bit
    yb, _ = dc.run(lora=False, flags=flags)
    none = case.seq_slot < 0
    assert none.any() and np.array_equal(y_split[none], yb[none])
    assert atlas.device_status() == 0
