"""LoRA activation tiles written by the shrink (scratch in `ws`) against the in-kernel build and the oracle.

Both ways put the same BF16 values into the same K-steps, so the outputs are compared bit for bit."""
import numpy as np
import pytest

from gpu_util import DeviceCase, assert_close, ideal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("flags_extra", ["", "fp4", "single"])
@pytest.mark.parametrize("M,K,N,ranks,max_rank,with_ranks,ids", [
    (16, 256, 128, [16] * 4, 16, True, "uniform"),
    (64, 512, 256, [8, 16, 32, 64] * 16, 64, True, "distinct"),    # every token its own adapter, mixed ranks
    (64, 512, 256, [8, 16, 32, 64] * 8, 64, False, "uniform"),     # no rank table: every slot counts max_rank
    (300, 512, 384, [32] * 16, 32, True, "uniform"),               # two token tiles, the second partial
    (130, 256, 200, [8, 24], 24, True, "uniform"),                 # max_rank not a multiple of 16
    (700, 256, 256, [16] * 40, 16, True, "zipf"),                  # three tiles, many adapters
])
def test_tiles_match_in_kernel_build(cuda, atlas, oracle, M, K, N, ranks, max_rank, with_ranks, ids, flags_extra):
    from atlas_b200 import synth
    case = synth.make_case("tiles", M=M, K=K, N=N, ranks=ranks, max_rank=max_rank, max_loras=len(ranks) + 3, ids=ids,
                           none_frac=0.15, scale2=0.02, b_std=0.1, seed=M + N + 7)
    dc = DeviceCase(cuda, atlas, case)
    fp4 = flags_extra == "fp4"
    mode = atlas.FLAG_FORCE_TCGEN05 | (atlas.FLAG_ACT_FP4 if fp4 else 0) | (atlas.FLAG_NO_CTA_PAIR if flags_extra == "single" else 0)
    y_build, _ = dc.run(with_ranks=with_ranks, flags=mode)
    dc.lora_t.zero_()                                   # the tile path must not depend on lora_t
    y_tiles, variant = dc.run(with_ranks=with_ranks, flags=mode, lora_ws=True)
    assert variant == atlas.VARIANT_TCGEN05
    assert atlas.device_status() == 0
    assert (dc.lora_t == 0).all()
    assert_close(oracle, y_tiles, ideal(oracle, case, use_ranks=with_ranks, act_fp4=fp4), "tiles")
    assert np.array_equal(y_tiles, y_build)
    # a second call (fresh scratch) gives the same bits
    y_again, _ = dc.run(with_ranks=with_ranks, flags=mode, lora_ws=True)
    assert np.array_equal(y_again, y_tiles)


def test_scratch_too_small_falls_back_to_the_build(cuda, atlas, oracle):
    from atlas_b200 import synth
    case = synth.make_case("tiles_small", M=64, K=256, N=128, ranks=[16] * 8, max_rank=16, seed=11, b_std=0.1, scale2=0.02)
    dc = DeviceCase(cuda, atlas, case)
    y0, _ = dc.run(flags=atlas.FLAG_FORCE_TCGEN05)
    y = cuda.full((64, 128), 0x7FC0, dtype=cuda.int16, device="cuda")
    ws = cuda.zeros(1024, dtype=cuda.uint8, device="cuda")
    d = atlas.make_linear_desc(x=dc.x, m=64, k=256, n=128, y=y, w_packed=dc.packed, w_scale=dc.scales, scale2=case.scale2,
                               seq_slot=dc.seq_slot, route=dc.pool.route(True, True), lora_t=dc.lora_t,
                               flags=atlas.FLAG_FORCE_TCGEN05, ws=ws, ws_bytes=1024)
    atlas.nvfp4_lora_linear(d)
    cuda.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy().view(np.uint16), y0)
    assert (ws == 0).all()
    assert atlas.device_status() == 0
