"""The shrink of a prefill batch computed in token ranges into several copies of the scratch (what the ranks of a
column-parallel group do for one another), consumed by the fused call with FLAG_REUSE_SHRINK: same bits as the fused
call that runs the whole shrink itself."""
import numpy as np
import pytest

from gpu_util import bits_from_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fp4", [False, True])
@pytest.mark.parametrize("M,parts", [(4096, 4), (3000, 3)])
def test_token_ranges_into_several_scratch_buffers(cuda, atlas, oracle, M, parts, fp4):
    from atlas_b200 import synth, tp as tpmod
    dims = dict(hidden_size=512, intermediate_size=4864, num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    layer = synth.make_layer("shard", dims=dims, modules=("gate",), M=M, ranks=[64, 32, 16, 64, 48], max_rank=64, max_loras=6,
                             ids="segments", segments=17, none_frac=0.1, seed=M, scale2=0.02, b_std=0.1)
    dl = tpmod.DeviceLayer(cuda, atlas, layer, 1, 0)
    c = layer.projections[0]
    mode = atlas.FLAG_ACT_FP4 if fp4 else 0
    y_ref = cuda.empty((M, c.N), dtype=cuda.bfloat16, device="cuda")
    atlas.nvfp4_lora_linear(dl.desc(0, y_ref, extra_flags=mode))
    assert atlas.last_launch_shape()["lora_tiles_from_shrink"]
    # two more copies of the scratch, filled range by range; the descriptor's own scratch is then overwritten with junk
    ws_len = dl.proj[0]["ws"].numel()
    copies = [cuda.full((ws_len,), 0x5A, dtype=cuda.uint8, device="cuda") for _ in range(2)]
    rows = (M // parts + 63) // 64 * 64
    d = dl.desc(0, y_ref, extra_flags=mode)
    for r in range(parts):
        begin = r * rows
        atlas.lora_shrink_tiles(d, begin, min(rows, M - begin), copies)
    cuda.cuda.synchronize()
    dl.proj[0]["ws"].fill_(0xEE)
    for cp in copies:
        # the quantised activations (FP4 mode) live in the same scratch: produced by a regular call into this copy first
        y = cuda.full((M, c.N), 0x7FC0, dtype=cuda.int16, device="cuda")
        dl.proj[0]["ws"] = cp
        if fp4:
            tmp = cuda.empty((M, c.N), dtype=cuda.bfloat16, device="cuda")
            saved = cp.clone()
            atlas.nvfp4_lora_linear(dl.desc(0, tmp, extra_flags=mode))     # writes codes and its own tiles
            off = (atlas.act_fp4_ws_bytes(M, c.K) + 255) // 256 * 256
            cp[off:].copy_(saved[off:])                                     # the range-by-range tiles back in place
        atlas.nvfp4_lora_linear(dl.desc(0, y, extra_flags=mode | atlas.FLAG_REUSE_SHRINK))
        cuda.cuda.synchronize()
        assert np.array_equal(bits_from_dev(y), bits_from_dev(y_ref.view(cuda.int16)))
    assert atlas.device_status() == 0


def test_small_batches_are_refused(cuda, atlas, oracle):
    """Below 1024 tokens the shrink is the clustered kernel, which takes no row range: -1, nothing launched."""
    from atlas_b200 import synth, tp as tpmod
    case = synth.make_case("small", M=256, K=512, N=1024, ranks=[16] * 4, max_rank=16, seed=2)
    sh = tpmod.DeviceShard(cuda, atlas, case, 1, 0)
    y = cuda.empty((case.M, case.N), dtype=cuda.bfloat16, device="cuda")
    d = sh.desc(y)
    with pytest.raises(atlas.AtlasError) as e:
        atlas.lora_shrink_tiles(d, 0, 128, [sh._ws])
    assert e.value.status == -1
    cuda.cuda.synchronize()


@pytest.mark.parametrize("rank,n_ad", [(64, 40), (16, 96)])
def test_more_adapters_in_a_cluster_than_fit_into_one_pass(cuda, atlas, oracle, rank, n_ad):
    """Uniformly mixed adapter ids: every 128-row cluster of the prefill shrink meets far more adapters than its 512
    accumulator columns hold (8 of rank 64, 32 of rank 16), so it walks its rows in several passes, re-using the ring
    and the exchange area each time.  Checked against the oracle, in both output forms (masked tiles for the fused
    kernel, and rows of lora_t when no scratch is given), which must also agree bit for bit."""
    from atlas_b200 import synth
    from gpu_util import DeviceCase, assert_close, ideal
    case = synth.make_case("mix", M=1280, K=512, N=512, ranks=[rank] * n_ad, max_rank=rank, ids="uniform", none_frac=0.05,
                           scale2=0.02, b_std=0.1, seed=rank)
    per_cluster = [len(set(int(s) for s in case.seq_slot[i:i + 128] if s >= 0)) for i in range(0, case.M, 128)]
    assert min(per_cluster) > 512 // rank                      # every cluster needs more than one pass
    dc = DeviceCase(cuda, atlas, case)
    y_tiles, variant = dc.run(lora_ws=True)
    assert variant == atlas.VARIANT_TCGEN05 and atlas.last_launch_shape()["lora_tiles_from_shrink"]
    y_rows, _ = dc.run(lora_ws=False)
    assert not atlas.last_launch_shape()["lora_tiles_from_shrink"]
    assert np.array_equal(y_tiles, y_rows)
    assert_close(oracle, y_tiles, ideal(oracle, case), "several passes per cluster")
    assert atlas.device_status() == 0
