"""Output placement of the tcgen05 epilogue: through shared memory with 16-byte stores, directly, and into the
gathered buffers of several tensor-parallel ranks (here: several buffers on the one GPU, standing in for peers)."""
import numpy as np
import pytest

from gpu_util import DeviceCase, assert_close, bits_from_dev, ideal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N", [(16, 256, 128), (100, 512, 200), (256, 256, 264), (300, 512, 384)])
def test_direct_and_staged_stores_agree(cuda, atlas, oracle, M, K, N):
    """A row stride that is not a multiple of 8 elements rules out 16-byte stores: same bits either way."""
    from atlas_b200 import synth
    case = synth.make_case("place", M=M, K=K, N=N, ranks=[16] * 4, max_rank=16, none_frac=0.2, scale2=0.02, b_std=0.1, seed=M + N)
    y_staged, _ = DeviceCase(cuda, atlas, case, out_row_stride=N + 8).run(flags=atlas.FLAG_FORCE_TCGEN05)
    y_direct, _ = DeviceCase(cuda, atlas, case, out_row_stride=N + 3).run(flags=atlas.FLAG_FORCE_TCGEN05)
    assert np.array_equal(y_staged[:, :N], y_direct[:, :N])
    assert (y_staged[:, N:] == 0x7FC0).all() and (y_direct[:, N:] == 0x7FC0).all()
    assert_close(oracle, y_staged[:, :N], ideal(oracle, case), "staged")
    assert atlas.device_status() == 0


@pytest.mark.parametrize("tp", [2, 4])
@pytest.mark.parametrize("act_fp4", [False, True])
def test_column_shards_fill_every_ranks_buffer(cuda, atlas, oracle, tp, act_fp4):
    from atlas_b200 import synth, tp as tpmod
    M, K, N = 200, 512, 1024
    case = synth.make_case("tp_place", M=M, K=K, N=N, ranks=[16, 32, 8, 32, 16], max_rank=32, none_frac=0.2,
                           scale2=0.02, b_std=0.1, seed=tp)
    mode = atlas.FLAG_FORCE_TCGEN05 | (atlas.FLAG_ACT_FP4 if act_fp4 else 0)
    # the unsharded layer
    whole = tpmod.DeviceShard(cuda, atlas, case, 1, 0)
    y_ref = cuda.empty((M, N), dtype=cuda.bfloat16, device="cuda")
    atlas.nvfp4_lora_linear(whole.desc(y_ref, extra_flags=mode))
    # every rank's shard writes its columns into every rank's gathered buffer (row stride wider than N)
    stride = N + 16
    bufs = [cuda.full((M, stride), 0x7FC0, dtype=cuda.int16, device="cuda") for _ in range(tp)]
    for r in range(tp):
        sh = tpmod.DeviceShard(cuda, atlas, case, tp, r)
        variant = atlas.nvfp4_lora_linear(sh.desc(None, extra_flags=mode, out_row_stride=stride, y_dest=bufs,
                                                  y_col_offset=r * sh.n_local))
        assert variant == atlas.VARIANT_TCGEN05
    cuda.cuda.synchronize()
    want = bits_from_dev(y_ref.view(cuda.int16))
    for b in bufs:
        got = bits_from_dev(b)
        assert np.array_equal(got[:, :N], want)
        assert (got[:, N:] == 0x7FC0).all()
    assert_close(oracle, want, ideal(oracle, case, act_fp4=act_fp4), "unsharded")
    assert atlas.device_status() == 0


def test_placement_argument_errors(cuda, atlas, oracle):
    from atlas_b200 import synth, tp as tpmod
    case = synth.make_case("tp_err", M=32, K=256, N=256, ranks=[8], max_rank=8, seed=2)
    sh = tpmod.DeviceShard(cuda, atlas, case, 2, 1)
    bufs = [cuda.zeros((32, 256), dtype=cuda.int16, device="cuda") for _ in range(2)]
    with pytest.raises(atlas.AtlasError) as e:      # columns beyond the row
        atlas.nvfp4_lora_linear(sh.desc(None, out_row_stride=256, y_dest=bufs, y_col_offset=192))
    assert e.value.status == -1
    with pytest.raises(atlas.AtlasError) as e:      # rows that cannot take 16-byte stores
        atlas.nvfp4_lora_linear(sh.desc(None, out_row_stride=260, y_dest=bufs, y_col_offset=128))
    assert e.value.status == -3
    with pytest.raises(atlas.AtlasError) as e:      # no CUDA-core form
        atlas.nvfp4_lora_linear(sh.desc(None, extra_flags=atlas.FLAG_FORCE_SIMT, out_row_stride=256, y_dest=bufs, y_col_offset=128))
    assert e.value.status == -1
    with pytest.raises(atlas.AtlasError) as e:
        atlas.nvfp4_lora_linear(sh.desc(None, out_row_stride=256, y_dest=bufs + [None], y_col_offset=128))
    assert e.value.status == -4
    cuda.cuda.synchronize()


@pytest.mark.parametrize("tp_n,K,r", [(8, 1024, 5), (4, 768, 2), (2, 1280, 1)])
def test_shards_of_configuration_1_shape(cuda, atlas, oracle, tp_n, K, r):
    """The column shard a tp_n-rank split of configuration 1 gives one rank (tp_n = 8: 17 feature tiles, an odd number, so
    the last CTA pair, where pairs are used, is half empty), 256 tokens, few tiles for the GPU (split K inside clusters,
    among them a three-way split of a 256-token tile), results stored into tp_n gathered buffers."""
    from atlas_b200 import synth, tp as tpmod
    M, N = 256, 17408
    case = synth.make_case("shard", M=M, K=K, N=N, ranks=[32] * 16, max_rank=32, none_frac=0.1, scale2=0.02, b_std=0.1, seed=tp_n)
    sh = tpmod.DeviceShard(cuda, atlas, case, tp_n, r)
    assert sh.n_local == N // tp_n
    bufs = [cuda.full((M, N), 0x7FC0, dtype=cuda.int16, device="cuda") for _ in range(tp_n)]
    atlas.nvfp4_lora_linear(sh.desc(None, out_row_stride=N, y_dest=bufs, y_col_offset=r * sh.n_local))
    cuda.cuda.synchronize()
    shape = atlas.last_launch_shape()
    assert shape["token_tile"] == 256 and shape["k_split"] >= 2
    lo, hi = r * sh.n_local, (r + 1) * sh.n_local
    rows = np.arange(0, M, 5).astype(np.uint32)
    cols = np.arange(lo, hi, 7).astype(np.uint32)
    want = ideal(oracle, case, rows=rows, cols=cols)
    first = bits_from_dev(bufs[0])
    assert_close(oracle, first[np.ix_(rows, cols)], want, f"shard {r} of {tp_n}")
    assert (first[:, :lo] == 0x7FC0).all() and (first[:, hi:] == 0x7FC0).all()
    for b in bufs[1:]:
        assert np.array_equal(bits_from_dev(b), first)
    assert atlas.device_status() == 0


def test_push_columns_copies_the_block_and_nothing_else(cuda, atlas):
    """atlas_b200_push_columns: an [m, n_cols] block of a row-major buffer into the same columns of several others
    (local buffers stand in for the peers' gathered buffers), ragged chunk counts included."""
    torch = cuda
    for m, n_total, col0, n_cols in ((8192, 4096, 512, 512), (77, 1536, 1024, 264), (3, 64, 8, 8)):
        src = torch.randint(-30000, 30000, (m, n_total), dtype=torch.int16, device="cuda")
        dests = [torch.full((m, n_total), 0x7FC0, dtype=torch.int16, device="cuda") for _ in range(3)]
        atlas.push_columns(src.data_ptr() + col0 * 2, n_total, [d.data_ptr() + col0 * 2 for d in dests], n_total, m, n_cols)
        torch.cuda.synchronize()
        for d in dests:
            assert torch.equal(d[:, col0:col0 + n_cols], src[:, col0:col0 + n_cols])
            assert (d[:, :col0] == 0x7FC0).all() and (d[:, col0 + n_cols:] == 0x7FC0).all()
    # rules: 16-byte chunks only, at most 8 destinations
    src = torch.zeros((4, 64), dtype=torch.int16, device="cuda")
    dst = torch.zeros((4, 64), dtype=torch.int16, device="cuda")
    with pytest.raises(atlas.AtlasError):
        atlas.push_columns(src.data_ptr(), 64, [dst.data_ptr()], 64, 4, 12)
    with pytest.raises(atlas.AtlasError):
        atlas.push_columns(src.data_ptr() + 2, 64, [dst.data_ptr()], 64, 4, 8)
    with pytest.raises(atlas.AtlasError):
        atlas.push_columns(src.data_ptr(), 64, [dst.data_ptr()] * 9, 64, 4, 8)
