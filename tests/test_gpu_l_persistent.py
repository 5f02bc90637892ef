"""The persistent form of the tcgen05 kernel (many output tiles per SM pair): same bits as the one-tile-per-CTA form,
for BF16 and FP4 activations, with and without LoRA, ragged edges, one and two token tiles per pass, and placement
into several destination buffers; and within the path's tolerance of the oracle."""
import numpy as np
import pytest

from gpu_util import DeviceCase, assert_close, bits_from_dev, ideal

pytestmark = pytest.mark.gpu


def _case(synth, M, K, N, seed, ids="uniform", segments=0):
    return synth.make_case("persist", M=M, K=K, N=N, ranks=[16, 64, 32, 8, 64, 48], max_rank=64, max_loras=8, ids=ids,
                           segments=segments, none_frac=0.15, scale2=0.02, b_std=0.1, seed=seed)


def _sample(case, n_rows, n_cols, seed):
    rng = np.random.default_rng(seed)
    rows = np.sort(rng.choice(case.M, n_rows, replace=False)).astype(np.uint32)
    cols = np.sort(rng.choice(case.N, n_cols, replace=False)).astype(np.uint32)
    return rows, cols


@pytest.mark.parametrize("fp4", [False, True])
@pytest.mark.parametrize("M,K,N,ids", [(2048, 512, 4864, "uniform"), (2085, 768, 4992, "segments"), (4096, 256, 2560, "segments")])
def test_same_bits_as_one_tile_per_cta(cuda, atlas, oracle, M, K, N, ids, fp4):
    from atlas_b200 import synth
    case = _case(synth, M, K, N, seed=M + N, ids=ids, segments=24)
    dc = DeviceCase(cuda, atlas, case)
    mode = atlas.FLAG_ACT_FP4 if fp4 else 0
    y, variant = dc.run(flags=mode | atlas.FLAG_ONE_TILE_PASS, lora_ws=True)
    assert variant == atlas.VARIANT_TCGEN05
    shape = atlas.last_launch_shape()
    assert shape["persistent_tiles_per_pass"] == 1 and shape["persistent_cta_pairs"] >= 32, shape
    y_one, _ = dc.run(flags=mode | atlas.FLAG_NO_PERSISTENT, lora_ws=True)
    assert atlas.last_launch_shape()["persistent_tiles_per_pass"] == 0
    assert np.array_equal(y, y_one)
    rows, cols = _sample(case, 48, 96, M)
    assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, case, rows=rows, cols=cols, act_fp4=fp4), "persistent sample")
    assert atlas.device_status() == 0


def test_base_only_and_second_call(cuda, atlas, oracle):
    """No LoRA operands at all; and the kernel leaves nothing behind that a second launch could trip over."""
    from atlas_b200 import synth
    case = _case(synth, 2304, 512, 4864, seed=5)
    dc = DeviceCase(cuda, atlas, case)
    y, _ = dc.run(lora=False)
    assert atlas.last_launch_shape()["persistent_tiles_per_pass"] == 2
    y2, _ = dc.run(lora=False)
    y_one, _ = dc.run(lora=False, flags=atlas.FLAG_NO_PERSISTENT)
    assert np.array_equal(y, y2) and np.array_equal(y, y_one)
    rows, cols = _sample(case, 32, 64, 7)
    assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, case, rows=rows, cols=cols, lora=False), "base only")
    assert atlas.device_status() == 0


@pytest.mark.parametrize("M,K,N", [(3072, 512, 9728), (3100, 256, 9600)])
def test_two_token_tiles_per_pass(cuda, atlas, oracle, M, K, N):
    """Passes of two 192-token tiles sharing each expanded weight stage: a token's bits do not depend on the tiling."""
    from atlas_b200 import synth
    case = _case(synth, M, K, N, seed=M, ids="segments", segments=20)
    dc = DeviceCase(cuda, atlas, case)
    y2, _ = dc.run(lora_ws=True)
    shape = atlas.last_launch_shape()
    assert shape["persistent_tiles_per_pass"] == 2 and shape["token_tile"] == 192, shape
    y1, _ = dc.run(flags=atlas.FLAG_ONE_TILE_PASS, lora_ws=True)
    assert atlas.last_launch_shape()["persistent_tiles_per_pass"] == 1
    assert np.array_equal(y2, y1)
    y_one, _ = dc.run(flags=atlas.FLAG_NO_PERSISTENT, lora_ws=True)
    assert np.array_equal(y2, y_one)
    assert atlas.device_status() == 0


def test_without_tile_scratch_the_one_tile_form_runs(cuda, atlas, oracle):
    """The persistent form needs the shrink's masked-t tiles; without scratch for them the call still succeeds."""
    from atlas_b200 import synth
    case = _case(synth, 2048, 256, 4864, seed=11)
    dc = DeviceCase(cuda, atlas, case)
    y, _ = dc.run(lora_ws=False)
    assert atlas.last_launch_shape()["persistent_tiles_per_pass"] == 0
    y_p, _ = dc.run(lora_ws=True)
    assert atlas.last_launch_shape()["persistent_tiles_per_pass"] == 2
    assert np.array_equal(y, y_p)
    assert atlas.device_status() == 0


@pytest.mark.parametrize("fp4", [False, True])
def test_placement_into_several_buffers(cuda, atlas, oracle, fp4):
    """A column shard that is large enough for the persistent form stores its tiles into every rank's gathered buffer."""
    from atlas_b200 import synth, tp as tpmod
    M, K, N, tp = 2048, 256, 9728, 2
    case = _case(synth, M, K, N, seed=3)
    mode = atlas.FLAG_ACT_FP4 if fp4 else 0
    whole = tpmod.DeviceShard(cuda, atlas, case, 1, 0)
    y_ref = cuda.empty((M, N), dtype=cuda.bfloat16, device="cuda")
    atlas.nvfp4_lora_linear(whole.desc(y_ref, extra_flags=mode | atlas.FLAG_NO_PERSISTENT))
    stride = N + 8
    bufs = [cuda.full((M, stride), 0x7FC0, dtype=cuda.int16, device="cuda") for _ in range(tp)]
    for r in range(tp):
        sh = tpmod.DeviceShard(cuda, atlas, case, tp, r)
        atlas.nvfp4_lora_linear(sh.desc(None, extra_flags=mode, out_row_stride=stride, y_dest=bufs, y_col_offset=r * sh.n_local))
        assert atlas.last_launch_shape()["persistent_tiles_per_pass"] == (1 if fp4 else 2)
    cuda.cuda.synchronize()
    want = bits_from_dev(y_ref.view(cuda.int16))
    for b in bufs:
        got = bits_from_dev(b)
        assert np.array_equal(got[:, :N], want)
        assert (got[:, N:] == 0x7FC0).all()
    assert atlas.device_status() == 0
