"""The benchmark's layer workloads as the bench runs them — every projection of the layer over ONE slot-major adapter
pool in the reference's layout (crates/spark-model/src/lora/slot_math.rs:109-162), one fused call per projection —
each sampled against the oracle on at least 4096 outputs: rows on both sides of segment boundaries plus random rows,
random columns.  The whole tensors are covered by "every element written" (the buffers start as NaN patterns)."""
import numpy as np
import pytest

from gpu_util import assert_close, bits_from_dev, ideal

pytestmark = pytest.mark.gpu

N_ROWS, N_COLS = 64, 64            # 4096 oracle outputs per projection


def _rows_cols(case, seed):
    rng = np.random.default_rng(seed)
    cuts = np.flatnonzero(np.diff(case.seq_slot) != 0)[:16]
    rows = np.unique(np.concatenate([cuts, cuts + 1])).astype(np.int64)
    rest = np.setdiff1d(np.arange(case.M), rows)
    need = min(N_ROWS, case.M) - len(rows)
    if need > 0:
        rows = np.concatenate([rows, rng.choice(rest, need, replace=False)])
    rows = np.sort(rows[:N_ROWS]).astype(np.uint32)
    cols = np.sort(rng.choice(case.N, N_COLS, replace=False)).astype(np.uint32)
    assert len(rows) * len(cols) >= 4096
    return rows, cols


def _nan_buffer(torch, m, n):
    return torch.full((m, n), np.int16(np.uint16(0x7FC0).view(np.int16)), dtype=torch.int16, device="cuda")


def _run(torch, atlas, dl, i, flags=0):
    c = dl.proj[i]["case"]
    y = _nan_buffer(torch, c.M, c.N)
    variant = atlas.nvfp4_lora_linear(dl.desc(i, y, extra_flags=flags))
    torch.cuda.synchronize()
    assert variant == atlas.VARIANT_TCGEN05
    assert atlas.device_status() == 0
    return bits_from_dev(y)


@pytest.fixture(scope="module")
def layer3(cuda, atlas):
    from atlas_b200 import synth, tp
    layer = synth.layer_config(3)
    return layer, tp.DeviceLayer(cuda, atlas, layer)


def test_config3_layer_every_projection(cuda, atlas, oracle, layer3):
    """Llama-3-8B layer: q, k, v, o, gate, up, down (K = 14336) at 8192 tokens, 8 adapters of rank 64 in segments."""
    layer, dl = layer3
    assert [c.name.split("/")[-1] for c in layer.projections] == ["q", "k", "v", "o", "gate", "up", "down"]
    for i, c in enumerate(layer.projections):
        y = _run(cuda, atlas, dl, i)
        shape = atlas.last_launch_shape()
        assert shape["persistent_cta_pairs"] > 0 and shape["lora_tiles_from_shrink"], c.name
        rows, cols = _rows_cols(c, 100 + i)
        assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, c, rows=rows, cols=cols), c.name)
        assert np.isfinite(oracle.bf16_to_f32(y)).all(), c.name


@pytest.mark.parametrize("name", ["gate", "down"])
def test_config3_layer_fp4_activations(cuda, atlas, oracle, layer3, name):
    """The W4A4 arm on the widest and the deepest projection, against the oracle's quantised-activation mode."""
    layer, dl = layer3
    i = [c.name.split("/")[-1] for c in layer.projections].index(name)
    c = layer.projections[i]
    y = _run(cuda, atlas, dl, i, flags=atlas.FLAG_ACT_FP4)
    rows, cols = _rows_cols(c, 200 + i)
    assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, c, rows=rows, cols=cols, act_fp4=True), c.name + " A4")
    assert np.isfinite(oracle.bf16_to_f32(y)).all()


def test_config4_mlp_every_projection(cuda, atlas, oracle):
    """70B-class MLP: gate, up (K = 8192, N = 28672) and down (K = 28672, N = 8192); 512 tokens, 128 adapters of rank
    16 with Zipf ids, a quarter of the rows adapter-less."""
    from atlas_b200 import synth, tp
    layer = synth.layer_config(4)
    dl = tp.DeviceLayer(cuda, atlas, layer)
    assert [(c.K, c.N) for c in layer.projections] == [(8192, 28672), (8192, 28672), (28672, 8192)]
    for i, c in enumerate(layer.projections):
        y = _run(cuda, atlas, dl, i)
        rows, cols = _rows_cols(c, 300 + i)
        assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, c, rows=rows, cols=cols), c.name)
        assert np.isfinite(oracle.bf16_to_f32(y)).all(), c.name
        # adapter-less rows equal the base-only call bit for bit
        yb = _nan_buffer(cuda, c.M, c.N)
        d = dl.desc(i, yb)
        d.seq_slot = None
        atlas.nvfp4_lora_linear(d)
        cuda.cuda.synchronize()
        none = c.seq_slot < 0
        assert none.sum() > 64 and np.array_equal(y[none], bits_from_dev(yb)[none]), c.name
    # down once more with FP4 activations (K = 28672: 112 raw stages per tile)
    c = layer.projections[2]
    y = _run(cuda, atlas, dl, 2, flags=atlas.FLAG_ACT_FP4)
    rows, cols = _rows_cols(c, 310)
    assert_close(oracle, y[np.ix_(rows, cols)], ideal(oracle, c, rows=rows, cols=cols, act_fp4=True), c.name + " A4")


def test_config2_three_modules_into_one_strided_qkv_buffer(cuda, atlas, oracle):
    """Decode batch: q (4096), k (1024), v (1024) as three LoRA modules written into column ranges of one
    [64, 6144] buffer (out_row_stride = 6144), 64 distinct adapters of ranks 8..64."""
    from atlas_b200 import synth, tp
    layer = synth.layer_config(2)
    dl = tp.DeviceLayer(cuda, atlas, layer)
    widths = [c.N for c in layer.projections]
    assert widths == [4096, 1024, 1024]
    total = sum(widths)
    y = _nan_buffer(cuda, layer.M, total + 64)                 # 64 guard columns past the last module
    stride = total + 64
    col0 = 0
    for i, c in enumerate(layer.projections):
        variant = atlas.nvfp4_lora_linear(dl.desc(i, y[:, col0:], out_row_stride=stride))
        assert variant == atlas.VARIANT_TCGEN05
        col0 += c.N
    cuda.cuda.synchronize()
    assert atlas.device_status() == 0
    yb = bits_from_dev(y)
    assert (yb[:, total:] == 0x7FC0).all()                     # nothing written past the three modules
    col0 = 0
    for i, c in enumerate(layer.projections):
        rows = np.arange(c.M, dtype=np.uint32)
        cols = np.sort(np.random.default_rng(400 + i).choice(c.N, N_COLS, replace=False)).astype(np.uint32)
        got = yb[:, col0:col0 + c.N]
        assert_close(oracle, got[np.ix_(rows, cols)], ideal(oracle, c, rows=rows, cols=cols), c.name)
        assert np.isfinite(oracle.bf16_to_f32(np.ascontiguousarray(got))).all(), c.name
        col0 += c.N
