"""apply_lora_bgmv / apply_lora_delta through the C ABI against the staged oracle."""
import numpy as np
import pytest

from gpu_util import ATOL, RTOL, assert_close, bits_from_dev, device_pool, host_pool, to_dev

pytestmark = pytest.mark.gpu


def _run_bgmv(torch, atlas, oracle, case, x_stride=None, out_stride=None, seed=0):
    xs, os_ = x_stride or case.K, out_stride or case.N
    rng = np.random.default_rng(seed)
    base = oracle.f32_to_bf16(rng.standard_normal((case.M, os_)).astype(np.float32))
    xh = np.zeros((case.M, xs), dtype=np.uint16)
    xh[:, :case.K] = case.x
    pool = device_pool(torch, atlas, case)
    out = to_dev(torch, base)
    xa = torch.full((case.M, case.max_rank), 0x1234, dtype=torch.int16, device="cuda")
    atlas.apply_lora_bgmv(pool.route(), to_dev(torch, xh), out, to_dev(torch, case.seq_slot), case.M, xs, os_, xa)
    torch.cuda.synchronize()
    want = base.copy()
    want_xa = oracle.lora_bgmv_staged(xh, case.seq_slot, host_pool(oracle, case), want, case.M, xs, os_)
    return bits_from_dev(out), bits_from_dev(xa), want, want_xa, base


@pytest.mark.parametrize("M,K,N,ranks,max_rank,xs,os_", [
    (7, 1024, 512, [8, 16, 4], 16, None, None),
    (64, 4096, 1024, [8, 16, 32, 64] * 4, 64, None, None),
    (5, 264, 100, [3, 8], 8, 300, 160),            # odd sizes, strided x and out, unaligned rows
    (300, 512, 256, [16] * 5, 16, None, 384),      # more rows than one scan chunk
])
def test_bgmv_matches_staged_oracle(cuda, atlas, oracle, M, K, N, ranks, max_rank, xs, os_):
    from atlas_b200 import synth
    case = synth.make_case("bgmv", M=M, K=K, N=N, ranks=ranks, max_rank=max_rank, max_loras=len(ranks) + 2,
                           none_frac=0.2, b_std=0.3, seed=M)
    got, got_xa, want, want_xa, base = _run_bgmv(cuda, atlas, oracle, case, xs, os_)
    routed = case.seq_slot >= 0
    # routing is exact: un-routed rows keep their bytes, their xa rows are never written
    assert np.array_equal(got[~routed], base[~routed])
    assert (got_xa[~routed] == 0x1234).all()
    # columns beyond n_out are never touched
    assert np.array_equal(got[:, N:], base[:, N:])
    assert_close(oracle, got_xa[routed], oracle.bf16_to_f32(want_xa[routed]), "xa")
    assert_close(oracle, got[routed][:, :N], oracle.bf16_to_f32(want[routed][:, :N]), "out")
    for m in np.nonzero(routed)[0]:
        r = case.adapters[case.seq_slot[m]].rank
        assert not got_xa[m, r:].any()              # pad ranks are exact zeros
    assert atlas.device_status() == 0


def test_bgmv_null_table_entries_and_out_of_range_slot(cuda, atlas, oracle):
    torch = cuda
    from atlas_b200 import synth
    case = synth.make_case("bgmv", M=6, K=256, N=128, ranks=[8, 8], max_rank=8, max_loras=4, ids="distinct", b_std=0.3, seed=3)
    case.seq_slot = np.array([0, 1, 2, 3, 9, -1], dtype=np.int32)     # 2,3: resident but empty; 9: beyond the tables
    got, got_xa, want, want_xa, base = _run_bgmv(torch, atlas, oracle, case)
    assert np.array_equal(got[2:], base[2:])
    assert not np.array_equal(got[:2], base[:2])
    assert_close(oracle, got[:2], oracle.bf16_to_f32(want[:2]), "out")
    assert atlas.device_status() == 1                                   # the out-of-range slot was recorded
    assert atlas.device_status() == 0                                   # and the word cleared


@pytest.mark.parametrize("m", [1, 33])
def test_lora_delta_single_adapter(cuda, atlas, oracle, m):
    torch = cuda
    from atlas_b200 import synth
    K, N, r, max_rank = 1024, 512, 8, 64             # the reference microtest's default shape
    case = synth.make_case("delta", M=m, K=K, N=N, ranks=[r], max_rank=max_rank, b_std=0.3, seed=7)
    hp = host_pool(oracle, case)
    base = oracle.f32_to_bf16(np.random.default_rng(1).standard_normal((m, N)).astype(np.float32))
    want = base.copy()
    want_xa, want_delta = oracle.lora_delta_staged(case.x, hp.a[0], hp.b[0], 2.0, want, m, K, N, max_rank)
    out = to_dev(torch, base)
    xa = torch.zeros((m, max_rank), dtype=torch.int16, device="cuda")
    delta = torch.zeros((m, N), dtype=torch.int16, device="cuda")
    atlas.apply_lora_delta(to_dev(torch, hp.a[0]), to_dev(torch, hp.b[0]), 2.0, K, N, max_rank,
                           to_dev(torch, case.x), out, m, xa, delta)
    torch.cuda.synchronize()
    assert_close(oracle, bits_from_dev(xa), oracle.bf16_to_f32(want_xa), "xa")
    assert_close(oracle, bits_from_dev(delta), oracle.bf16_to_f32(want_delta), "delta")
    assert_close(oracle, bits_from_dev(out), oracle.bf16_to_f32(want), "out")
    # cosine gate of the reference's microtest (lora_apply_microtest.rs:29)
    g, w = oracle.bf16_to_f32(bits_from_dev(out)).ravel().astype(np.float64), oracle.bf16_to_f32(want).ravel().astype(np.float64)
    assert g @ w / (np.linalg.norm(g) * np.linalg.norm(w)) >= 0.999
