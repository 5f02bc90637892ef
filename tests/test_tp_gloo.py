"""Column-parallel sharding of the layer across ranks, on CPU with the gloo backend (world_size 2 and 4).

Each rank computes its shard with the oracle, the shards are all-gathered exactly as bench.py gathers the
GPU shards, and the re-assembled output must equal the unsharded oracle result bit for bit (the
contraction of one output column never crosses a shard)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_path):
    for p in (ROOT, os.path.join(ROOT, "apathy-atlas_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch
    import torch.distributed as dist
    from atlas_b200 import synth, tp
    from oracle import oracle_ctypes as oc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    case = synth.make_case("tp", M=24, K=256, N=512, ranks=[8, 16, 4, 16], max_rank=16, none_frac=0.25,
                           scale2=0.02, b_std=0.1, seed=4)
    local = tp.shard_case(case, world, rank)
    assert local.N == case.N // world and local.packed.shape[0] == local.N
    pool = oc.HostPool(local.K, local.N, local.max_rank, local.max_loras)
    for s, ad in enumerate(local.adapters):
        if ad is not None:
            pool.pack(s, ad.a, np.ascontiguousarray(ad.b), ad.scale)
    y_loc, _ = oc.reference_sequence(local.x, local.M, local.N, local.K, packed=np.ascontiguousarray(local.packed),
                                     scales=np.ascontiguousarray(local.scales), scale2=local.scale2,
                                     seq_slot=local.seq_slot, pool=pool)
    # bytes on the wire, as the reference's all_gather wrapper sends them (ncclUint8)
    y_loc_t = torch.from_numpy(y_loc.view(np.uint8).copy())
    y_all = torch.empty((world, local.M, local.N * 2), dtype=torch.uint8)
    dist.all_gather_into_tensor(y_all.view(world * local.M, local.N * 2), y_loc_t)
    if rank == 0:
        full_pool = oc.HostPool(case.K, case.N, case.max_rank, case.max_loras)
        for s, ad in enumerate(case.adapters):
            if ad is not None:
                full_pool.pack(s, ad.a, ad.b, ad.scale)
        want, _ = oc.reference_sequence(case.x, case.M, case.N, case.K, packed=case.packed, scales=case.scales,
                                        scale2=case.scale2, seq_slot=case.seq_slot, pool=full_pool)
        got = tp.gathered_to_row_major(y_all.numpy().view(np.uint16).reshape(world, local.M, local.N))
        np.save(out_path, np.array([int(np.array_equal(got, want)), int((want != 0).sum())]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_parallel_all_gather_reassembles_the_layer(world, tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "res.npy")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    res = np.load(out)
    assert res[0] == 1 and res[1] > 0


def test_shard_case_rejects_indivisible_n():
    sys.path.insert(0, os.path.join(ROOT, "apathy-atlas_b200"))
    from atlas_b200 import synth, tp
    case = synth.make_case("tp", M=4, K=64, N=96, ranks=[8], max_rank=8, seed=1)
    with pytest.raises(ValueError):
        tp.shard_case(case, 5, 0)
    y = np.arange(2 * 3 * 4, dtype=np.uint16).reshape(2, 3, 4)
    rm = tp.gathered_to_row_major(y)
    assert rm.shape == (3, 8) and list(rm[1]) == [4, 5, 6, 7, 16, 17, 18, 19]


def _shrink_worker(rank, world, port, out_path):
    """Token-sharded shrink: every rank computes t = A_s x for its own rows only and the rows are all-gathered; the
    result must equal the unsharded shrink bit for bit (a row's shrink does not depend on the other rows)."""
    for p in (ROOT, os.path.join(ROOT, "apathy-atlas_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch
    import torch.distributed as dist
    from atlas_b200 import synth, tp
    from oracle import oracle_ctypes as oc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M = 200                                                   # not a multiple of world * 64: the last rank gets a short share
    case = synth.make_case("tok", M=M, K=128, N=64, ranks=[8, 16, 4], max_rank=16, none_frac=0.2, scale2=0.02, seed=6)
    pool = oc.HostPool(case.K, case.N, case.max_rank, case.max_loras)
    for s, ad in enumerate(case.adapters):
        if ad is not None:
            pool.pack(s, ad.a, ad.b, ad.scale)
    begin, count = tp.token_shard(M, world, rank)
    per = tp.token_shard(M, world, 0)[1]
    mine = np.zeros((per, case.max_rank), dtype=np.uint16)
    if count:
        scratch = np.zeros((count, case.N), dtype=np.uint16)
        mine[:count] = oc.lora_bgmv_staged(np.ascontiguousarray(case.x[begin:begin + count]), case.seq_slot[begin:begin + count],
                                           pool, scratch, count)
    t_all = torch.empty((world, per, case.max_rank * 2), dtype=torch.uint8)
    dist.all_gather_into_tensor(t_all.view(world * per, case.max_rank * 2), torch.from_numpy(mine.view(np.uint8).copy()))
    if rank == 0:
        scratch = np.zeros((M, case.N), dtype=np.uint16)
        want = oc.lora_bgmv_staged(case.x, case.seq_slot, pool, scratch, M)
        got = t_all.numpy().view(np.uint16).reshape(world * per, case.max_rank)[:M]
        np.save(out_path, np.array([int(np.array_equal(got, want)), int((want != 0).sum())]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_token_sharded_shrink_reassembles(world, tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "res.npy")
    mp.spawn(_shrink_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    res = np.load(out)
    assert res[0] == 1 and res[1] > 0


def test_token_shard_ranges_tile_the_batch():
    sys.path.insert(0, os.path.join(ROOT, "apathy-atlas_b200"))
    from atlas_b200 import tp
    for M in (1, 63, 64, 65, 200, 8192, 8193):
        for world in (1, 2, 3, 4, 8):
            at = 0
            for r in range(world):
                b, c = tp.token_shard(M, world, r)
                assert b % 64 == 0 or c == 0
                assert b == min(at, M) and c >= 0
                at = b + c
            assert at == M
    with pytest.raises(ValueError):
        tp.token_shard(64, 2, 2)


def _swiglu_worker(rank, world, port, out_path):
    """Gathering what the consumer reads: SwiGLU applied by every rank to its own columns of gate and up and the results
    all-gathered must equal SwiGLU of the gathered gate and up (the op is element-wise and a rank owns the same columns of
    both), bit for bit after the BF16 rounding."""
    for p in (ROOT, os.path.join(ROOT, "apathy-atlas_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch
    import torch.distributed as dist
    from atlas_b200 import tp
    from oracle import oracle_ctypes as oc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, N = 24, 64 * world
    rng = np.random.default_rng(9)
    gate = oc.f32_to_bf16(rng.standard_normal((M, N)).astype(np.float32) * 3)
    up = oc.f32_to_bf16(rng.standard_normal((M, N)).astype(np.float32))
    n_loc = N // world
    lo = rank * n_loc
    h_loc = oc.f32_to_bf16(oc.silu_mul(np.ascontiguousarray(gate[:, lo:lo + n_loc]), np.ascontiguousarray(up[:, lo:lo + n_loc])))
    h_all = torch.empty((world, M, n_loc * 2), dtype=torch.uint8)
    dist.all_gather_into_tensor(h_all.view(world * M, n_loc * 2), torch.from_numpy(h_loc.view(np.uint8).copy()))
    if rank == 0:
        got = tp.gathered_to_row_major(h_all.numpy().view(np.uint16).reshape(world, M, n_loc))
        want = oc.f32_to_bf16(oc.silu_mul(gate, up))
        np.save(out_path, np.array([int(np.array_equal(got, want)), int((want != 0).sum())]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_swiglu_on_own_columns_then_gather_equals_swiglu_of_the_gathered(world, tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "res.npy")
    mp.spawn(_swiglu_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    res = np.load(out)
    assert res[0] == 1 and res[1] > 0
