"""Host logic of the shared library and its exported surface (no GPU, no compute calls)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(atlas):
    header = open(os.path.join(ROOT, "include", "atlas_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(atlas_b200_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 19
    L = atlas.lib()
    for name in declared:
        assert hasattr(L, name), f"{name} declared in include/atlas_b200.h but not exported"
    assert sorted(atlas.EXPORTS) == declared
    assert b"sm_100a" in L.atlas_b200_version()


def test_linear_desc_layout_matches_header(atlas):
    # field order and natural alignment of the C struct
    d = atlas.LinearDesc
    assert d.x.offset == 0 and d.m.offset == 8 and d.k.offset == 12 and d.x_row_stride.offset == 16
    assert d.n.offset == 20 and d.w_packed.offset == 24 and d.w_bf16.offset == 40
    assert d.scale2.offset == 48 and d.flags.offset == 52 and d.seq_slot.offset == 56
    assert d.max_loras.offset == 96 and d.y.offset == 104 and d.lora_t.offset == 120
    assert d.b_pool_base.offset == 144 and d.b_slot_stride.offset == 152
    assert C.sizeof(d) == 248


def test_seq_slot_and_scaling_match_oracle(atlas, oracle):
    assert atlas.build_seq_slot_host([1, -1, 0], 4, 2) == [1, 2, 0, -1]
    rng = np.random.default_rng(1)
    for _ in range(20):
        n = int(rng.integers(0, 40))
        pad = n + int(rng.integers(0, 9))
        slots = rng.integers(-1, 6, size=n).tolist()
        active = int(rng.integers(0, 6))
        assert atlas.build_seq_slot_host(slots, pad, active) == oracle.build_seq_slot_host(slots, pad, active)
    assert atlas.build_seq_slot_host([], 3, 1) == [-1, -1, -1]
    with pytest.raises(atlas.AtlasError):
        atlas.build_seq_slot_host([0, 1, 2], 2, 0)                      # padded_n < n
    assert atlas.peft_scaling(32.0, 16) == 2.0 and atlas.peft_scaling(32.0, 16, True) == 8.0
    assert atlas.peft_scaling(16.5, 8) == float(np.float32(16.5 / 8))
    assert atlas.routed_prefill_slot_of(1, 0, 4) == 1
    assert atlas.routed_prefill_slot_of(-1, 0, 4) is None
    assert atlas.routed_prefill_slot_of(7, 0, 4) is None


def test_pool_layout_golden_and_walk(atlas):
    cfg = atlas.ModelDims(2048, 5120, 16, 2, 256, 1, 12)
    assert atlas.pool_slot_bytes(cfg, 16) == 16_515_072
    sb = atlas.pool_slot_bytes(cfg, 16)
    for k in range(8):
        assert atlas.slot_base_offset(k, cfg, 16) == k * sb
    off = 0
    for layer in range(12):
        for m in range(7):
            o, i = atlas.module_dims(cfg, m)
            assert atlas.module_slot_offsets(cfg, 16, layer, m) == (off, off + 16 * i * 2)
            off += (16 * i + o * 16) * 2
    assert off == sb
    assert atlas.module_slot_offsets(cfg, 16, 12, 0) is None
    assert atlas.module_dims(cfg, 0) == (8192, 2048)                     # gated q_proj is [Q|gate]
    assert atlas.module_dims(cfg, 3) == (2048, 4096)


def test_pack_module_matches_oracle_pack(atlas, oracle):
    cfg = atlas.ModelDims(64, 96, 2, 1, 16, 0, 2)
    max_rank, r = 16, 4
    img = np.full(atlas.pool_slot_bytes(cfg, max_rank), 0xAB, dtype=np.uint8)
    out_dim, in_dim = atlas.module_dims(cfg, 4)
    rng = np.random.default_rng(2)
    a = rng.integers(0, 65535, size=(r, in_dim), dtype=np.uint16)
    b = rng.integers(0, 65535, size=(out_dim, r), dtype=np.uint16)
    st = atlas.lib().atlas_b200_pack_module(C.byref(cfg), max_rank, 1, 4, a.ctypes.data, b.ctypes.data, r, img.ctypes.data)
    assert st == 0
    a_off, b_off = atlas.module_slot_offsets(cfg, max_rank, 1, 4)
    pool = oracle.HostPool(in_dim, out_dim, max_rank, 1)
    pool.pack(0, a, b, 1.0)
    got_a = img[a_off:a_off + max_rank * in_dim * 2].view(np.uint16).reshape(max_rank, in_dim)
    got_b = img[b_off:b_off + out_dim * max_rank * 2].view(np.uint16).reshape(out_dim, max_rank)
    assert np.array_equal(got_a, pool.a[0]) and np.array_equal(got_b, pool.b[0])
    assert not got_a[r:].any() and not got_b[:, r:].any()
    assert (img[:a_off] == 0xAB).all()                                    # neighbours untouched
    assert atlas.lib().atlas_b200_pack_module(C.byref(cfg), max_rank, 1, 4, a.ctypes.data, b.ctypes.data, 17, img.ctypes.data) == -5


def test_select_victim_slot_policy(atlas):
    # spark-model/src/lora/slot_math.rs:25-38: free first, then least recently used idle, never a busy slot
    assert atlas.select_victim_slot([(2, True, 0, 5), (3, False, 0, 0), (4, True, 0, 1)]) == 3
    assert atlas.select_victim_slot([(2, True, 0, 9), (3, True, 1, 1), (4, True, 0, 4)]) == 4
    assert atlas.select_victim_slot([(2, True, 1, 9), (3, True, 2, 1)]) is None
    assert atlas.select_victim_slot([]) is None


def test_column_shard(atlas):
    assert atlas.column_shard(28672, 8, 3) == (3 * 3584, 3584)
    assert atlas.column_shard(17408, 1, 0) == (0, 17408)
    with pytest.raises(atlas.AtlasError):
        atlas.column_shard(100, 8, 0)
    with pytest.raises(atlas.AtlasError):
        atlas.column_shard(64, 4, 4)


def test_launchers_validate_before_touching_the_device(atlas):
    L = atlas.lib()
    d = atlas.LinearDesc()
    assert L.atlas_b200_nvfp4_lora_linear(None, None) == -4
    assert L.atlas_b200_nvfp4_lora_linear(C.byref(d), None) == -4        # null x / y
    d.x, d.y, d.w_packed, d.w_scale = 16, 16, 16, 16
    d.m, d.k, d.n, d.x_row_stride, d.out_row_stride = 4, 24, 8, 24, 8
    assert L.atlas_b200_nvfp4_lora_linear(C.byref(d), None) == -1        # k not a multiple of 16
    d.k, d.x_row_stride = 32, 16
    assert L.atlas_b200_nvfp4_lora_linear(C.byref(d), None) == -1        # row stride shorter than k
    d.x_row_stride = 32
    d.seq_slot = 16
    assert L.atlas_b200_nvfp4_lora_linear(C.byref(d), None) == -4        # routing without tables
    d.a_table = d.b_table = d.scale_table = d.lora_t = 16
    assert L.atlas_b200_nvfp4_lora_linear(C.byref(d), None) == -1        # max_loras == 0
    d.max_loras, d.max_rank = 4, 512
    assert L.atlas_b200_nvfp4_lora_linear(C.byref(d), None) == -5        # rank beyond the limit
    assert L.atlas_b200_lora_bgmv(None, None, None, None, None, None, None, 4, 8, 8, 8, 8, 8, 2, None) == -4
    assert L.atlas_b200_lora_bgmv(None, None, None, None, None, None, None, 0, 8, 8, 8, 8, 8, 2, None) == 0
    assert L.atlas_b200_dequant_nvfp4_to_bf16(16, 16, 16, 1.0, 4, 24, None) == -1
