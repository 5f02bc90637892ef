"""The multi-adapter LoRA pool as the reference lays it out, on the current CUDA device.

Mirror of `LoraWeights` as `load_lora_adapters_multi` leaves it (crates/spark-model/src/lora/loading.rs:242-389,
lora/types.rs:120-200): ONE device allocation of max_loras equal slots, slot k at byte offset
k * pool_slot_bytes; inside a slot the walk (adapted layer ascending) x (q,k,v,o,gate,up,down) x (A then B), A as
[max_rank, in], B as [out, max_rank], zero padded (lora/slot_math.rs:109-162); per (layer, module) one `[max_loras]`
u64 A table and B table (0 = slot not packed / module not adapted) and one `[max_loras]` f32 scale table shared by
all modules.  All layout arithmetic is done by the C library (atlas_b200_pool_slot_bytes, _module_slot_offsets,
_pack_module, _build_route_tables); torch only holds the bytes.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import numpy as np

from . import LoraRoute, ModelDims, MODULES, _check, lib, module_dims, pool_slot_bytes


def model_dims(hidden_size, intermediate_size, num_attention_heads, num_key_value_heads, head_dim, attn_gated=0,
               num_full_attention_layers=1) -> ModelDims:
    return ModelDims(hidden_size, intermediate_size, num_attention_heads, num_key_value_heads, head_dim, attn_gated,
                     num_full_attention_layers)


class LoraWeights:
    """Slot-major adapter pool plus its routing tables."""

    def __init__(self, cfg: ModelDims, max_loras: int, max_rank: int, device="cuda"):
        import torch
        self.torch, self.cfg, self.max_loras, self.max_rank = torch, cfg, max_loras, max_rank
        self.slot_bytes = pool_slot_bytes(cfg, max_rank)
        self.pool_bytes = self.slot_bytes * max_loras
        self.pool = torch.zeros(self.pool_bytes, dtype=torch.uint8, device=device)      # zeroed once: pads stay 0
        self.scale_host = np.zeros(max_loras, dtype=np.float32)
        self.rank_host = np.zeros(max_loras, dtype=np.uint32)
        self.scale_table = torch.zeros(max_loras, dtype=torch.float32, device=device)
        self.rank_table = torch.zeros(max_loras, dtype=torch.int32, device=device)
        # (layer ordinal, module) -> per-slot presence; device tables are built from it on demand
        self.present: Dict[Tuple[int, int], np.ndarray] = {}
        self._tables: Dict[Tuple[int, int, int], tuple] = {}

    # ---- packing -------------------------------------------------------------------------------
    def pack_slot(self, slot: int, modules: Dict[Tuple[int, int], Tuple[np.ndarray, np.ndarray]], scale: float) -> None:
        """`pack_slot` (loading.rs:128-230): `modules` maps (layer ordinal, module index) to PEFT-shaped
        (A [r, in], B [out, r]) BF16 bit arrays; modules the adapter omits stay zero / null."""
        assert 0 <= slot < self.max_loras
        image = np.zeros(self.slot_bytes, dtype=np.uint8)
        r_seen = None
        for (layer, module), (a, b) in modules.items():
            out_dim, in_dim = module_dims(self.cfg, module)
            r = a.shape[0]
            assert a.shape == (r, in_dim) and b.shape == (out_dim, r) and a.dtype == np.uint16 and b.dtype == np.uint16
            assert r_seen in (None, r), "one rank per adapter (uniform r)"
            r_seen = r
            a_c, b_c = np.ascontiguousarray(a), np.ascontiguousarray(b)
            _check("atlas_b200_pack_module", lib().atlas_b200_pack_module(
                C.byref(self.cfg), self.max_rank, layer, module, a_c.ctypes.data, b_c.ctypes.data, r, image.ctypes.data))
        lo = slot * self.slot_bytes
        self.pool[lo:lo + self.slot_bytes].copy_(self.torch.from_numpy(image))
        for key in list(self.present):
            self.present[key][slot] = 0
        for key in modules:
            self.present.setdefault(key, np.zeros(self.max_loras, dtype=np.uint8))[slot] = 1
        self.scale_host[slot] = np.float32(scale)
        self.rank_host[slot] = r_seen or 0
        self.scale_table.copy_(self.torch.from_numpy(self.scale_host))
        self.rank_table.copy_(self.torch.from_numpy(self.rank_host.view(np.int32)))
        self._tables.clear()

    # ---- tables --------------------------------------------------------------------------------
    def host_tables(self, layer: int, module: int, row_begin: int = 0):
        """The [max_loras] u64 A/B table images for (layer, module); `row_begin` offsets every B entry to output row
        row_begin of B_s (a column shard of the module: rows of B [out, max_rank] are contiguous)."""
        a = np.zeros(self.max_loras, dtype=np.uint64)
        b = np.zeros(self.max_loras, dtype=np.uint64)
        present = self.present.get((layer, module))
        if present is None:
            return a, b
        _check("atlas_b200_build_route_tables", lib().atlas_b200_build_route_tables(
            C.byref(self.cfg), self.max_rank, layer, module, self.pool.data_ptr(), self.max_loras,
            present.ctypes.data, a.ctypes.data, b.ctypes.data))
        if row_begin:
            b[b != 0] += np.uint64(row_begin * self.max_rank * 2)
        return a, b

    def route(self, layer: int, module: int, row_begin: int = 0, row_count: Optional[int] = None,
              with_ranks: bool = True, strided: bool = True) -> LoraRoute:
        """`LoraRoute` of (layer, module) — for the whole module, or for output rows [row_begin, row_begin + row_count)."""
        torch = self.torch
        out_dim, in_dim = module_dims(self.cfg, module)
        n = out_dim - row_begin if row_count is None else row_count
        key = (layer, module, row_begin)
        if key not in self._tables:
            a, b = self.host_tables(layer, module, row_begin)
            self._tables[key] = (torch.from_numpy(a.view(np.int64)).to(self.pool.device),
                                 torch.from_numpy(b.view(np.int64)).to(self.pool.device), b)
        a_dev, b_dev, b_host = self._tables[key]
        r = LoraRoute(a_dev, b_dev, self.scale_table, in_dim, n, self.max_rank, self.max_loras,
                      self.rank_table if with_ranks else None)
        if strided:
            # slot s's B of this module sits s * pool_slot_bytes after slot 0's (slot_math.rs:124-137)
            a0, b0 = np.zeros(1, np.uint64), np.zeros(1, np.uint64)
            _check("atlas_b200_build_route_tables", lib().atlas_b200_build_route_tables(
                C.byref(self.cfg), self.max_rank, layer, module, self.pool.data_ptr(), 1, None, a0.ctypes.data, b0.ctypes.data))
            r.b_pool_base, r.b_slot_stride = int(b0[0]) + row_begin * self.max_rank * 2, self.slot_bytes
            r.a_pool_base, r.a_slot_stride = int(a0[0]), self.slot_bytes
        return r

    def module_name(self, module: int) -> str:
        return MODULES[module]
