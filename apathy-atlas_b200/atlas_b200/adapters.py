"""Adapter ingest and the adapter registry: Python face of the C library's host-side LoRA registry.

Mirrors, by name and behaviour:
  parse_peft_adapter_config      crates/atlas-core/src/config/parsers/lora.rs:121-262
  classify_key, adapter_id_hash  crates/spark-model/src/lora/key.rs:33-113
  load_lora_adapters_multi       crates/spark-model/src/lora/loading.rs:242-389     (AdapterRegistry.load_adapters)
  pack_store_into_slot           crates/spark-model/src/lora/loading.rs:401-459     (AdapterRegistry.load_adapter on a filled slot)
  LoraWeights lifecycle          crates/spark-model/src/lora/types.rs:268-413
All parsing, auditing, packing and bookkeeping happens in the library; this module marshals arguments and — when a
torch device pool is attached — uploads the slot images and table images the library hands back.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np

from . import AtlasError, ModelDims, PeftConfig, _check, lib

ERR_REJECT, ERR_BUSY = -6, -7


class AdapterRejected(AtlasError):
    """The adapter cannot be applied faithfully; `reason` carries the named REJECT text."""

    def __init__(self, fn: str, status: int, reason: str):
        RuntimeError.__init__(self, f"{fn}: {reason}" if reason else f"{fn} failed with status {status}")
        self.status, self.reason = status, reason


def _call_with_message(fn_name: str, fn, *args):
    buf = C.create_string_buffer(1024)
    st = fn(*args, buf, len(buf))
    if st != 0:
        raise AdapterRejected(fn_name, st, buf.value.decode("utf-8", "replace"))


def parse_peft_adapter_config(text: str) -> dict:
    raw = text.encode("utf-8")
    cfg = PeftConfig()
    _call_with_message("atlas_b200_peft_parse", lib().atlas_b200_peft_parse, raw, len(raw), C.byref(cfg))
    return {"r": cfg.r, "lora_alpha": cfg.lora_alpha, "use_rslora": bool(cfg.use_rslora),
            "target_modules": [cfg.target_modules[i].value.decode() for i in range(cfg.n_target_modules)],
            "layers_to_transform": ([cfg.layers_to_transform[i] for i in range(cfg.n_layers_to_transform)]
                                    if cfg.has_layers_to_transform else None),
            "scaling": float(lib().atlas_b200_peft_config_scaling(C.byref(cfg)))}


def classify_key(key: str, num_hidden_layers: int, full_attention: Optional[Sequence[int]] = None):
    """-> (global layer index, module index 0..6 in q,k,v,o,gate,up,down order, 0 = lora_A / 1 = lora_B)."""
    fa = None if full_attention is None else np.ascontiguousarray(full_attention, dtype=np.uint8)
    layer, module, ab = C.c_uint32(), C.c_int(), C.c_int()
    _call_with_message("atlas_b200_classify_key", lib().atlas_b200_classify_key, key.encode(), num_hidden_layers,
                       None if fa is None else fa.ctypes.data, C.byref(layer), C.byref(module), C.byref(ab))
    return layer.value, module.value, ab.value


def adapter_id_hash(name: str, generation: int = 0) -> int:
    return int(lib().atlas_b200_adapter_id_hash(name.encode(), generation))


def convert_to_bf16(dtype: str, raw: np.ndarray) -> np.ndarray:
    """F16 / F32 / BF16 element bytes (any numpy array of that element size) -> BF16 bit patterns (uint16)."""
    src = np.ascontiguousarray(raw)
    out = np.empty(src.size, dtype=np.uint16)
    _check("atlas_b200_convert_to_bf16", lib().atlas_b200_convert_to_bf16(dtype.encode(), src.ctypes.data, src.size, out.ctypes.data))
    return out.reshape(src.shape)


class AdapterRegistry:
    """`LoraWeights` without kernels: resident adapters, their slot images, routing tables and lifecycle.

    With `device_pool` (a torch uint8 tensor of pool_bytes on the GPU) loads upload the packed slot and refresh the
    device tables; without it the registry is host-only (pool_base is then just a number the tables are built from)."""

    def __init__(self, cfg: ModelDims, num_hidden_layers: int, full_attention: Optional[Sequence[int]], max_loras: int,
                 max_rank: int, pool_base: int = 0, device_pool=None):
        self.cfg, self.max_loras, self.max_rank = cfg, max_loras, max_rank
        self.num_hidden_layers = num_hidden_layers
        fa = None if full_attention is None else np.ascontiguousarray(full_attention, dtype=np.uint8)
        self._fa = fa
        self.device_pool = device_pool
        if device_pool is not None:
            pool_base = device_pool.data_ptr()
        h = C.c_void_p()
        _check("atlas_b200_registry_create", lib().atlas_b200_registry_create(
            C.byref(cfg), num_hidden_layers, None if fa is None else fa.ctypes.data, max_loras, max_rank, pool_base, C.byref(h)))
        self._h = h
        self.slot_bytes = lib().atlas_b200_registry_slot_bytes(h)
        self.pool_bytes = lib().atlas_b200_registry_pool_bytes(h)
        self.pool_base = pool_base
        if device_pool is not None:
            assert device_pool.numel() >= self.pool_bytes

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib().atlas_b200_registry_destroy(h)

    # ---- loading ---------------------------------------------------------------------------------
    def load_adapter(self, slot: int, name: str, config_json: str, safetensors_bytes: bytes) -> np.ndarray:
        """Audit + pack into `slot`; returns the slot's byte image (and uploads it when a device pool is attached)."""
        image = np.zeros(self.slot_bytes, dtype=np.uint8)
        cj = config_json.encode("utf-8")
        _call_with_message("atlas_b200_registry_load_adapter", lib().atlas_b200_registry_load_adapter, self._h, slot,
                           name.encode(), cj, len(cj), safetensors_bytes, len(safetensors_bytes), image.ctypes.data)
        if self.device_pool is not None:
            import torch
            lo = slot * self.slot_bytes
            self.device_pool[lo:lo + self.slot_bytes].copy_(torch.from_numpy(image))
        return image

    def load_adapter_dir(self, slot: int, name: str, adapter_dir: str) -> np.ndarray:
        """`load_adapter_safetensors` + pack: reads adapter_config.json and adapter_model.safetensors from a PEFT directory."""
        st = os.path.join(adapter_dir, "adapter_model.safetensors")
        if not os.path.exists(st):
            if os.path.exists(os.path.join(adapter_dir, "adapter_model.bin")):
                raise AdapterRejected("load_adapter_dir", ERR_REJECT, f"REJECT[pickle-adapter]: {adapter_dir} ships adapter_model.bin "
                                      "(torch pickle); re-save with safe_serialization=True")
            raise FileNotFoundError(f"No adapter_model.safetensors in {adapter_dir}")
        with open(os.path.join(adapter_dir, "adapter_config.json"), "r", encoding="utf-8") as f:
            cfg = f.read()
        with open(st, "rb") as f:
            raw = f.read()
        return self.load_adapter(slot, name, cfg, raw)

    def load_adapters(self, adapters: Sequence[tuple]) -> None:
        """`load_lora_adapters_multi`: (name, config_json, safetensors_bytes) per adapter into slots 0..n-1, which become
        the pinned set; the remaining slots are the promotion cache."""
        if not adapters:
            raise AdapterRejected("load_adapters", ERR_REJECT, "REJECT[no-adapters]: load_lora_adapters_multi called with an empty set")
        if len(adapters) > self.max_loras:
            raise AdapterRejected("load_adapters", ERR_REJECT, f"REJECT[too-many-adapters]: {len(adapters)} --lora-adapter given but "
                                  f"--max-loras={self.max_loras} (pool has {self.max_loras} slots)")
        for k, (name, cfg, raw) in enumerate(adapters):
            self.load_adapter(k, name, cfg, raw)
        self.set_pinned(len(adapters))
        self.set_active(0)

    def set_pinned(self, pinned: int) -> None:
        _check("atlas_b200_registry_set_pinned", lib().atlas_b200_registry_set_pinned(self._h, pinned))

    def set_active(self, slot: int) -> None:
        _check("atlas_b200_registry_set_active", lib().atlas_b200_registry_set_active(self._h, slot))

    # ---- tables ----------------------------------------------------------------------------------
    def route_tables(self, layer: int, module: int):
        a = np.zeros(self.max_loras, dtype=np.uint64)
        b = np.zeros(self.max_loras, dtype=np.uint64)
        _check("atlas_b200_registry_route_tables", lib().atlas_b200_registry_route_tables(self._h, layer, module, a.ctypes.data, b.ctypes.data))
        return a, b

    def scale_table(self) -> np.ndarray:
        out = np.zeros(self.max_loras, dtype=np.float32)
        _check("atlas_b200_registry_scale_table", lib().atlas_b200_registry_scale_table(self._h, out.ctypes.data))
        return out

    def rank_table(self) -> np.ndarray:
        out = np.zeros(self.max_loras, dtype=np.uint32)
        _check("atlas_b200_registry_rank_table", lib().atlas_b200_registry_rank_table(self._h, out.ctypes.data))
        return out

    def route(self, layer: int, module: int, with_ranks: bool = True):
        """Device `LoraRoute` of (global layer, module) over the attached pool (tables uploaded now)."""
        import torch
        from . import LoraRoute, module_dims
        assert self.device_pool is not None
        a, b = self.route_tables(layer, module)
        dev = self.device_pool.device
        out_dim, in_dim = module_dims(self.cfg, module)
        r = LoraRoute(torch.from_numpy(a.view(np.int64)).to(dev), torch.from_numpy(b.view(np.int64)).to(dev),
                      torch.from_numpy(self.scale_table()).to(dev), in_dim, out_dim, self.max_rank, self.max_loras,
                      torch.from_numpy(self.rank_table().view(np.int32)).to(dev) if with_ranks else None)
        # slot s of this module's A / B sits s * slot_bytes after slot 0's
        a0 = np.zeros(1, np.uint64); b0 = np.zeros(1, np.uint64)
        ordinal = int(np.cumsum(self._fa)[layer] - 1) if self._fa is not None else layer
        _check("atlas_b200_build_route_tables", lib().atlas_b200_build_route_tables(
            C.byref(self.cfg), self.max_rank, ordinal, module, self.pool_base, 1, None, a0.ctypes.data, b0.ctypes.data))
        r.a_pool_base, r.a_slot_stride = int(a0[0]), self.slot_bytes
        r.b_pool_base, r.b_slot_stride = int(b0[0]), self.slot_bytes
        return r

    # ---- lifecycle -------------------------------------------------------------------------------
    def acquire_slot(self, slot: int) -> int:
        return lib().atlas_b200_registry_acquire_slot(self._h, slot)

    def release_slot(self, resolved: int) -> None:
        lib().atlas_b200_registry_release_slot(self._h, resolved)

    def touch_slot(self, slot: int) -> None:
        lib().atlas_b200_registry_touch_slot(self._h, slot)

    def slot_ref_count(self, slot: int) -> int:
        return lib().atlas_b200_registry_slot_ref_count(self._h, slot)

    def slot_last_used(self, slot: int) -> int:
        return lib().atlas_b200_registry_slot_last_used(self._h, slot)

    def slot_generation(self, slot: int) -> int:
        return lib().atlas_b200_registry_slot_generation(self._h, slot)

    def slot_of(self, name: str) -> Optional[int]:
        r = lib().atlas_b200_registry_slot_of(self._h, name.encode())
        return None if r < 0 else r

    def adapter_id_for_slot(self, slot: int) -> int:
        return int(lib().atlas_b200_registry_adapter_id_for_slot(self._h, slot))

    def select_victim(self) -> Optional[int]:
        r = lib().atlas_b200_registry_select_victim(self._h)
        return None if r < 0 else r
