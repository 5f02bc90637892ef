"""ctypes bindings of libatlas_b200.so and the host-side mirror of the reference's LoRA operator surface.

The compute lives in the shared library (CUDA for sm_100a behind a C ABI, see include/atlas_b200.h).
This module only marshals arguments: torch is used for device memory and streams, never for math.
There is no fallback: if the library is missing, or a call returns a non-zero status, an exception
is raised.

Mirrors, by name and argument meaning:
  LoraRoute          crates/spark-model/src/layers/ops/lora_delta.rs:51-58
  apply_lora_bgmv    crates/spark-model/src/layers/ops/lora_delta.rs:269-314
  apply_lora_delta   crates/spark-model/src/layers/ops/lora_delta.rs:145-235
  w4a16_gemm         crates/spark-model/src/layers/ops/gemm_dense.rs:258-281
  LoraPool           crates/spark-model/src/lora/loading.rs:242-389 (pool + per-module tables)
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libatlas_b200.so")

VARIANT_NONE, VARIANT_SIMT, VARIANT_TCGEN05 = 0, 1, 2
FLAG_FORCE_SIMT, FLAG_FORCE_TCGEN05, FLAG_STAGED_LORA, FLAG_REUSE_SHRINK, FLAG_ACT_FP4, FLAG_NO_CTA_PAIR, FLAG_NO_K_SPLIT = 1, 2, 4, 8, 16, 32, 64
FLAG_NO_PERSISTENT, FLAG_ONE_TILE_PASS, FLAG_ACT_FP4_READY = 128, 256, 512


def lora_ws_bytes(m: int, max_loras: int, max_rank: int) -> int:
    """Scratch that lets the shrink hand the LoRA K-steps' activation tiles to the fused kernel (ATLAS_B200_LORA_WS_BYTES)."""
    return ((m + 255) // 256 * 256 + 256) * min(max_loras, 256) * ((max_rank + 15) // 16) * 32


def act_fp4_ws_bytes(m: int, k: int) -> int:
    """Scratch a FLAG_ACT_FP4 call needs in `ws` (ATLAS_B200_ACT_FP4_WS_BYTES): packed codes, then scale bytes."""
    return (m * (k // 2) + 255) // 256 * 256 + m * (k // 16)
MODULES = ("q", "k", "v", "o", "gate", "up", "down")

EXPORTS = (
    "atlas_b200_lora_bgmv", "atlas_b200_lora_delta", "atlas_b200_w4a16_gemm",
    "atlas_b200_dequant_nvfp4_to_bf16", "atlas_b200_quantize_bf16_to_nvfp4", "atlas_b200_nvfp4_global_absmax",
    "atlas_b200_nvfp4_scale2_from_absmax", "atlas_b200_nvfp4_combined_global_scale", "atlas_b200_silu_mul",
    "atlas_b200_silu_mul_quant_nvfp4", "atlas_b200_kv_norm_rope_cache_write", "atlas_b200_kv_norm_mrope_cache_write", "atlas_b200_k_norm_rope_cache_write_fp8", "atlas_b200_qkv_norm_rope_cache_write",
    "atlas_b200_nvfp4_lora_linear", "atlas_b200_nvfp4_lora_linear_noalloc", "atlas_b200_lora_shrink_tiles",
    "atlas_b200_push_columns", "atlas_b200_copy_columns", "atlas_b200_selftest_bounded_wait", "atlas_b200_column_shard",
    "atlas_b200_build_seq_slot", "atlas_b200_routed_prefill_slot_of", "atlas_b200_peft_scaling",
    "atlas_b200_module_dims", "atlas_b200_pool_slot_bytes", "atlas_b200_slot_base_offset",
    "atlas_b200_module_slot_offsets", "atlas_b200_pack_module", "atlas_b200_build_route_tables", "atlas_b200_select_victim_slot",
    "atlas_b200_device_status", "atlas_b200_last_variant", "atlas_b200_last_launch_shape", "atlas_b200_last_persistent_shape",
    "atlas_b200_set_profile_buffer", "atlas_b200_peft_parse", "atlas_b200_peft_config_scaling", "atlas_b200_classify_key",
    "atlas_b200_adapter_id_hash", "atlas_b200_convert_to_bf16", "atlas_b200_registry_create", "atlas_b200_registry_destroy",
    "atlas_b200_registry_slot_bytes", "atlas_b200_registry_pool_bytes", "atlas_b200_registry_load_adapter",
    "atlas_b200_registry_set_pinned", "atlas_b200_registry_set_active", "atlas_b200_registry_route_tables",
    "atlas_b200_registry_scale_table", "atlas_b200_registry_rank_table", "atlas_b200_registry_acquire_slot",
    "atlas_b200_registry_release_slot", "atlas_b200_registry_touch_slot", "atlas_b200_registry_slot_ref_count",
    "atlas_b200_registry_slot_last_used", "atlas_b200_registry_slot_generation", "atlas_b200_registry_slot_of",
    "atlas_b200_registry_adapter_id_for_slot", "atlas_b200_registry_select_victim",
    "atlas_b200_version",
)


class AtlasError(RuntimeError):
    def __init__(self, fn: str, status: int):
        super().__init__(f"{fn} failed with status {status}")
        self.status = status


class LinearDesc(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("m", C.c_uint32), ("k", C.c_uint32), ("x_row_stride", C.c_uint32),
        ("n", C.c_uint32),
        ("w_packed", C.c_void_p), ("w_scale", C.c_void_p), ("w_bf16", C.c_void_p),
        ("scale2", C.c_float), ("flags", C.c_uint32),
        ("seq_slot", C.c_void_p), ("a_table", C.c_void_p), ("b_table", C.c_void_p),
        ("scale_table", C.c_void_p), ("rank_table", C.c_void_p),
        ("max_loras", C.c_uint32), ("max_rank", C.c_uint32),
        ("y", C.c_void_p), ("out_row_stride", C.c_uint32), ("reserved0", C.c_uint32),
        ("lora_t", C.c_void_p), ("ws", C.c_void_p), ("ws_bytes", C.c_size_t),
        ("b_pool_base", C.c_void_p), ("b_slot_stride", C.c_size_t),
        ("n_dest", C.c_uint32), ("y_col_offset", C.c_uint32), ("y_dest", C.c_void_p * 8),
        ("a_pool_base", C.c_void_p), ("a_slot_stride", C.c_size_t),
    ]


class PeftConfig(C.Structure):
    _fields_ = [("r", C.c_size_t), ("lora_alpha", C.c_double), ("use_rslora", C.c_int32), ("n_target_modules", C.c_uint32),
                ("target_modules", (C.c_char * 96) * 16), ("has_layers_to_transform", C.c_int32),
                ("n_layers_to_transform", C.c_uint32), ("layers_to_transform", C.c_uint32 * 256)]


class ModelDims(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads", "head_dim",
        "attn_gated", "num_full_attention_layers")]


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.dirname(os.path.dirname(LIB_PATH))}` "
            "(there is no non-CUDA fallback)")
    L = C.CDLL(LIB_PATH)
    u32, vp, f32, i32, sz = C.c_uint32, C.c_void_p, C.c_float, C.c_int32, C.c_size_t
    L.atlas_b200_lora_bgmv.argtypes = [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, vp]
    L.atlas_b200_lora_delta.argtypes = [vp, vp, vp, f32, vp, vp, vp, u32, u32, u32, u32, vp]
    L.atlas_b200_w4a16_gemm.argtypes = [vp, vp, vp, f32, vp, u32, u32, u32, vp, sz, vp]
    L.atlas_b200_dequant_nvfp4_to_bf16.argtypes = [vp, vp, vp, f32, u32, u32, vp]
    L.atlas_b200_quantize_bf16_to_nvfp4.argtypes = [vp, vp, vp, f32, u32, u32, vp]
    L.atlas_b200_nvfp4_lora_linear.argtypes = [C.POINTER(LinearDesc), vp]
    L.atlas_b200_nvfp4_global_absmax.argtypes = [vp, vp, sz, vp]
    L.atlas_b200_nvfp4_scale2_from_absmax.argtypes, L.atlas_b200_nvfp4_scale2_from_absmax.restype = [f32], f32
    L.atlas_b200_nvfp4_combined_global_scale.argtypes, L.atlas_b200_nvfp4_combined_global_scale.restype = [f32, C.c_int], f32
    L.atlas_b200_silu_mul.argtypes = [vp, vp, vp, f32, f32, f32, u32, u32, u32, u32, vp]
    L.atlas_b200_silu_mul_quant_nvfp4.argtypes = [vp, vp, vp, sz, f32, f32, f32, u32, u32, u32, vp]
    L.atlas_b200_nvfp4_lora_linear_noalloc.argtypes = [C.POINTER(LinearDesc), vp]
    L.atlas_b200_kv_norm_rope_cache_write.argtypes = [vp, vp, u32, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, f32, f32, vp]
    L.atlas_b200_kv_norm_mrope_cache_write.argtypes = [vp, vp, u32, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, f32, f32, vp]
    L.atlas_b200_k_norm_rope_cache_write_fp8.argtypes = [vp, u32, vp, vp, vp, vp, u32, u32, u32, u32, u32, f32, f32, f32, vp]
    L.atlas_b200_qkv_norm_rope_cache_write.argtypes = [vp, vp, vp, u32, u32, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, f32,
                                                       C.c_int, vp]
    L.atlas_b200_lora_shrink_tiles.argtypes = [C.POINTER(LinearDesc), u32, u32, C.POINTER(vp), u32, vp]
    L.atlas_b200_push_columns.argtypes = [vp, u32, C.POINTER(vp), u32, u32, u32, u32, vp]
    L.atlas_b200_copy_columns.argtypes = [vp, u32, C.POINTER(vp), u32, u32, u32, u32, vp]
    L.atlas_b200_selftest_bounded_wait.argtypes = [C.c_uint64, C.POINTER(u32)]
    L.atlas_b200_column_shard.argtypes = [u32, u32, u32, C.POINTER(u32), C.POINTER(u32)]
    L.atlas_b200_build_seq_slot.argtypes = [C.POINTER(i32), sz, sz, i32, C.POINTER(i32)]
    L.atlas_b200_routed_prefill_slot_of.argtypes = [i32, sz, sz]
    L.atlas_b200_routed_prefill_slot_of.restype = i32
    L.atlas_b200_peft_scaling.argtypes = [C.c_double, sz, C.c_int]
    L.atlas_b200_peft_scaling.restype = f32
    L.atlas_b200_module_dims.argtypes = [C.POINTER(ModelDims), C.c_int, C.POINTER(sz), C.POINTER(sz)]
    L.atlas_b200_pool_slot_bytes.argtypes = [C.POINTER(ModelDims), sz]
    L.atlas_b200_pool_slot_bytes.restype = sz
    L.atlas_b200_slot_base_offset.argtypes = [sz, C.POINTER(ModelDims), sz]
    L.atlas_b200_slot_base_offset.restype = sz
    L.atlas_b200_module_slot_offsets.argtypes = [C.POINTER(ModelDims), sz, sz, C.c_int, C.POINTER(sz), C.POINTER(sz)]
    L.atlas_b200_pack_module.argtypes = [C.POINTER(ModelDims), sz, sz, C.c_int, vp, vp, sz, vp]
    L.atlas_b200_build_route_tables.argtypes = [C.POINTER(ModelDims), sz, sz, C.c_int, C.c_uint64, sz, vp, vp, vp]
    L.atlas_b200_select_victim_slot.argtypes = [C.POINTER(sz), C.POINTER(C.c_uint8), C.POINTER(sz),
                                                C.POINTER(C.c_uint64), sz]
    L.atlas_b200_device_status.argtypes = [C.POINTER(u32), C.c_int]
    L.atlas_b200_set_profile_buffer.argtypes = [vp, sz]
    L.atlas_b200_version.restype = C.c_char_p
    u64, cp = C.c_uint64, C.c_char_p
    L.atlas_b200_peft_parse.argtypes = [cp, sz, C.POINTER(PeftConfig), cp, sz]
    L.atlas_b200_peft_config_scaling.argtypes = [C.POINTER(PeftConfig)]
    L.atlas_b200_peft_config_scaling.restype = f32
    L.atlas_b200_classify_key.argtypes = [cp, u32, vp, C.POINTER(u32), C.POINTER(C.c_int), C.POINTER(C.c_int), cp, sz]
    L.atlas_b200_adapter_id_hash.argtypes = [cp, u64]
    L.atlas_b200_adapter_id_hash.restype = u64
    L.atlas_b200_convert_to_bf16.argtypes = [cp, vp, sz, vp]
    L.atlas_b200_registry_create.argtypes = [C.POINTER(ModelDims), u32, vp, sz, sz, u64, C.POINTER(vp)]
    L.atlas_b200_registry_destroy.argtypes = [vp]
    L.atlas_b200_registry_destroy.restype = None
    for fn in (L.atlas_b200_registry_slot_bytes, L.atlas_b200_registry_pool_bytes):
        fn.argtypes, fn.restype = [vp], sz
    L.atlas_b200_registry_load_adapter.argtypes = [vp, sz, cp, cp, sz, vp, sz, vp, cp, sz]
    L.atlas_b200_registry_set_pinned.argtypes = [vp, sz]
    L.atlas_b200_registry_set_active.argtypes = [vp, sz]
    L.atlas_b200_registry_route_tables.argtypes = [vp, u32, C.c_int, vp, vp]
    L.atlas_b200_registry_scale_table.argtypes = [vp, vp]
    L.atlas_b200_registry_rank_table.argtypes = [vp, vp]
    L.atlas_b200_registry_acquire_slot.argtypes, L.atlas_b200_registry_acquire_slot.restype = [vp, i32], i32
    L.atlas_b200_registry_release_slot.argtypes, L.atlas_b200_registry_release_slot.restype = [vp, i32], None
    L.atlas_b200_registry_touch_slot.argtypes, L.atlas_b200_registry_touch_slot.restype = [vp, sz], None
    L.atlas_b200_registry_slot_ref_count.argtypes, L.atlas_b200_registry_slot_ref_count.restype = [vp, sz], sz
    L.atlas_b200_registry_slot_last_used.argtypes, L.atlas_b200_registry_slot_last_used.restype = [vp, sz], u64
    L.atlas_b200_registry_slot_generation.argtypes, L.atlas_b200_registry_slot_generation.restype = [vp, sz], u64
    L.atlas_b200_registry_slot_of.argtypes, L.atlas_b200_registry_slot_of.restype = [vp, cp], i32
    L.atlas_b200_registry_adapter_id_for_slot.argtypes, L.atlas_b200_registry_adapter_id_for_slot.restype = [vp, i32], u64
    L.atlas_b200_registry_select_victim.argtypes, L.atlas_b200_registry_select_victim.restype = [vp], i32
    _lib = L
    return L


def _check(fn: str, status: int) -> None:
    if status != 0:
        raise AtlasError(fn, status)


def _ptr(t) -> Optional[int]:
    """Device (or host) address of a torch tensor / int / None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream_ptr(stream) -> Optional[int]:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


# ------------------------------------------------------------------------------------------
# registry: slot math (host only)
# ------------------------------------------------------------------------------------------
def build_seq_slot_host(adapter_slots: Sequence[int], padded_n: int, active: int) -> list:
    n = len(adapter_slots)
    src = (C.c_int32 * max(n, 1))(*adapter_slots)
    out = (C.c_int32 * max(padded_n, 1))()
    _check("atlas_b200_build_seq_slot", lib().atlas_b200_build_seq_slot(src, n, padded_n, active, out))
    return list(out[:padded_n])


def routed_prefill_slot_of(adapter_slot: int, active: int, num_slots: int) -> Optional[int]:
    r = lib().atlas_b200_routed_prefill_slot_of(adapter_slot, active, num_slots)
    return None if r < 0 else r


def peft_scaling(lora_alpha: float, r: int, use_rslora: bool = False) -> float:
    return float(lib().atlas_b200_peft_scaling(float(lora_alpha), r, int(use_rslora)))


def module_dims(cfg: ModelDims, module: int):
    o, i = C.c_size_t(), C.c_size_t()
    _check("atlas_b200_module_dims", lib().atlas_b200_module_dims(C.byref(cfg), module, C.byref(o), C.byref(i)))
    return o.value, i.value


def pool_slot_bytes(cfg: ModelDims, max_rank: int) -> int:
    return lib().atlas_b200_pool_slot_bytes(C.byref(cfg), max_rank)


def slot_base_offset(slot: int, cfg: ModelDims, max_rank: int) -> int:
    return lib().atlas_b200_slot_base_offset(slot, C.byref(cfg), max_rank)


def module_slot_offsets(cfg: ModelDims, max_rank: int, layer_ordinal: int, module: int):
    a, b = C.c_size_t(), C.c_size_t()
    st = lib().atlas_b200_module_slot_offsets(C.byref(cfg), max_rank, layer_ordinal, module, C.byref(a), C.byref(b))
    if st != 0:
        return None
    return a.value, b.value


def select_victim_slot(cache) -> Optional[int]:
    """cache: sequence of (slot_index, filled, ref_count, last_used); None when every slot is busy."""
    n = len(cache)
    idx = (C.c_size_t * max(n, 1))(*[c[0] for c in cache])
    fil = (C.c_uint8 * max(n, 1))(*[1 if c[1] else 0 for c in cache])
    ref = (C.c_size_t * max(n, 1))(*[c[2] for c in cache])
    lru = (C.c_uint64 * max(n, 1))(*[c[3] for c in cache])
    r = lib().atlas_b200_select_victim_slot(idx, fil, ref, lru, n)
    return None if r < 0 else r


def column_shard(n: int, tp: int, rank: int):
    b, c = C.c_uint32(), C.c_uint32()
    _check("atlas_b200_column_shard", lib().atlas_b200_column_shard(n, tp, rank, C.byref(b), C.byref(c)))
    return b.value, c.value


# ------------------------------------------------------------------------------------------
# operator surface
# ------------------------------------------------------------------------------------------
@dataclass
class LoraRoute:
    """Per-(layer, module) routing tables, fixed at load time; adapter identity flows only through seq_slot."""
    a_table: object          # [max_loras] u64 device tensor (or address)
    b_table: object
    scale_table: object      # [max_loras] f32
    k_in: int
    n_out: int
    max_rank: int
    max_loras: int
    rank_table: object = None   # optional [max_loras] u32 true ranks (not in the reference)
    b_pool_base: object = None  # optional: B side of the pool as a strided array (see atlas_b200.h)
    b_slot_stride: int = 0
    a_pool_base: object = None  # optional: A side of the pool as a strided array
    a_slot_stride: int = 0


def apply_lora_bgmv(route: LoraRoute, x, base_out, seq_slot, n: int, x_row_stride: int, out_row_stride: int,
                    lora_xa, stream=None) -> None:
    _check("atlas_b200_lora_bgmv", lib().atlas_b200_lora_bgmv(
        _ptr(x), _ptr(seq_slot), _ptr(route.a_table), _ptr(route.b_table), _ptr(route.scale_table),
        _ptr(base_out), _ptr(lora_xa), n, route.k_in, route.n_out, route.max_rank,
        x_row_stride, out_row_stride, route.max_loras, _stream_ptr(stream)))


def apply_lora_delta(a, b, scale: float, k_in: int, n_out: int, max_rank: int, x, base_out, m: int,
                     lora_xa, lora_delta=None, stream=None) -> None:
    _check("atlas_b200_lora_delta", lib().atlas_b200_lora_delta(
        _ptr(x), _ptr(a), _ptr(b), scale, _ptr(base_out), _ptr(lora_xa), _ptr(lora_delta),
        m, k_in, n_out, max_rank, _stream_ptr(stream)))


def w4a16_gemm(a, b_packed, b_scale, scale2: float, c, m: int, n: int, k: int, stream=None) -> None:
    _check("atlas_b200_w4a16_gemm", lib().atlas_b200_w4a16_gemm(
        _ptr(a), _ptr(b_packed), _ptr(b_scale), scale2, _ptr(c), m, n, k, None, 0, _stream_ptr(stream)))


def dequant_nvfp4_to_bf16(packed, scales, out, combined_global: float, n: int, k: int, stream=None) -> None:
    _check("atlas_b200_dequant_nvfp4_to_bf16", lib().atlas_b200_dequant_nvfp4_to_bf16(
        _ptr(packed), _ptr(scales), _ptr(out), combined_global, n, k, _stream_ptr(stream)))


def quantize_bf16_to_nvfp4(inp, packed, scales, scale2: float, n: int, k: int, stream=None) -> None:
    _check("atlas_b200_quantize_bf16_to_nvfp4", lib().atlas_b200_quantize_bf16_to_nvfp4(
        _ptr(inp), _ptr(packed), _ptr(scales), scale2, n, k, _stream_ptr(stream)))


def nvfp4_global_absmax(inp, out_max, total: int, stream=None) -> None:
    """max |inp| into the device float `out_max` (zeroed by the caller)."""
    _check("atlas_b200_nvfp4_global_absmax", lib().atlas_b200_nvfp4_global_absmax(_ptr(inp), _ptr(out_max), total, _stream_ptr(stream)))


def scale2_from_absmax(global_max: float) -> float:
    return float(lib().atlas_b200_nvfp4_scale2_from_absmax(global_max))


def combined_global_scale(stored: float, is_reciprocal: bool) -> float:
    return float(lib().atlas_b200_nvfp4_combined_global_scale(stored, int(is_reciprocal)))


def silu_mul(gate, up, out, m: int, k: int, gate_scale=1.0, up_scale=1.0, swiglu_limit=0.0, in_row_stride=None,
             out_row_stride=None, stream=None) -> None:
    _check("atlas_b200_silu_mul", lib().atlas_b200_silu_mul(_ptr(gate), _ptr(up), _ptr(out), gate_scale, up_scale, swiglu_limit,
                                                            m, k, in_row_stride or k, out_row_stride or k, _stream_ptr(stream)))


def silu_mul_quant_nvfp4(gate, up, ws, ws_bytes: int, m: int, k: int, gate_scale=1.0, up_scale=1.0, swiglu_limit=0.0,
                         in_row_stride=None, stream=None) -> None:
    _check("atlas_b200_silu_mul_quant_nvfp4", lib().atlas_b200_silu_mul_quant_nvfp4(
        _ptr(gate), _ptr(up), _ptr(ws), ws_bytes, gate_scale, up_scale, swiglu_limit, m, k, in_row_stride or k, _stream_ptr(stream)))


def kv_norm_rope_cache_write(k_in, v_in, in_row_stride: int, k_norm_weight, positions, slot_mapping, k_cache, v_cache,
                             tokens: int, kv_heads: int, head_dim: int, rotary_dim: int, block_size: int,
                             rms_eps: float, theta: float, stream=None, positions_h=None, positions_w=None) -> None:
    """K heads: RMS norm (1 + w), rotary embedding, one BF16 rounding, paged cache write; V heads: paged cache write.
    k_in / v_in: tensors or device addresses of the first K / V column of token 0 (v_in None: K side only).
    positions_h / positions_w: the two further position streams of MRoPE (both or neither)."""
    if positions_h is not None or positions_w is not None:
        _check("atlas_b200_kv_norm_mrope_cache_write", lib().atlas_b200_kv_norm_mrope_cache_write(
            _ptr(k_in), _ptr(v_in), in_row_stride, _ptr(k_norm_weight), _ptr(positions), _ptr(positions_h), _ptr(positions_w),
            _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), tokens, kv_heads, head_dim, rotary_dim, block_size, rms_eps, theta,
            _stream_ptr(stream)))
        return
    _check("atlas_b200_kv_norm_rope_cache_write", lib().atlas_b200_kv_norm_rope_cache_write(
        _ptr(k_in), _ptr(v_in), in_row_stride, _ptr(k_norm_weight), _ptr(positions), _ptr(slot_mapping), _ptr(k_cache),
        _ptr(v_cache), tokens, kv_heads, head_dim, rotary_dim, block_size, rms_eps, theta, _stream_ptr(stream)))


def k_norm_rope_cache_write_fp8(k_in, in_row_stride: int, k_norm_weight, positions, slot_mapping, k_cache_fp8, tokens: int, kv_heads: int,
                                head_dim: int, rotary_dim: int, block_size: int, rms_eps: float, theta: float, inv_scale: float, stream=None) -> None:
    """The K side into an E4M3 paged cache (one byte per element): value * inv_scale, saturating cast."""
    _check("atlas_b200_k_norm_rope_cache_write_fp8", lib().atlas_b200_k_norm_rope_cache_write_fp8(
        _ptr(k_in), in_row_stride, _ptr(k_norm_weight), _ptr(positions), _ptr(slot_mapping), _ptr(k_cache_fp8), tokens, kv_heads, head_dim,
        rotary_dim, block_size, rms_eps, theta, inv_scale, _stream_ptr(stream)))


def qkv_norm_rope_cache_write(q, k_in, v_in, q_row_stride: int, kv_row_stride: int, q_norm_weight, k_norm_weight, positions, inv_freq,
                              slot_mapping, k_cache, v_cache, tokens: int, q_heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                              block_size: int, rms_eps: float, attention_factor: float = 1.0, norm_offset_one: bool = True, stream=None) -> None:
    """Decode-path QKV consumer: Q normed and rotated in place, K normed, rotated and written to the paged cache, V copied."""
    _check("atlas_b200_qkv_norm_rope_cache_write", lib().atlas_b200_qkv_norm_rope_cache_write(
        _ptr(q), _ptr(k_in), _ptr(v_in), q_row_stride, kv_row_stride, _ptr(q_norm_weight), _ptr(k_norm_weight), _ptr(positions),
        _ptr(inv_freq), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), tokens, q_heads, kv_heads, head_dim, rotary_dim, block_size,
        rms_eps, attention_factor, 1 if norm_offset_one else 0, _stream_ptr(stream)))


def make_linear_desc(*, x, m, k, n, y, w_packed=None, w_scale=None, scale2=1.0, w_bf16=None,
                     x_row_stride=None, out_row_stride=None, seq_slot=None, route: Optional[LoraRoute] = None,
                     lora_t=None, flags=0, ws=None, ws_bytes=0, y_dest=None, y_col_offset=0) -> LinearDesc:
    d = LinearDesc()
    d.x, d.m, d.k = _ptr(x), m, k
    d.x_row_stride = x_row_stride if x_row_stride is not None else k
    d.n = n
    d.w_packed, d.w_scale, d.w_bf16 = _ptr(w_packed), _ptr(w_scale), _ptr(w_bf16)
    d.scale2, d.flags = scale2, flags
    if seq_slot is not None:
        assert route is not None
        d.seq_slot = _ptr(seq_slot)
        d.a_table, d.b_table, d.scale_table = _ptr(route.a_table), _ptr(route.b_table), _ptr(route.scale_table)
        d.rank_table = _ptr(route.rank_table)
        d.max_loras, d.max_rank = route.max_loras, route.max_rank
        d.lora_t = _ptr(lora_t)
        d.b_pool_base, d.b_slot_stride = _ptr(route.b_pool_base), route.b_slot_stride
        d.a_pool_base, d.a_slot_stride = _ptr(route.a_pool_base), route.a_slot_stride
    d.y = _ptr(y)
    d.out_row_stride = out_row_stride if out_row_stride is not None else n
    d.ws, d.ws_bytes = _ptr(ws), ws_bytes
    if y_dest is not None:                       # tensor-parallel placement: one gathered buffer per rank
        d.n_dest, d.y_col_offset = len(y_dest), y_col_offset
        for i, t in enumerate(y_dest):
            d.y_dest[i] = _ptr(t)
    return d


def nvfp4_lora_linear(desc: LinearDesc, stream=None) -> int:
    """Launch the fused layer; returns the kernel family that ran (VARIANT_*)."""
    _check("atlas_b200_nvfp4_lora_linear", lib().atlas_b200_nvfp4_lora_linear(C.byref(desc), _stream_ptr(stream)))
    return lib().atlas_b200_last_variant()


def lora_shrink_tiles(desc: LinearDesc, row_begin: int, row_count: int, ws_dest, stream=None) -> None:
    """The shrink of `desc` for rows [row_begin, row_begin + row_count) only, its tiles stored into every scratch buffer
    of `ws_dest` (device addresses or tensors laid out like desc.ws); the fused call then runs with FLAG_REUSE_SHRINK."""
    arr = (C.c_void_p * len(ws_dest))(*[_ptr(w) for w in ws_dest])
    _check("atlas_b200_lora_shrink_tiles", lib().atlas_b200_lora_shrink_tiles(
        C.byref(desc), row_begin, row_count, arr, len(ws_dest), _stream_ptr(stream)))


def push_columns(src_ptr: int, src_row_stride: int, dest_ptrs, dst_row_stride: int, m: int, n_cols: int, stream=None,
                 copy_engines: bool = False) -> None:
    """Copy the [m, n_cols] BF16 block at device address `src_ptr` into the same block of every buffer in `dest_ptrs`
    (addresses of the block's first element in the peers' gathered buffers): by the push kernel, or by the copy engines."""
    arr = (C.c_void_p * len(dest_ptrs))(*[int(p) for p in dest_ptrs])
    fn = lib().atlas_b200_copy_columns if copy_engines else lib().atlas_b200_push_columns
    _check("atlas_b200_copy_columns" if copy_engines else "atlas_b200_push_columns", fn(
        C.c_void_p(int(src_ptr)), src_row_stride, arr, len(dest_ptrs), dst_row_stride, m, n_cols, _stream_ptr(stream)))


def selftest_bounded_wait(limit_ns: int):
    """(first waiter gave up, second waiter gave up, ns the first waited) of the library's bounded-wait self-test."""
    out = (C.c_uint32 * 3)()
    _check("atlas_b200_selftest_bounded_wait", lib().atlas_b200_selftest_bounded_wait(limit_ns, out))
    return int(out[0]), int(out[1]), int(out[2])


STATIC_SCRATCH_ELEMS = 512 * 1024


def nvfp4_lora_linear_noalloc(desc: LinearDesc, stream=None) -> int:
    """The fused layer without a caller-provided shrink scratch (`desc.lora_t` is ignored).

    For callers that may launch kernels but may not allocate device memory: the scratch is a fixed
    1 MiB array inside the library (m * max_rank <= STATIC_SCRATCH_ELEMS, else AtlasError -5).  Calls
    share that array, so calls that could overlap on the GPU must be serialised by the caller.
    Returns the kernel family that ran (VARIANT_*)."""
    _check("atlas_b200_nvfp4_lora_linear_noalloc",
           lib().atlas_b200_nvfp4_lora_linear_noalloc(C.byref(desc), _stream_ptr(stream)))
    return lib().atlas_b200_last_variant()


def last_launch_shape() -> dict:
    """Token tile, pairing, K split and LoRA-tile source of this thread's most recent tcgen05 launch."""
    out = (C.c_uint32 * 4)()
    _check("atlas_b200_last_launch_shape", lib().atlas_b200_last_launch_shape(out))
    per = (C.c_uint32 * 2)()
    _check("atlas_b200_last_persistent_shape", lib().atlas_b200_last_persistent_shape(per))
    return {"token_tile": out[0], "cta_pair": bool(out[1]), "k_split": out[2], "lora_tiles_from_shrink": bool(out[3]),
            "persistent_tiles_per_pass": per[0], "persistent_cta_pairs": per[1]}


def device_status(clear: bool = True) -> int:
    w = C.c_uint32()
    _check("atlas_b200_device_status", lib().atlas_b200_device_status(C.byref(w), int(clear)))
    return w.value


# ------------------------------------------------------------------------------------------
# a one-module pool on the device (what `load_lora_adapters_multi` leaves behind for one module)
# ------------------------------------------------------------------------------------------
class LoraPool:
    """Rank-padded adapter pool for ONE (layer, module) on the current CUDA device.

    Slot s holds A_s as [max_rank, k_in] and B_s as [n_out, max_rank] (zero padded, BF16), and the
    pool owns the [max_loras] address tables, the scale table and a true-rank table.  `pack`
    uploads one adapter; an un-packed slot keeps null table entries (= no adapter).
    """

    def __init__(self, k_in: int, n_out: int, max_rank: int, max_loras: int, device="cuda"):
        import torch
        self.k_in, self.n_out, self.max_rank, self.max_loras = k_in, n_out, max_rank, max_loras
        self.a_pool = torch.zeros((max_loras, max_rank, k_in), dtype=torch.bfloat16, device=device)
        self.b_pool = torch.zeros((max_loras, n_out, max_rank), dtype=torch.bfloat16, device=device)
        self._a_host = [0] * max_loras
        self._b_host = [0] * max_loras
        self._scale_host = [0.0] * max_loras
        self._rank_host = [0] * max_loras
        self.a_table = torch.zeros(max_loras, dtype=torch.int64, device=device)
        self.b_table = torch.zeros(max_loras, dtype=torch.int64, device=device)
        self.scale_table = torch.zeros(max_loras, dtype=torch.float32, device=device)
        self.rank_table = torch.zeros(max_loras, dtype=torch.int32, device=device)

    def pack(self, slot: int, a, b, scale: float) -> None:
        """a: [r, k_in] bf16 tensor, b: [n_out, r] bf16 tensor (PEFT lora_A / lora_B layout)."""
        import torch
        r = a.shape[0]
        assert r <= self.max_rank and a.shape[1] == self.k_in and tuple(b.shape) == (self.n_out, r)
        self.a_pool[slot].zero_()
        self.b_pool[slot].zero_()
        self.a_pool[slot, :r].copy_(a)
        self.b_pool[slot, :, :r].copy_(b)
        self._a_host[slot] = self.a_pool[slot].data_ptr()
        self._b_host[slot] = self.b_pool[slot].data_ptr()
        self._scale_host[slot] = float(scale)
        self._rank_host[slot] = r
        self.refresh_tables()

    def refresh_tables(self) -> None:
        import torch
        self.a_table.copy_(torch.tensor(self._a_host, dtype=torch.int64))
        self.b_table.copy_(torch.tensor(self._b_host, dtype=torch.int64))
        self.scale_table.copy_(torch.tensor(self._scale_host, dtype=torch.float32))
        self.rank_table.copy_(torch.tensor(self._rank_host, dtype=torch.int32))

    def route(self, with_ranks: bool = True, strided: bool = True) -> LoraRoute:
        r = LoraRoute(self.a_table, self.b_table, self.scale_table, self.k_in, self.n_out,
                      self.max_rank, self.max_loras, self.rank_table if with_ranks else None)
        if strided:     # slot s of b_pool starts s * n_out * max_rank * 2 bytes after slot 0
            r.b_pool_base, r.b_slot_stride = self.b_pool.data_ptr(), self.n_out * self.max_rank * 2
            r.a_pool_base, r.a_slot_stride = self.a_pool.data_ptr(), self.max_rank * self.k_in * 2
        return r
