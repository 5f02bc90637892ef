"""numpy/ctypes front end of the CPU oracle (libatlas_oracle.so).  TEST INFRASTRUCTURE ONLY.

Imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs — never by the
shipped package.  BF16 tensors travel as numpy uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libatlas_oracle.so")
REF_DIR = os.path.join(_HERE, "_ref")

_lib = None


class ModelDims(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads", "head_dim",
        "attn_gated", "num_full_attention_layers")]


class FusedArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("M", C.c_uint32), ("N", C.c_uint32), ("K", C.c_uint32), ("x_row_stride", C.c_uint32),
        ("packed", C.c_void_p), ("scales", C.c_void_p), ("scale2", C.c_float),
        ("w_bf16", C.c_void_p), ("act_fp4", C.c_int),
        ("seq_slot", C.c_void_p), ("a_ptrs", C.c_void_p), ("b_ptrs", C.c_void_p),
        ("scale_table", C.c_void_p), ("rank_table", C.c_void_p),
        ("max_loras", C.c_uint32), ("max_rank", C.c_uint32),
    ]


def build() -> None:
    subprocess.run(["make", "-C", _HERE, "--no-print-directory"], check=True, stdout=subprocess.DEVNULL)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        L.orc_e2m1_decode.restype = C.c_float
        L.orc_e2m1_decode.argtypes = [C.c_uint32]
        L.orc_e4m3_decode.restype = C.c_float
        L.orc_e4m3_decode.argtypes = [C.c_uint8]
        L.orc_e4m3_encode.restype = C.c_uint8
        L.orc_e4m3_encode.argtypes = [C.c_float]
        L.orc_e2m1_quantize.restype = C.c_uint32
        L.orc_e2m1_quantize.argtypes = [C.c_float]
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_splitmix64_next.restype = C.c_uint64
        L.orc_splitmix64_next.argtypes = [C.POINTER(C.c_uint64)]
        L.orc_rng_uniform.restype = C.c_float
        L.orc_rng_uniform.argtypes = [C.POINTER(C.c_uint64), C.c_float, C.c_float]
        L.orc_gen_val.restype = C.c_float
        L.orc_gen_val.argtypes = [C.c_uint64]
        L.orc_nvfp4_global_absmax.restype = C.c_float
        L.orc_nvfp4_global_absmax.argtypes = [C.c_void_p, C.c_size_t]
        L.orc_peft_scaling.restype = C.c_float
        L.orc_peft_scaling.argtypes = [C.c_double, C.c_size_t, C.c_int]
        L.orc_pool_slot_bytes.restype = C.c_size_t
        L.orc_pool_slot_bytes.argtypes = [C.POINTER(ModelDims), C.c_size_t]
        L.orc_module_slot_offsets.argtypes = [C.POINTER(ModelDims), C.c_size_t, C.c_size_t, C.c_int,
                                              C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        L.orc_module_dims.argtypes = [C.POINTER(ModelDims), C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        L.orc_routed_prefill_slot_of.restype = C.c_int32
        L.orc_routed_prefill_slot_of.argtypes = [C.c_int32, C.c_size_t, C.c_size_t]
        L.orc_build_seq_slot_host.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int32, C.c_void_p]
        L.orc_dequant_nvfp4_to_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_uint32, C.c_uint32]
        L.orc_dequant_nvfp4_to_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_uint32, C.c_uint32]
        L.orc_quantize_bf16_to_nvfp4.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_uint32, C.c_uint32]
        L.orc_act_quant_max6.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32]
        L.orc_pack_pair.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                    C.c_void_p, C.c_void_p]
        L.orc_lora_bgmv_staged.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32,
                                           C.c_void_p, C.c_void_p] + [C.c_uint32] * 6
        L.orc_lora_delta_staged.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p,
                                            C.c_void_p] + [C.c_uint32] * 4
        L.orc_w4a16_gemm_bf16w.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p] + [C.c_uint32] * 3
        L.orc_dense_gemm_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_uint32] * 3
        L.orc_fused_linear_f32.argtypes = [C.POINTER(FusedArgs), C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
        L.orc_reference_sequence.argtypes = [C.POINTER(FusedArgs), C.c_void_p, C.c_void_p, C.c_uint32]
        L.orc_num_threads.restype = C.c_int
        L.orc_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_float, C.c_size_t]
        L.orc_qkv_norm_rope_cache_write.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p,
                                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                                    C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_int]
        L.orc_k_norm_rope_cache_write.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                                  C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float]
        L.orc_quantize_f32_to_nvfp4_scale1.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32]
        L.orc_set_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ---- codecs over numpy arrays -------------------------------------------------------------------
def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even BF16 bits of a float32 array (vectorised form of orc_f32_to_bf16)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = ((bits.astype(np.uint64) + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((bits >> 16) | 0x40).astype(np.uint16), rounded)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_decode_table() -> np.ndarray:
    L = lib()
    return np.array([L.orc_e4m3_decode(i) for i in range(256)], dtype=np.float32)


def e2m1_decode_table() -> np.ndarray:
    L = lib()
    return np.array([L.orc_e2m1_decode(i) for i in range(16)], dtype=np.float32)


def dequant_nvfp4_to_bf16(packed, scales, g, N, K) -> np.ndarray:
    out = np.empty((N, K), dtype=np.uint16)
    lib().orc_dequant_nvfp4_to_bf16(_p(packed), _p(scales), _p(out), g, N, K)
    return out


def dequant_nvfp4_to_f32(packed, scales, g, N, K) -> np.ndarray:
    out = np.empty((N, K), dtype=np.float32)
    lib().orc_dequant_nvfp4_to_f32(_p(packed), _p(scales), _p(out), g, N, K)
    return out


def quantize_bf16_to_nvfp4(inp, scale2, N, K):
    packed = np.empty((N, K // 2), dtype=np.uint8)
    scales = np.empty((N, K // 16), dtype=np.uint8)
    lib().orc_quantize_bf16_to_nvfp4(_p(inp), _p(packed), _p(scales), scale2, N, K)
    return packed, scales


def act_quant_max6(inp, M, K):
    packed = np.empty((M, K // 2), dtype=np.uint8)
    scales = np.empty((M, K // 16), dtype=np.uint8)
    lib().orc_act_quant_max6(_p(inp), _p(packed), _p(scales), M, K)
    return packed, scales


def build_seq_slot_host(slots, padded_n, active):
    src = np.asarray(slots, dtype=np.int32)
    out = np.empty(padded_n, dtype=np.int32)
    lib().orc_build_seq_slot_host(_p(src), len(src), padded_n, active, _p(out))
    return out.tolist()


class HostPool:
    """Host image of a one-module adapter pool: padded A/B per slot, pointer arrays, scales, ranks."""

    def __init__(self, k_in, n_out, max_rank, max_loras):
        self.k_in, self.n_out, self.max_rank, self.max_loras = k_in, n_out, max_rank, max_loras
        self.a = [None] * max_loras
        self.b = [None] * max_loras
        self.scale = np.zeros(max_loras, dtype=np.float32)
        self.rank = np.zeros(max_loras, dtype=np.uint32)

    def pack(self, slot, a_bits, b_bits, scale):
        r = a_bits.shape[0]
        ap = np.empty((self.max_rank, self.k_in), dtype=np.uint16)
        bp = np.empty((self.n_out, self.max_rank), dtype=np.uint16)
        lib().orc_pack_pair(_p(np.ascontiguousarray(a_bits)), _p(np.ascontiguousarray(b_bits)), r, self.k_in,
                            self.n_out, self.max_rank, _p(ap), _p(bp))
        self.a[slot], self.b[slot] = ap, bp
        self.scale[slot] = scale
        self.rank[slot] = r

    def ptr_arrays(self):
        pa = (C.c_void_p * self.max_loras)(*[None if t is None else t.ctypes.data for t in self.a])
        pb = (C.c_void_p * self.max_loras)(*[None if t is None else t.ctypes.data for t in self.b])
        return pa, pb


def lora_bgmv_staged(x, seq_slot, pool: HostPool, base_out, n, x_row_stride=None, out_row_stride=None):
    """In place on base_out (uint16 bits); returns xa."""
    xs = x_row_stride or pool.k_in
    os_ = out_row_stride or pool.n_out
    xa = np.zeros((n, pool.max_rank), dtype=np.uint16)
    pa, pb = pool.ptr_arrays()
    lib().orc_lora_bgmv_staged(_p(x), _p(np.asarray(seq_slot, dtype=np.int32)), pa, pb, _p(pool.scale), pool.max_loras,
                               _p(base_out), _p(xa), n, pool.k_in, pool.n_out, pool.max_rank, xs, os_)
    return xa


def lora_delta_staged(x, a_pool, b_pool, scale, base_out, m, k_in, n_out, max_rank):
    xa = np.zeros((m, max_rank), dtype=np.uint16)
    delta = np.zeros((m, n_out), dtype=np.uint16)
    lib().orc_lora_delta_staged(_p(x), _p(a_pool), _p(b_pool), scale, _p(base_out), _p(xa), _p(delta), m, k_in, n_out, max_rank)
    return xa, delta


def w4a16_gemm_bf16w(a, packed, scales, scale2, M, N, K):
    c = np.empty((M, N), dtype=np.uint16)
    lib().orc_w4a16_gemm_bf16w(_p(a), _p(packed), _p(scales), scale2, _p(c), M, N, K)
    return c


def _fused_args(x, M, N, K, *, packed=None, scales=None, scale2=1.0, w_bf16=None, seq_slot=None,
                pool: HostPool = None, use_ranks=True, act_fp4=False, x_row_stride=None):
    g = FusedArgs()
    keep = [x, packed, scales, w_bf16]
    g.x, g.M, g.N, g.K = x.ctypes.data, M, N, K
    g.x_row_stride = x_row_stride or K
    g.packed = None if packed is None else packed.ctypes.data
    g.scales = None if scales is None else scales.ctypes.data
    g.scale2 = scale2
    g.w_bf16 = None if w_bf16 is None else w_bf16.ctypes.data
    g.act_fp4 = int(act_fp4)
    if seq_slot is not None:
        ss = np.ascontiguousarray(seq_slot, dtype=np.int32)
        pa, pb = pool.ptr_arrays()
        keep += [ss, pa, pb, pool]
        g.seq_slot = ss.ctypes.data
        g.a_ptrs = C.cast(pa, C.c_void_p)
        g.b_ptrs = C.cast(pb, C.c_void_p)
        g.scale_table = pool.scale.ctypes.data
        g.rank_table = pool.rank.ctypes.data if use_ranks else None
        g.max_loras, g.max_rank = pool.max_loras, pool.max_rank
    return g, keep


def fused_linear_f32(x, M, N, K, rows=None, cols=None, **kw) -> np.ndarray:
    """FP32-accumulated ideal of the fused layer on rows x cols (None = all)."""
    g, keep = _fused_args(x, M, N, K, **kw)
    r = None if rows is None else np.ascontiguousarray(rows, dtype=np.uint32)
    c = None if cols is None else np.ascontiguousarray(cols, dtype=np.uint32)
    nr = M if r is None else len(r)
    nc = N if c is None else len(c)
    out = np.empty((nr, nc), dtype=np.float32)
    lib().orc_fused_linear_f32(C.byref(g), _p(r), nr, _p(c), nc, _p(out))
    return out


def reference_sequence(x, M, N, K, out_row_stride=None, **kw):
    """Base linear (BF16 out) followed by the staged routed LoRA, as the reference launches them."""
    g, keep = _fused_args(x, M, N, K, **kw)
    os_ = out_row_stride or N
    y = np.zeros((M, os_), dtype=np.uint16)
    xa = np.zeros((M, max(g.max_rank, 1)), dtype=np.uint16)
    lib().orc_reference_sequence(C.byref(g), _p(y), _p(xa), os_)
    return y, xa


def k_norm_rope_cache_write(k_in, in_row_stride, k_norm_w, positions, slot_mapping, k_cache, kv_heads, head_dim, rotary_dim, block_size,
                            rms_eps, theta) -> None:
    """In place on k_cache (uint16 bits, [blocks, block_size, kv_heads, head_dim]); k_in [tokens, in_row_stride] bits."""
    k_in = np.ascontiguousarray(k_in)
    lib().orc_k_norm_rope_cache_write(_p(k_in), in_row_stride, _p(np.ascontiguousarray(k_norm_w)), _p(np.ascontiguousarray(positions, dtype=np.uint32)),
                                      _p(np.ascontiguousarray(slot_mapping, dtype=np.int64)), _p(k_cache), len(positions), kv_heads, head_dim,
                                      rotary_dim, block_size, rms_eps, theta)


def qkv_norm_rope_cache_write(q, q_row_stride, k_in, v_in, kv_row_stride, q_norm_w, k_norm_w, positions, inv_freq, slot_mapping, k_cache, v_cache,
                              q_heads, kv_heads, head_dim, rotary_dim, block_size, eps, factor=1.0, offset_one=True) -> None:
    """In place on q (uint16 bits, [tokens, q_row_stride]) and on the two caches."""
    assert q.flags["C_CONTIGUOUS"] and k_cache.flags["C_CONTIGUOUS"] and v_cache.flags["C_CONTIGUOUS"]
    lib().orc_qkv_norm_rope_cache_write(_p(q), q_row_stride, _p(np.ascontiguousarray(k_in)), _p(np.ascontiguousarray(v_in)), kv_row_stride,
                                        _p(np.ascontiguousarray(q_norm_w)), _p(np.ascontiguousarray(k_norm_w)),
                                        _p(np.ascontiguousarray(positions, dtype=np.uint32)), _p(np.ascontiguousarray(inv_freq, dtype=np.float32)),
                                        _p(np.ascontiguousarray(slot_mapping, dtype=np.int64)), _p(k_cache), _p(v_cache), len(positions),
                                        q_heads, kv_heads, head_dim, rotary_dim, block_size, eps, factor, 1 if offset_one else 0)


def silu_mul(gate, up, gate_scale=1.0, up_scale=1.0, limit=0.0) -> np.ndarray:
    """FP32 SwiGLU of two BF16 bit arrays of one shape."""
    out = np.empty(gate.shape, dtype=np.float32)
    lib().orc_silu_mul(_p(np.ascontiguousarray(gate)), _p(np.ascontiguousarray(up)), _p(out), gate_scale, up_scale, limit, gate.size)
    return out


def quantize_f32_to_nvfp4_scale1(v: np.ndarray):
    """[M, K] FP32 -> (packed [M, K/2], scales [M, K/16]) with the activation quantiser (tensor scale 1)."""
    M, K = v.shape
    packed = np.empty((M, K // 2), dtype=np.uint8)
    scales = np.empty((M, K // 16), dtype=np.uint8)
    lib().orc_quantize_f32_to_nvfp4_scale1(_p(np.ascontiguousarray(v, dtype=np.float32)), _p(packed), _p(scales), M, K)
    return packed, scales


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int = 0) -> int:
    """Threads for the OpenMP loops (0 = one per online core, whatever OMP_NUM_THREADS says); returns the count in effect."""
    return lib().orc_set_num_threads(n)
