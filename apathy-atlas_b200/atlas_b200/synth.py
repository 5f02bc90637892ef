"""Seeded synthetic inputs for the NVFP4 + multi-LoRA linear (numpy only).

The reference seeds its microtests with SplitMix64 (crates/spark-model/examples/lora_apply_microtest.rs:31-44);
the same generator is used here in counter form (value i = mix(seed + (i+1)*gamma)) so tensors can be
produced in one vectorised pass.  Uniforms take the top 24 bits as the reference does; normals are a
Box-Muller transform of two such uniforms.  Nothing here comes from a dataset: shapes, sizes and value
distributions are those the benchmark configurations name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


_CHUNK = 1 << 22
_POOL = None


def _chunks(n: int, fn):
    """Run fn(start, count) over [0, n) in pieces on a few threads (numpy releases the GIL) and concatenate."""
    if n <= _CHUNK:
        return fn(0, n)
    global _POOL
    if _POOL is None:
        import os
        from concurrent.futures import ThreadPoolExecutor
        _POOL = ThreadPoolExecutor(max_workers=max(1, min(8, (os.cpu_count() or 2) - 1)))
    parts = list(_POOL.map(lambda s: fn(s, min(_CHUNK, n - s)), range(0, n, _CHUNK)))
    return np.concatenate(parts)


def _splitmix_range(seed: int, start: int, count: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + _GAMMA * np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def splitmix64(seed: int, n: int) -> np.ndarray:
    return _chunks(n, lambda s, c: _splitmix_range(seed, s, c))


def _uniform01_range(seed: int, start: int, count: int) -> np.ndarray:
    return (_splitmix_range(seed, start, count) >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / (1 << 24))


def uniform01(seed: int, n: int) -> np.ndarray:
    return _chunks(n, lambda s, c: _uniform01_range(seed, s, c))


def uniform(seed: int, n: int, lo: float, hi: float) -> np.ndarray:
    return (lo + uniform01(seed, n) * np.float32(hi - lo)).astype(np.float32)


def normal(seed: int, n: int, std: float = 1.0) -> np.ndarray:
    """Box-Muller in FP32 over pairs of uniforms: element 2i is the cosine branch of pair i, 2i+1 the sine branch."""
    half = (n + 1) // 2

    def part(s, c):
        u1 = np.maximum(_uniform01_range(seed, s, c), np.float32(2.0 ** -25))
        u2 = _uniform01_range(seed ^ 0x5DEECE66D, s, c)
        r = np.sqrt(np.float32(-2.0) * np.log(u1)) * np.float32(std)
        ang = np.float32(2.0 * np.pi) * u2
        out = np.empty((c, 2), dtype=np.float32)
        out[:, 0] = r * np.cos(ang)
        out[:, 1] = r * np.sin(ang)
        return out.reshape(-1)
    return _chunks(half, part)[:n]


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round to nearest even (finite inputs; the generators here produce nothing else)."""
    flat = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)

    def part(s, c):
        bits = flat[s:s + c].view(np.uint32)
        with np.errstate(over="ignore"):
            return ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    return _chunks(flat.size, part).reshape(np.shape(a))


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_encode_positive(v: np.ndarray) -> np.ndarray:
    """E4M3 bytes of non-negative floats: saturate at 448, round the mantissa half-up with carry,
    subnormals as round(v*512).  Never yields the NaN byte 0x7F or a sign bit."""
    v = np.minimum(np.asarray(v, dtype=np.float32), np.float32(448.0))
    bits = v.view(np.uint32)
    fe = ((bits >> 23) & 0xFF).astype(np.int32) - 127
    fm = bits & 0x7FFFFF
    e = fe + 7
    man = (fm + (1 << 19)) >> 20
    carry = man > 7
    man = np.where(carry, 0, man)
    e = np.where(carry, e + 1, e)
    over = e > 15
    e = np.where(over, 15, e)
    man = np.where(over, 6, man)
    man = np.where((e == 15) & (man == 7), 6, man)
    normal_b = ((e.astype(np.uint32) << 3) | man.astype(np.uint32)).astype(np.uint8)
    sub = np.clip((v * np.float32(512.0) + np.float32(0.5)).astype(np.int32), 0, 7).astype(np.uint8)
    out = np.where(fe < -6, sub, normal_b)
    out = np.where((fe < -9) | (v == 0), 0, out)
    return out.astype(np.uint8)


def zipf_ids(seed: int, n: int, n_items: int, s: float = 1.1) -> np.ndarray:
    w = 1.0 / np.arange(1, n_items + 1, dtype=np.float64) ** s
    cdf = np.cumsum(w / w.sum())
    return np.minimum(np.searchsorted(cdf, uniform01(seed, n).astype(np.float64)), n_items - 1).astype(np.int32)


@dataclass
class Adapter:
    a: np.ndarray      # [r, K] bf16 bits
    b: np.ndarray      # [N, r] bf16 bits
    scale: float
    rank: int


@dataclass
class Case:
    name: str
    M: int
    K: int
    N: int
    max_rank: int
    max_loras: int
    x: np.ndarray                      # [M, K] bf16 bits
    seq_slot: np.ndarray               # [M] i32
    adapters: List[Optional[Adapter]]  # per slot
    packed: Optional[np.ndarray] = None    # [N, K/2] u8
    scales: Optional[np.ndarray] = None    # [N, K/16] u8 (E4M3)
    scale2: float = 1.0
    w_bf16: Optional[np.ndarray] = None    # [N, K] bf16 bits (dense base)
    meta: dict = field(default_factory=dict)


def make_nvfp4_weight(seed: int, N: int, K: int):
    """Codes uniform over the 16 E2M1 values; block scales E4M3(|N(0,1)|)."""
    packed = _chunks(N * (K // 2), lambda s, c: (_splitmix_range(seed, s, c) >> np.uint64(56)).astype(np.uint8)).reshape(N, K // 2)
    scales = e4m3_encode_positive(np.abs(normal(seed + 1, N * (K // 16)))).reshape(N, K // 16)
    return packed, scales


def make_adapter(seed: int, K: int, N: int, r: int, alpha: float, b_std: float = 0.02) -> Adapter:
    lim = 1.0 / np.sqrt(K)
    a = f32_to_bf16_bits(uniform(seed, r * K, -lim, lim)).reshape(r, K)
    b = f32_to_bf16_bits(normal(seed + 7, N * r, b_std)).reshape(N, r)
    return Adapter(a, b, float(np.float32(alpha / r)), r)


def make_case(name: str, *, M: int, K: int, N: int, ranks: List[int], max_rank: int, max_loras: Optional[int] = None,
              ids: str = "uniform", none_frac: float = 0.0, base: str = "nvfp4", scale2: float = 1.0,
              alpha_over_r: float = 2.0, b_std: float = 0.02, seed: int = 1, segments: int = 0) -> Case:
    n_ad = len(ranks)
    max_loras = max_loras or n_ad
    x = f32_to_bf16_bits(normal(seed * 1000 + 1, M * K)).reshape(M, K)
    adapters: List[Optional[Adapter]] = [None] * max_loras
    for s, r in enumerate(ranks):
        adapters[s] = make_adapter(seed * 1000 + 100 + 13 * s, K, N, r, alpha_over_r * r, b_std)
    if ids == "uniform":
        slot = np.minimum((uniform01(seed * 1000 + 3, M) * n_ad).astype(np.int32), n_ad - 1)
    elif ids == "distinct":
        slot = (np.arange(M) % n_ad).astype(np.int32)
    elif ids == "zipf":
        slot = zipf_ids(seed * 1000 + 3, M, n_ad)
    elif ids == "segments":
        # `segments` contiguous runs of random length (each >= 1), one adapter per run
        cand = (uniform01(seed * 1000 + 5, 16 * segments) * (M - 1)).astype(np.int64) + 1       # in [1, M-1]
        _, first = np.unique(cand, return_index=True)
        cuts = np.sort(cand[np.sort(first)[: segments - 1]])        # the first segments-1 distinct draws: min length 1
        bounds = np.concatenate([[0], cuts, [M]])
        seg_ad = np.minimum((uniform01(seed * 1000 + 6, len(bounds) - 1) * n_ad).astype(np.int32), n_ad - 1)
        slot = np.repeat(seg_ad, np.diff(bounds)).astype(np.int32)
    else:
        raise ValueError(ids)
    if none_frac > 0:
        slot = np.where(uniform01(seed * 1000 + 4, M) < none_frac, -1, slot).astype(np.int32)
    case = Case(name, M, K, N, max_rank, max_loras, x, slot.astype(np.int32), adapters, scale2=scale2)
    if base == "nvfp4":
        case.packed, case.scales = make_nvfp4_weight(seed * 1000 + 50, N, K)
    else:
        case.w_bf16 = f32_to_bf16_bits(normal(seed * 1000 + 50, N * K, 0.02)).reshape(N, K)
    return case


def baseline_config(idx: int, seed: int = 1, **override) -> Case:
    """One projection of each benchmark configuration (the whole layers are `layer_config`)."""
    if idx == 0:   # CPU-runnable single linear, dense BF16 base
        kw = dict(M=16, K=4096, N=4096, ranks=[16] * 4, max_rank=16, base="bf16", alpha_over_r=2.0)
    elif idx == 1:  # NVFP4 K=5120 N=17408, 256 tokens, 16 adapters rank 32, 10 % adapter-less
        kw = dict(M=256, K=5120, N=17408, ranks=[32] * 16, max_rank=32, none_frac=0.10)
    elif idx == 2:  # decode: 64 tokens, 64 distinct adapters, heterogeneous ranks, fused QKV
        rk = [(8, 16, 32, 64)[int(v)] for v in (uniform01(seed * 77 + 9, 64) * 4).astype(np.int32).clip(0, 3)]
        kw = dict(M=64, K=4096, N=6144, ranks=rk, max_rank=64, ids="distinct")
    elif idx == 3:  # prefill, Llama-3-8B gate/up projection: 8192 tokens in 32 segments, 8 adapters rank 64
        kw = dict(M=8192, K=4096, N=14336, ranks=[64] * 8, max_rank=64, ids="segments", segments=32)
    elif idx == 4:  # 70B-shaped MLP gate/up: 512 tokens, 128 adapters rank 16 Zipf(1.1), 25 % adapter-less
        kw = dict(M=512, K=8192, N=28672, ranks=[16] * 128, max_rank=16, ids="zipf", none_frac=0.25)
    else:
        raise ValueError(idx)
    kw.update(override)
    return make_case(f"config{idx}", seed=seed, **kw)


# ------------------------------------------------------------------------------------------------
# whole layers: every projection the configuration names, over one batch of tokens
# ------------------------------------------------------------------------------------------------
MODULE_NAMES = ("q", "k", "v", "o", "gate", "up", "down")     # LoraModule::ALL order (crates/spark-model/src/lora/types.rs:30-38)


@dataclass
class LayerCase:
    """The projections of one transformer layer over one token batch.

    `projections[i].meta` carries {"module": index into MODULE_NAMES, "input": name of the activation
    tensor it reads}; projections that read the same activations (q/k/v; gate/up) share one array.
    Every projection has its own NVFP4 weight and its own A/B per adapter slot; seq_slot is shared."""
    name: str
    dims: dict                         # hidden_size, intermediate_size, num_attention_heads, num_key_value_heads, head_dim
    M: int
    max_rank: int
    max_loras: int
    seq_slot: np.ndarray
    projections: List[Case]
    inputs: dict                       # name -> [M, K] bf16 bits

    @property
    def ranks(self):
        return [None if a is None else a.rank for a in self.projections[0].adapters]


def _slots(seed, M, n_ad, ids, segments, none_frac):
    return make_case("ids", M=M, K=16, N=16, ranks=[1] * n_ad, max_rank=16, ids=ids, segments=segments,
                     none_frac=none_frac, seed=seed).seq_slot


def make_layer(name: str, *, dims: dict, modules, M: int, ranks: List[int], max_rank: int, ids: str, segments: int = 0,
               none_frac: float = 0.0, seed: int = 1, max_loras: Optional[int] = None, alpha_over_r: float = 2.0,
               b_std: float = 0.02, scale2: float = 1.0) -> LayerCase:
    h, inter = dims["hidden_size"], dims["intermediate_size"]
    qw, kvw = dims["num_attention_heads"] * dims["head_dim"], dims["num_key_value_heads"] * dims["head_dim"]
    shape = {"q": (qw, h, "x_attn"), "k": (kvw, h, "x_attn"), "v": (kvw, h, "x_attn"), "o": (h, qw, "x_o"),
             "gate": (inter, h, "x_mlp"), "up": (inter, h, "x_mlp"), "down": (h, inter, "x_down")}
    n_ad = len(ranks)
    max_loras = max_loras or n_ad
    slot = _slots(seed, M, n_ad, ids, segments, none_frac)
    inputs, projs = {}, []
    for mi, mod in enumerate(MODULE_NAMES):
        if mod not in modules:
            continue
        N, K, xin = shape[mod]
        if xin not in inputs:
            inputs[xin] = f32_to_bf16_bits(normal(seed * 1000 + 11 + len(inputs), M * K)).reshape(M, K)
        adapters: List[Optional[Adapter]] = [None] * max_loras
        for s, r in enumerate(ranks):
            adapters[s] = make_adapter(seed * 1000 + 100 + 13 * s + 1009 * (mi + 1), K, N, r, alpha_over_r * r, b_std)
        c = Case(f"{name}/{mod}", M, K, N, max_rank, max_loras, inputs[xin], slot, adapters, scale2=scale2,
                 meta={"module": mi, "input": xin})
        c.packed, c.scales = make_nvfp4_weight(seed * 1000 + 50 + 7 * mi, N, K)
        projs.append(c)
    return LayerCase(name, dims, M, max_rank, max_loras, slot, projs, inputs)


LLAMA3_8B = dict(hidden_size=4096, intermediate_size=14336, num_attention_heads=32, num_key_value_heads=8, head_dim=128)
LLAMA_70B = dict(hidden_size=8192, intermediate_size=28672, num_attention_heads=64, num_key_value_heads=8, head_dim=128)


def layer_config(idx: int, seed: int = 1, **override) -> LayerCase:
    """Benchmark configurations 3 and 4 as they are written: every projection of the layer.

    3: Llama-3-8B-shaped layer, q/k/v/o/gate/up/down NVFP4 linears, 8192 tokens in 32 contiguous segments of
       random length, 8 adapters of rank 64 on all seven projections.
    4: 70B-shaped MLP (gate, up, down), 512 tokens, 128 adapters of rank 16 with Zipf(1.1) ids, 25 % adapter-less.
    2: the decode batch's fused QKV as its three LoRA modules (q 4096 | k 1024 | v 1024 of one 6144-wide output)."""
    if idx == 3:
        kw = dict(dims=LLAMA3_8B, modules=MODULE_NAMES, M=8192, ranks=[64] * 8, max_rank=64, ids="segments", segments=32)
    elif idx == 4:
        kw = dict(dims=LLAMA_70B, modules=("gate", "up", "down"), M=512, ranks=[16] * 128, max_rank=16, ids="zipf", none_frac=0.25)
    elif idx == 2:
        rk = [(8, 16, 32, 64)[int(v)] for v in (uniform01(seed * 77 + 9, 64) * 4).astype(np.int32).clip(0, 3)]
        kw = dict(dims=LLAMA3_8B, modules=("q", "k", "v"), M=64, ranks=rk, max_rank=64, ids="distinct")
    else:
        raise ValueError(idx)
    kw.update(override)
    return make_layer(f"config{idx}-layer", seed=seed, **kw)
