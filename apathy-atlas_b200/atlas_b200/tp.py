"""Column-parallel split of the layer over `tp` ranks (one GPU each).

Rank r owns output rows [r*N/tp, (r+1)*N/tp) of the packed weight, of its block scales and of every
B_s (contiguous slices, as `shard_quantized_nvfp4` ColumnParallel does for the base weight,
crates/spark-model/src/tp_shard/quant_shard.rs:57-90); scale2, x, seq_slot, every A_s and the scale
table are replicated, so the shrink is recomputed on every rank and the only exchange is one
all-gather of the [M, N/tp] output shards.  The gathered tensor is laid out [tp, M, N/tp]
(`gathered_to_row_major` gives the [M, N] view).
"""
from __future__ import annotations

import copy

import numpy as np

from . import synth


def shard_case(case: synth.Case, tp: int, rank: int) -> synth.Case:
    """Host-side shard of a synthetic case (numpy slices; A and x are shared, not copied)."""
    if case.N % tp != 0:
        raise ValueError(f"N={case.N} is not divisible by tp={tp}")
    n_loc = case.N // tp
    lo, hi = rank * n_loc, (rank + 1) * n_loc
    c = copy.copy(case)
    c.N = n_loc
    c.name = f"{case.name}/tp{tp}r{rank}"
    if case.packed is not None:
        c.packed, c.scales = case.packed[lo:hi], case.scales[lo:hi]
    if case.w_bf16 is not None:
        c.w_bf16 = case.w_bf16[lo:hi]
    c.adapters = [None if a is None else synth.Adapter(a.a, a.b[lo:hi], a.scale, a.rank) for a in case.adapters]
    return c


def token_shard(M: int, tp: int, rank: int, align: int = 64):
    """(row_begin, row_count) of rank `rank`'s share of the M tokens for the token-sharded shrink: equal shares rounded
    up to `align` rows (the shrink kernel's rows per CTA), the last ranks taking what is left (possibly nothing)."""
    if tp < 1 or not 0 <= rank < tp:
        raise ValueError(f"rank {rank} of {tp}")
    per = (-(-M // tp) + align - 1) // align * align
    begin = min(rank * per, M)
    return begin, max(0, min(per, M - begin))


def gathered_to_row_major(y_all: np.ndarray) -> np.ndarray:
    """[tp, M, N/tp] (all-gather order) -> [M, N]."""
    tp, M, n_loc = y_all.shape
    return np.ascontiguousarray(y_all.transpose(1, 0, 2)).reshape(M, tp * n_loc)


class DeviceShard:
    """This rank's tensors resident on the current CUDA device, and the call descriptor over them."""

    def __init__(self, torch, ab, case: synth.Case, tp: int, rank: int):
        self.ab, self.torch = ab, torch
        self.local_case = lc = shard_case(case, tp, rank) if tp > 1 else case
        self.n_local = lc.N

        def dev(a):
            if a is None:
                return None
            if a.dtype == np.uint16:
                return torch.from_numpy(a.view(np.int16).copy()).cuda()
            return torch.from_numpy(np.ascontiguousarray(a)).cuda()

        self.x = dev(lc.x)
        self.seq_slot = dev(lc.seq_slot.astype(np.int32))
        self.packed, self.scales, self.w_bf16 = dev(lc.packed), dev(lc.scales), dev(lc.w_bf16)
        self.pool = ab.LoraPool(lc.K, lc.N, lc.max_rank, lc.max_loras)
        for s, ad in enumerate(lc.adapters):
            if ad is None:
                continue
            self.pool.a_pool[s, :ad.rank].copy_(dev(ad.a).view(torch.bfloat16))
            self.pool.b_pool[s, :, :ad.rank].copy_(dev(np.ascontiguousarray(ad.b)).view(torch.bfloat16))
            self.pool._a_host[s] = self.pool.a_pool[s].data_ptr()
            self.pool._b_host[s] = self.pool.b_pool[s].data_ptr()
            self.pool._scale_host[s] = ad.scale
            self.pool._rank_host[s] = ad.rank
        self.pool.refresh_tables()
        self.lora_t = torch.zeros((lc.M, lc.max_rank), dtype=torch.int16, device="cuda")

    def desc(self, y, extra_flags: int = 0, out_row_stride=None, y_dest=None, y_col_offset=0):
        """Call descriptor.  y_dest (a list of [M, out_row_stride] buffers, one per rank) makes the kernel store
        this shard's columns into every one of them at y_col_offset instead of into `y`."""
        lc = self.local_case
        # scratch: the FP4 activations (when asked for), then the LoRA activation tiles.  Sized once for the larger
        # mode: descriptors keep raw addresses, so this buffer must never be replaced once one has been built.
        ws_bytes = self.ab.lora_ws_bytes(lc.M, lc.max_loras, lc.max_rank)
        if extra_flags & self.ab.FLAG_ACT_FP4:
            ws_bytes += (self.ab.act_fp4_ws_bytes(lc.M, lc.K) + 255) // 256 * 256
        if getattr(self, "_ws", None) is None:
            cap = self.ab.lora_ws_bytes(lc.M, lc.max_loras, lc.max_rank) + (self.ab.act_fp4_ws_bytes(lc.M, lc.K) + 255) // 256 * 256
            self._ws = self.torch.empty(cap, dtype=self.torch.uint8, device="cuda")
        assert self._ws.numel() >= ws_bytes
        ws = self._ws
        return self.ab.make_linear_desc(ws=ws, ws_bytes=ws_bytes, y_dest=y_dest, y_col_offset=y_col_offset,
            x=self.x, m=lc.M, k=lc.K, n=lc.N, y=y, w_packed=self.packed, w_scale=self.scales, scale2=lc.scale2,
            w_bf16=self.w_bf16, seq_slot=self.seq_slot, route=self.pool.route(), lora_t=self.lora_t,
            flags=extra_flags, out_row_stride=out_row_stride)


class DeviceLayer:
    """Every projection of a `synth.LayerCase` resident on the current CUDA device, column-sharded for rank `rank`
    of `tp`, over ONE slot-major adapter pool in the reference's layout (`registry.LoraWeights`).

    Activations, seq_slot, the whole pool (A and B of every slot) and the scale table are replicated on every rank;
    a rank's B_s rows are addressed inside the replicated pool by offsetting the module's B table and pool base."""

    def __init__(self, torch, ab, layer: synth.LayerCase, tp: int = 1, rank: int = 0):
        from . import registry
        self.torch, self.ab, self.layer, self.tp, self.rank = torch, ab, layer, tp, rank

        def dev(a):
            if a.dtype == np.uint16:
                return torch.from_numpy(a.view(np.int16)).cuda()
            return torch.from_numpy(np.ascontiguousarray(a)).cuda()

        self.inputs = {k: dev(v) for k, v in layer.inputs.items()}
        self.seq_slot = dev(layer.seq_slot.astype(np.int32))
        d = layer.dims
        self.cfg = registry.model_dims(d["hidden_size"], d["intermediate_size"], d["num_attention_heads"],
                                       d["num_key_value_heads"], d["head_dim"])
        self.weights = registry.LoraWeights(self.cfg, layer.max_loras, layer.max_rank)
        for s in range(layer.max_loras):
            mods = {(0, c.meta["module"]): (c.adapters[s].a, c.adapters[s].b) for c in layer.projections
                    if c.adapters[s] is not None}
            if mods:
                self.weights.pack_slot(s, mods, next(c.adapters[s].scale for c in layer.projections if c.adapters[s] is not None))
        self.proj = []
        for c in layer.projections:
            if c.N % tp != 0:
                raise ValueError(f"{c.name}: N={c.N} is not divisible by tp={tp}")
            n_loc = c.N // tp
            lo = rank * n_loc
            self.proj.append(dict(case=c, n_local=n_loc, row_begin=lo, x=self.inputs[c.meta["input"]],
                                  packed=dev(c.packed[lo:lo + n_loc]), scales=dev(c.scales[lo:lo + n_loc]),
                                  route=self.weights.route(0, c.meta["module"], lo, n_loc),
                                  lora_t=torch.zeros((c.M, c.max_rank), dtype=torch.int16, device="cuda"),
                                  ws=torch.empty(ab.lora_ws_bytes(c.M, c.max_loras, c.max_rank) +
                                                 (ab.act_fp4_ws_bytes(c.M, c.K) + 255) // 256 * 256,
                                                 dtype=torch.uint8, device="cuda")))

    def local_case(self, i: int) -> synth.Case:
        """Host-side view of projection i's shard (for the algorithmic-work figures)."""
        return shard_case(self.proj[i]["case"], self.tp, self.rank) if self.tp > 1 else self.proj[i]["case"]

    def desc(self, i: int, y, extra_flags: int = 0, out_row_stride=None, y_dest=None, y_col_offset=0, x=None, seq_slot=None):
        pr = self.proj[i]
        c = pr["case"]
        return self.ab.make_linear_desc(
            ws=pr["ws"], ws_bytes=pr["ws"].numel(), y_dest=y_dest, y_col_offset=y_col_offset,
            x=pr["x"] if x is None else x, m=c.M, k=c.K, n=pr["n_local"], y=y, w_packed=pr["packed"], w_scale=pr["scales"],
            scale2=c.scale2, seq_slot=self.seq_slot if seq_slot is None else seq_slot, route=pr["route"], lora_t=pr["lora_t"],
            flags=extra_flags, out_row_stride=out_row_stride)
