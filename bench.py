#!/usr/bin/env python
"""Benchmark of the fused NVFP4 + multi-LoRA linear layer.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload config3-layer] [--impl reference]

One step = one pass of every projection of the workload over one synthetic token batch, one fused call
(shrink + tcgen05 kernel) per projection.  The default workload is the 8B-shape multi-adapter prefill layer:
q/k/v/o/gate/up/down NVFP4 linears of a Llama-3-8B-shaped layer (hidden 4096, intermediate 14336, GQA 32/8,
head_dim 128), 8192 tokens in 32 contiguous segments of random length, 8 adapters of rank 64 on all seven
projections, the adapters in one slot-major pool laid out as the reference lays its pool out.  Other workloads:
config4-mlp (70B-shaped gate/up/down, 512 tokens, 128 adapters of rank 16 with Zipf ids), config2-qkv (decode batch,
q/k/v LoRA modules into column segments of one fused-QKV output) and the single linears config0..config4.

With N > 1 (launched by torch.distributed.run, one rank per GPU) every projection is split column-parallel over
the ranks — W, its scales and every B_s by output rows; x, A_s and seq_slot replicated: strong scaling.  Every
rank's gathered [M, N] buffers live in symmetric memory mapped into every process.  `--collective fused`: the kernel's
own store phase writes each tile into all ranks' buffers; `--collective push`: a projection's kernels store into the
rank's own buffer and a small copy kernel on a second stream sends those columns to the peers over NVLink while the next
projection computes (`copy`: the same by the copy engines); `--collective auto` (default) takes the first where the
rank's share runs as the persistent kernel and the second where it is a single wave of tiles.  What remains of the
collective is one device-side barrier per step.  From four ranks on (`--gather consumer`, default) gate and up stay on
their rank, which applies SwiGLU to its own columns, and h = silu(gate) * up is gathered instead of the two.
`--collective nccl` (or a box where the peer mapping cannot be made) runs the projections followed by one NCCL
all-gather each instead.

Rank 0 prints one JSON line.  `value` is device-timed (CUDA events on the launching stream, L2 flushed between
steps, inputs resident in HBM); `e2e` runs the same calls with host buffers, with the H2D copies of the step's
inputs and the D2H copies of its results inside the timed region.  `--impl reference` times the CPU oracle (a
scalar restatement of the reference's launch sequence — the reference itself is Rust + GB10 CUDA and has no CPU
build of this path) on a bounded row sample with all host threads.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "apathy-atlas_b200"))

import numpy as np

METRIC = "NVFP4+multi-LoRA linear tokens/s"
FP4_PEAK_TFLOPS = 9000.0          # B200 dense NVFP4, nominal (no measured figure on this pool)
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel instance, from the ncu captures
# summarised under profiles/ (per workload and activation mode; absent = no capture)
NCU_TRAFFIC_BYTES = {
    # (workload, dominant projection, activations)
    ("config3-layer", "gate", "bf16"): 432.6e6,      # persistent kernel <192, 2, A16>
    ("config3-layer", "gate", "fp4"): 336.8e6,       # persistent kernel <256, 1, A4>
    ("config4-mlp", "gate", "bf16"): 409.1e6,        # persistent kernel <256, 1, A16>
    ("config1", "config1", "bf16"): 73.1e6,          # one-tile kernel <256>
    ("config2", "config2", "bf16"): 66.1e6,          # one-tile kernel <64>
    ("config0", "config0", "bf16"): 33.7e6,          # dense BF16 kernel <16>
}
WORKLOADS = {
    "config3-layer": dict(kind="layer", idx=3),
    "config4-mlp": dict(kind="layer", idx=4),
    "config2-qkv": dict(kind="layer", idx=2, fused_out=True),
    "config0": dict(kind="single", idx=0), "config1": dict(kind="single", idx=1), "config2": dict(kind="single", idx=2),
    "config3": dict(kind="single", idx=3), "config4": dict(kind="single", idx=4),
}
DEFAULT_WORKLOAD = "config3-layer"


def peaks():
    """(HBM GB/s, dense BF16 TFLOP/s of a kernel timed alone, the same inside a long step, "measured" | "fallback")."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def algorithmic_work(case):
    """Bytes and flops of one pass of one projection, each tensor counted once (adapters at their true rank)."""
    M, N, K = case.M, case.N, case.K
    w_bytes = N * K * 2 if case.w_bf16 is not None else N * K * (0.5 + 1.0 / 16.0)
    slots = np.asarray(case.seq_slot)
    hit, counts = np.unique(slots[slots >= 0], return_counts=True)
    a_bytes = sum(case.adapters[int(s)].rank * K * 2 for s in hit)
    b_bytes = sum(case.adapters[int(s)].rank * N * 2 for s in hit)
    x_bytes, y_bytes, slot_bytes = M * K * 2, M * N * 2, 4 * M
    flops = 2.0 * M * N * K + 2.0 * sum(int(c) * case.adapters[int(s)].rank * (K + N) for s, c in zip(hit, counts))
    return dict(w=w_bytes, a=a_bytes, b=b_bytes, x=x_bytes, y=y_bytes, slot=slot_bytes,
                total=w_bytes + a_bytes + b_bytes + x_bytes + y_bytes + slot_bytes, flops=flops,
                main_kernel=w_bytes + b_bytes + x_bytes + y_bytes + slot_bytes)


def total_work(cases):
    w = [algorithmic_work(c) for c in cases]
    return {k: sum(d[k] for d in w) for k in w[0]}


class HostWork:
    """The workload on the host: its projections (synth.Case each), their shared inputs and seq_slot."""

    def __init__(self, name, only=None):
        from atlas_b200 import synth
        spec = WORKLOADS[name]
        self.name, self.kind, self.fused_out = name, spec["kind"], bool(spec.get("fused_out"))
        if self.kind == "layer":
            self.layer = synth.layer_config(spec["idx"], **({"modules": tuple(only)} if only else {}))
            self.projections, self.inputs, self.seq_slot = self.layer.projections, self.layer.inputs, self.layer.seq_slot
        else:
            case = synth.baseline_config(spec["idx"])
            case.meta = {"module": 0, "input": "x"}
            self.layer = None
            self.projections, self.inputs, self.seq_slot = [case], {"x": case.x}, case.seq_slot
        self.M = self.projections[0].M
        self.n_total = sum(c.N for c in self.projections)
        self.nvfp4 = all(c.packed is not None for c in self.projections)

    def config(self, args, tp):
        c0 = self.projections[0]
        slots = np.asarray(self.seq_slot)
        return {"workload": self.name, "M": self.M,
                "projections": [{"name": c.name.split("/")[-1], "K": c.K, "N": c.N} for c in self.projections],
                "base": "nvfp4" if self.nvfp4 else "bf16",
                "adapters": sum(a is not None for a in c0.adapters), "adapters_hit": int(len(np.unique(slots[slots >= 0]))),
                "max_rank": c0.max_rank, "adapter_less_rows": int((slots < 0).sum()),
                "segments": int((np.diff(slots) != 0).sum() + 1),
                "adapter_pool": "slot-major pool, slot k at k * pool_slot_bytes (reference layout)" if self.kind == "layer"
                                else "one-module pool",
                "activation_mode": "A4 (x quantised to NVFP4)" if getattr(args, "activations", "bf16") == "fp4" else "A16 (exact BF16 x)",
                "parallelism": (f"column-parallel tp{tp}, " + getattr(args, "collective_used", "all-gather")) if tp > 1 else "single GPU",
                "l2": "flushed between timed steps", "seed": 1}


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self._stop_evt = index, [], threading.Event()

    def run(self):
        while not self._stop_evt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                self.rows.append([c.strip() for c in out.strip().split(",")])
            except Exception:
                pass
            self._stop_evt.wait(0.2)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=6)
        sm, mx, reasons, power = [], 0.0, set(), []
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1])); power.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------------
# CPU arm: the oracle on host cores
# --------------------------------------------------------------------------------------------------
def cpu_sample(work, rows):
    """The reference's launch sequence (base linear, then staged routed LoRA) for every projection of the workload,
    on the first `rows` tokens, with every host thread.  Returns (step() -> seconds, rows, threads)."""
    from oracle import oracle_ctypes as oc
    cores = oc.set_num_threads(0)          # launchers export OMP_NUM_THREADS=1; the baseline uses every core
    rows = max(1, min(rows, work.M))
    prepared = []
    for c in work.projections:
        pool = oc.HostPool(c.K, c.N, c.max_rank, c.max_loras)
        for s, ad in enumerate(c.adapters):
            if ad is not None:
                pool.pack(s, ad.a, ad.b, ad.scale)
        prepared.append((c, np.ascontiguousarray(c.x[:rows]), np.ascontiguousarray(c.seq_slot[:rows]), pool))

    def step():
        t0 = time.perf_counter()
        for c, x, slot, pool in prepared:
            oc.reference_sequence(x, rows, c.N, c.K, packed=c.packed, scales=c.scales, scale2=c.scale2, w_bf16=c.w_bf16,
                                  seq_slot=slot, pool=pool)
        return time.perf_counter() - t0
    return step, rows, cores


def default_cpu_rows(work):
    """Rows whose pass costs the host a few seconds (about 1e9 multiply-adds per second and core)."""
    macs_per_row = sum(c.N * c.K for c in work.projections)
    return max(1, min(work.M, int(2.0e10 / macs_per_row)))


def run_reference_arm(args, work):
    """The CPU port of the reference's launch sequence, timed on this box's host cores: each step is one pass over a
    fixed row sample of the workload; `ms_per_step` is the measured time of that sample, `value` = rows / time."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    rows = args.cpu_rows or default_cpu_rows(work)
    step, rows, cores = cpu_sample(work, rows)
    for _ in range(args.warmup):
        step()
    times = [step() for _ in range(args.steps)]
    t = float(np.mean(times))
    tok_s = rows / t
    sample = (f"first {rows} of {work.M} tokens x all outputs of all {len(work.projections)} projections, every step "
              f"(ms_per_step is the measured time of that sample, not extrapolated)")
    args.activations = "bf16"
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": work.config(args, 1),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
class DevWork:
    """The workload resident on this rank's GPU: per projection the column shard, its scratch and descriptors."""

    def __init__(self, torch, ab, work, tp, rank):
        from atlas_b200 import tp as tpmod
        self.torch, self.ab, self.work, self.tp, self.rank = torch, ab, work, tp, rank
        if work.kind == "layer":
            self.dl = tpmod.DeviceLayer(torch, ab, work.layer, tp, rank)
            self.inputs, self.seq_slot = self.dl.inputs, self.dl.seq_slot
            self.n_local = [p["n_local"] for p in self.dl.proj]
            self.local_cases = [self.dl.local_case(i) for i in range(len(self.n_local))]
            # Projections that read the same activations (q/k/v; gate/up) run one after the other over ONE scratch: the
            # first one's quantised activations (FP4 mode) serve the others, which skip the quantiser
            # (ATLAS_B200_FLAG_ACT_FP4_READY); each call's shrink overwrites the LoRA-tile part with its own tiles.
            # (One GPU only: with N > 1 the scratch of every projection is a symmetric buffer of its own.)
            self.shares_x_with = {}
            if tp == 1:
                first = {}
                for i, c in enumerate(work.projections):
                    key = c.meta["input"]
                    if key in first and self.dl.proj[first[key]]["ws"].numel() == self.dl.proj[i]["ws"].numel():
                        self.dl.proj[i]["ws"] = self.dl.proj[first[key]]["ws"]
                        self.shares_x_with[i] = first[key]
                    first.setdefault(key, i)
        else:
            self.shares_x_with = {}
            self.ds = tpmod.DeviceShard(torch, ab, work.projections[0], tp, rank)
            self.inputs, self.seq_slot = {"x": self.ds.x}, self.ds.seq_slot
            self.n_local = [self.ds.n_local]
            self.local_cases = [self.ds.local_case]
        self.n = len(self.n_local)

    def desc(self, i, y, flags=0, x=None, seq_slot=None, **place):
        if self.work.kind == "layer":
            if (flags & self.ab.FLAG_ACT_FP4) and i in self.shares_x_with:
                flags |= self.ab.FLAG_ACT_FP4_READY
            return self.dl.desc(i, y, extra_flags=flags, x=x, seq_slot=seq_slot, **place)
        d = self.ds.desc(y, extra_flags=flags, **place)
        if x is not None:
            d.x = x.data_ptr()
        if seq_slot is not None:
            d.seq_slot = seq_slot.data_ptr()
        return d


def run_lora_bgmv(args, torch, ab, work, dw, outs, out_stride, flush):
    """The routed LoRA op alone: out[i] += scale_s B_s (A_s x[i]) in place, reference rounding (two launches per projection)."""
    M = work.M
    for o in outs:
        o.zero_()
    routes, xs = [], []
    for i, c in enumerate(work.projections):
        if work.kind == "layer":
            routes.append(dw.dl.proj[i]["route"]); xs.append(dw.dl.proj[i]["x"])
        else:
            routes.append(dw.ds.pool.route()); xs.append(dw.ds.x)
    xa = [torch.zeros((M, c.max_rank), dtype=torch.int16, device=outs[0].device) for c in work.projections]
    stream = torch.cuda.current_stream()

    def step():
        for i, c in enumerate(work.projections):
            ab.apply_lora_bgmv(routes[i], xs[i], outs[i], dw.seq_slot, M, c.K, out_stride or c.N, xa[i], stream)
    for _ in range(args.warmup):
        flush.fill_(1)
        step()
    torch.cuda.synchronize()
    if ab.device_status() != 0:
        raise RuntimeError("device status word set after warm-up")
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in ev:
        flush.fill_(1)
        a.record(stream)
        step()
        b.record(stream)
    torch.cuda.synchronize()
    ms = float(np.mean([a.elapsed_time(b) for a, b in ev]))
    hbm_gbs, _, _, peak_kind = peaks()
    # bytes of the op: x, A and B of the adapters hit at their true rank, the routed rows of out read and written, seq_slot, xa
    byts = 0.0
    for c in work.projections:
        w = algorithmic_work(c)
        routed = int((np.asarray(c.seq_slot) >= 0).sum())
        byts += w["x"] + w["a"] + w["b"] + 2 * routed * c.N * 2 + w["slot"] + 2 * routed * c.max_rank * 2
    line = {"metric": "routed LoRA op (apply_lora_bgmv) tokens/s", "op": "lora_bgmv", "value": M / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "config": work.config(args, 1),
            "roofline": {"bound": "hbm", "achieved": byts / (ms * 1e-3) / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                         "frac": byts / (ms * 1e-3) / 1e9 / hbm_gbs, "peak_kind": f"{peak_kind} HBM copy", "algorithmic_bytes": byts,
                         "kernel": "lora_shrink_* + lora_expand_fold_kernel (whole op)"},
            "gpu_launches": args.steps * 2 * len(work.projections)}
    print(json.dumps(line), flush=True)


def run_qkv_epilogue(args, form):
    """The consumers of the fused QKV projection on the Llama-3-8B shape of the default workload (8192 tokens, 32 Q + 8 KV
    heads of 128, rotary 64, pages of 16): `prefill` = K norm + RoPE + paged K cache write and V cache write
    (atlas_b200_kv_norm_rope_cache_write); `decode` = Q norm + RoPE in place, K into the cache, V copied
    (atlas_b200_qkv_norm_rope_cache_write).  K and V (and Q) are read in place from [tokens, q | k | v] buffers; six sets of
    buffers (600 MB) are rotated so that no launch finds its input in L2.  One GPU."""
    import torch
    import atlas_b200 as ab
    torch.cuda.set_device(0)
    tokens, nq, nkv, hd, rot, bs, n_set = 8192, 32, 8, 128, 64, 16, 6
    stride = (nq + 2 * nkv) * hd
    g = torch.Generator(device="cuda").manual_seed(1)
    qkv = [torch.randn((tokens, stride), device="cuda", generator=g).to(torch.bfloat16) for _ in range(n_set)]
    wq = (torch.randn(hd, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    wk = (torch.randn(hd, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    pos = torch.arange(tokens, dtype=torch.int32, device="cuda")
    slot = torch.arange(tokens, dtype=torch.int64, device="cuda")
    inv_freq = torch.tensor((1e6 ** (-2.0 * np.arange(rot // 2) / rot)).astype(np.float32), device="cuda")
    caches = [(torch.empty((tokens // bs, bs, nkv, hd), dtype=torch.bfloat16, device="cuda"),
               torch.empty((tokens // bs, bs, nkv, hd), dtype=torch.bfloat16, device="cuda")) for _ in range(n_set)]
    stream = torch.cuda.current_stream()

    def step(i):
        b, (kc, vc) = qkv[i % n_set], caches[i % n_set]
        k_at, v_at = b.data_ptr() + nq * hd * 2, b.data_ptr() + (nq + nkv) * hd * 2
        if form == "prefill":
            ab.kv_norm_rope_cache_write(k_at, v_at, stride, wk, pos, slot, kc, vc, tokens, nkv, hd, rot, bs, 1e-6, 1e6, stream)
        else:
            ab.qkv_norm_rope_cache_write(b.data_ptr(), k_at, v_at, stride, stride, wq, wk, pos, inv_freq, slot, kc, vc, tokens, nq, nkv, hd, rot,
                                         bs, 1e-6, 1.0, True, stream)
    for i in range(max(args.warmup, n_set)):
        step(i)
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for i, (a, b) in enumerate(ev):
        a.record(stream)
        step(i)
        b.record(stream)
    torch.cuda.synchronize()
    ms = float(np.mean([a.elapsed_time(b) for a, b in ev]))
    hbm_gbs, _, _, peak_kind = peaks()
    # bytes: K and V read and written once (prefill form); Q read and written in place as well (decode form)
    byts = float(tokens * hd * 2 * (4 * nkv + (2 * nq if form == "decode" else 0)))
    kernel = "kv_norm_rope_cache_kernel" if form == "prefill" else "qkv_norm_rope_cache_kernel"
    print(json.dumps({"metric": f"QKV consumer ({form} form) tokens/s", "op": f"qkv_epilogue_{form}", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16",
                      "data": "synthetic",
                      "config": {"workload": "qkv-epilogue", "tokens": tokens, "q_heads": nq, "kv_heads": nkv, "head_dim": hd, "rotary_dim": rot,
                                 "block_size": bs, "l2": f"{n_set} buffer sets rotated (600 MB)"},
                      "roofline": {"bound": "hbm", "achieved": byts / (ms * 1e-3) / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                                   "frac": byts / (ms * 1e-3) / 1e9 / hbm_gbs, "peak_kind": f"{peak_kind} HBM copy", "algorithmic_bytes": byts,
                                   "kernel": kernel},
                      "gpu_launches": args.steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="atlas_b200", choices=["atlas_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-rows", type=int, default=0, help="rows of the CPU sample (0: sized for a few seconds per pass)")
    ap.add_argument("--collective", default="auto", choices=["auto", "copy", "push", "fused", "nccl"],
                    help="N > 1: fused = the kernel's own store phase writes every tile into every rank's buffer; push = each "
                         "projection's columns copied to the peers by a small kernel on a second stream while the next projection "
                         "computes; copy = the same by the copy engines (one strided copy per peer, no SM involved); auto = fused where the rank's share runs as the persistent kernel (stores hidden under the next "
                         "tile), push where it is a single wave of tiles; nccl = all-gather after each projection")
    ap.add_argument("--gather", default="consumer", choices=["consumer", "outputs"],
                    help="N >= 4, layers with gate and up: consumer = SwiGLU on the rank's own columns of gate and up, then gather "
                         "h = silu(gate) * up (what the down projection reads) instead of both outputs; outputs = gather every output")
    ap.add_argument("--activations", default="bf16", choices=["bf16", "fp4"],
                    help="bf16: the layer as specified (exact activations); fp4: the opt-in W4A4 mode as the timed step")
    ap.add_argument("--op", default="fused", choices=["fused", "lora_bgmv", "qkv_epilogue_prefill", "qkv_epilogue_decode"],
                    help="fused: the fused layer (the benchmark); lora_bgmv: the routed LoRA op alone (shrink + expand/fold in place, "
                         "the reference's apply_lora_bgmv) on the workload's projections, 1 GPU; qkv_epilogue_*: the consumers of the fused "
                         "QKV projection (norm + RoPE + paged cache writes) on the 8B shape, 1 GPU")
    ap.add_argument("--only", default="", help="layer workloads: run these projections only, e.g. --only gate or --only q,k,v (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end loops (profiling runs)")
    ap.add_argument("--no-other-mode", action="store_true", help="skip the secondary activation-mode timing (profiling runs)")
    args = ap.parse_args()
    reference = args.impl == "reference"
    if args.steps is None:
        args.steps = 3 if reference else 30
    if args.warmup is None:
        args.warmup = 1 if reference else 5

    if args.op.startswith("qkv_epilogue_") and not reference:
        run_qkv_epilogue(args, args.op[len("qkv_epilogue_"):])
        return
    work = HostWork(args.workload, only=[m for m in args.only.split(",") if m] or None)
    if reference:
        run_reference_arm(args, work)
        return

    # peer mappings without an NVLink multicast object bound to them (plain loads and stores only)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch
    import atlas_b200 as ab
    ab.lib()                                      # fail loudly when the CUDA library is missing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        dist = None
        torch.cuda.set_device(0)
    assert args.warmup >= 3, "at least 3 warm-up steps"
    tp = world
    dev = torch.device("cuda", local_rank)
    M = work.M

    dw = DevWork(torch, ab, work, tp, rank)
    n_proj = dw.n
    # Output buffers.  One [M, n_local] per projection — or, for the fused-QKV workload, column segments of one
    # [M, sum n_local] buffer (the reference's strided QKV layout).
    cols0 = np.concatenate([[0], np.cumsum(dw.n_local)]).astype(int)
    full_cols0 = np.concatenate([[0], np.cumsum([c.N for c in work.projections])]).astype(int)

    def make_outputs():
        if work.fused_out:
            buf = torch.empty((M, int(cols0[-1])), dtype=torch.bfloat16, device=dev)
            return [buf[:, cols0[i]:cols0[i + 1]] for i in range(n_proj)], buf
        return [torch.empty((M, dw.n_local[i]), dtype=torch.bfloat16, device=dev) for i in range(n_proj)], None
    y_loc, y_loc_buf = make_outputs()
    loc_stride = int(cols0[-1]) if work.fused_out else None

    # fused collective: every rank's gathered result buffers, mapped into every process.  Two sets, used in turn:
    # a rank that has passed step i's barrier may start step i+1's stores while a slower rank still reads step i's
    # result, so consecutive steps must not write the same buffers.
    fused, sym_sets, collective_note = False, [], None
    if tp > 1 and args.collective in ("auto", "copy", "fused", "push"):
        try:
            import torch.distributed._symmetric_memory as symm_mem
            if hasattr(symm_mem, "enable_symm_mem_for_group"):
                try:
                    symm_mem.enable_symm_mem_for_group(dist.group.WORLD.group_name)
                except Exception:
                    pass
            for _ in range(2):
                if work.fused_out:
                    bufs = [symm_mem.empty((M, work.n_total), dtype=torch.bfloat16, device=dev)]
                else:
                    bufs = [symm_mem.empty((M, c.N), dtype=torch.bfloat16, device=dev) for c in work.projections]
                handles = [symm_mem.rendezvous(b, dist.group.WORLD) for b in bufs]
                ptrs = [[int(p) for p in h.buffer_ptrs] for h in handles]
                assert all(len(p) == tp and all(p) for p in ptrs)
                sym_sets.append(dict(bufs=bufs, handles=handles, ptrs=ptrs))
            fused = True
        except Exception as e:                     # no peer mapping on this box: the NCCL path still measures the layer
            collective_note = f"peer mapping unavailable ({type(e).__name__}: {e}); NCCL all-gather used"
        ok = torch.tensor([1 if fused else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        fused = bool(int(ok.item()))
    # push: the kernels store into this rank's own gathered buffer only; a copy kernel on a second stream sends each
    # projection's columns to the peers while the next projection computes
    push_proj = [fused and args.collective in ("push", "copy")] * n_proj          # per projection; "auto" decides below
    by_copy_engines = args.collective == "copy"
    sides = [torch.cuda.Stream(device=dev) for _ in range(min(tp - 1, 4))] if fused else []
    # Gather what the consumer needs: gate and up are read by nothing but the element-wise SwiGLU, and a rank owns the same
    # columns of both — so the rank applies SwiGLU to its own columns and the ranks gather h = silu(gate) * up (the down
    # projection's input, [M, intermediate]) instead of gate AND up: a third less to exchange for the 8B layer.
    names_all = [c.name.split("/")[-1] for c in work.projections]
    mlp_h = None
    # (from four ranks on, where the step is bound by the exchange; at two ranks it is bound by the arithmetic and the extra
    #  kernel and copies cost more than they save: 1.84 against 1.77 ms)
    if fused and args.gather == "consumer" and tp >= 4 and not work.fused_out and "gate" in names_all and "up" in names_all:
        gi_, ui_ = names_all.index("gate"), names_all.index("up")
        try:
            h_bufs = [symm_mem.empty((M, work.projections[gi_].N), dtype=torch.bfloat16, device=dev) for _ in sym_sets]
            h_handles = [symm_mem.rendezvous(b, dist.group.WORLD) for b in h_bufs]
            mlp_h = dict(gate=gi_, up=ui_, bufs=h_bufs, handles=h_handles, ptrs=[[int(p_) for p_ in h_.buffer_ptrs] for h_ in h_handles],
                         event=[torch.cuda.Event() for _ in sym_sets])
        except Exception as e:
            collective_note = f"h could not be mapped to the peers ({type(e).__name__}: {e}); every output is gathered"
    local_only = set((mlp_h["gate"], mlp_h["up"])) if mlp_h else set()      # projections whose output stays on the rank
    y_all = ([torch.empty((tp, M, dw.n_local[i]), dtype=torch.bfloat16, device=dev) for i in range(n_proj)]
             if tp > 1 else None)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # > L2 (126 MB)
    mode = ab.FLAG_ACT_FP4 if args.activations == "fp4" else 0

    if args.op == "lora_bgmv":
        run_lora_bgmv(args, torch, ab, work, dw, y_loc, loc_stride, flush)
        return

    def build_descs(flags, sym=None, outs=None, x_of=None, seq_slot=None):
        outs = outs or y_loc
        ds = []
        for i in range(n_proj):
            xin = None if x_of is None else x_of[work.projections[i].meta["input"]]
            if sym is not None:
                j = 0 if work.fused_out else i
                place = dict(y_dest=(sym["ptrs"][j] if not (push_proj[i] or i in local_only) else [sym["ptrs"][j][rank]]), out_row_stride=(work.n_total if work.fused_out else work.projections[i].N),
                             y_col_offset=(int(full_cols0[i]) if work.fused_out else 0) + rank * dw.n_local[i])
                ds.append(dw.desc(i, None, flags, x=xin, seq_slot=seq_slot, **place))
            else:
                ds.append(dw.desc(i, outs[i], flags, x=xin, seq_slot=seq_slot, out_row_stride=loc_stride))
        return ds

    # Token-sharded shrink (fused collective, prefill layers): the LoRA scratch of every projection lives in symmetric
    # memory; each rank shrinks its own 1/tp of the tokens and stores the tiles into every rank's scratch, one device
    # barrier, then the fused calls run with the shrink result reused — instead of tp identical shrinks over all of x.
    sharded_shrink, ws_sym = False, None
    if fused and work.kind == "layer":
        try:
            ws_bufs = [symm_mem.empty(pr["ws"].numel(), dtype=torch.uint8, device=dev) for pr in dw.dl.proj]
            ws_handles = [symm_mem.rendezvous(b, dist.group.WORLD) for b in ws_bufs]
            ws_ptrs = [[int(p) for p in h.buffer_ptrs] for h in ws_handles]
            for pr, b in zip(dw.dl.proj, ws_bufs):
                pr["ws"] = b
            ws_sym = dict(bufs=ws_bufs, handles=ws_handles, ptrs=ws_ptrs)
        except Exception as e:
            collective_note = f"scratch could not be mapped to the peers ({type(e).__name__}: {e}); every rank runs the whole shrink"
    if fused and args.collective == "auto":
        # which of this rank's shares run as the persistent kernel (the same on every rank: the shapes are)
        for i, d_ in enumerate(build_descs(mode, sym_sets[0])):
            ab.nvfp4_lora_linear(d_, torch.cuda.current_stream())
            push_proj[i] = i not in local_only and not ab.last_launch_shape()["persistent_tiles_per_pass"]
        torch.cuda.synchronize()
        dist.barrier()
    for i in local_only:
        push_proj[i] = False
    pushed = any(push_proj) or bool(mlp_h)
    descs = [build_descs(mode, s) for s in sym_sets] if fused else [build_descs(mode)]
    descs_reuse = [build_descs(mode | ab.FLAG_REUSE_SHRINK, s) for s in sym_sets] if fused else None
    from atlas_b200 import tp as tpmod
    row_begin, row_count = tpmod.token_shard(M, tp, rank)
    if ws_sym is not None:
        try:
            for i in range(n_proj):
                if row_count:
                    ab.lora_shrink_tiles(descs[0][i], row_begin, row_count, ws_sym["ptrs"][i])
            sharded_shrink = True
        except ab.AtlasError:
            sharded_shrink = False
        ok = torch.tensor([1 if sharded_shrink else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        sharded_shrink = bool(int(ok.item()))
    descs_plain = build_descs(mode)                                    # this rank's shard into its own buffers, no placement
    stream = torch.cuda.current_stream()
    step_no = [0]

    push_events = [[torch.cuda.Event() for _ in range(n_proj + 1)] for _ in range(2)] if pushed else None
    push_joins = [[torch.cuda.Event() for _ in sides] for _ in range(2)]
    shrink_streams = [torch.cuda.Stream(device=dev) for _ in range(n_proj)] if sharded_shrink else None
    shrink_fork = torch.cuda.Event()
    shrink_join = [torch.cuda.Event() for _ in range(n_proj)]

    def push_block(ptrs, n_row, col, width, event):
        """Columns [col, col + width) of this rank's buffer into the same columns of every peer's buffer (`ptrs`: the buffer
        on every rank), once `event` has passed.  The peers are taken in the order rank+1, rank+2, ...: at any moment every
        GPU is then the target of one sender, not of all."""
        peers = [(rank + o) % tp for o in range(1, tp)]
        for s_ in sides:
            s_.wait_event(event)
        if by_copy_engines:
            for o, r in enumerate(peers):           # one strided copy per peer, spread over the side streams (and so over copy engines)
                ab.push_columns(ptrs[rank] + col * 2, n_row, [ptrs[r] + col * 2], n_row, M, width, sides[o % len(sides)], copy_engines=True)
        else:
            ab.push_columns(ptrs[rank] + col * 2, n_row, [ptrs[r] + col * 2 for r in peers], n_row, M, width, sides[0])

    def push(k, i):
        """Projection i's columns of this rank's gathered buffer (set k) to the peers."""
        j = 0 if work.fused_out else i
        n_row = work.n_total if work.fused_out else work.projections[i].N
        col = (int(full_cols0[i]) if work.fused_out else 0) + rank * dw.n_local[i]
        push_block(sym_sets[k]["ptrs"][j], n_row, col, dw.n_local[i], push_events[k][i])

    def swiglu_and_push(k):
        """h = silu(gate) * up on this rank's columns (read from its own gate / up buffers of set k), then those columns to the peers."""
        gi_, ui_ = mlp_h["gate"], mlp_h["up"]
        n_loc, n_row, col = dw.n_local[gi_], work.projections[gi_].N, rank * dw.n_local[gi_]
        g_ptr, u_ptr = sym_sets[k]["ptrs"][gi_][rank] + col * 2, sym_sets[k]["ptrs"][ui_][rank] + col * 2
        ab.silu_mul(g_ptr, u_ptr, mlp_h["ptrs"][k][rank] + col * 2, M, n_loc, in_row_stride=n_row, out_row_stride=n_row, stream=stream)
        mlp_h["event"][k].record(stream)
        push_block(mlp_h["ptrs"][k], n_row, col, n_loc, mlp_h["event"][k])

    def step(marks=None):
        """One step.  `marks`: optional list that receives CUDA events recorded between the step's phases."""
        def mark():
            if marks is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record(stream)
                marks.append(e)
        k = step_no[0] % len(descs)
        step_no[0] += 1
        v = None
        mark()
        if sharded_shrink:
            # the projections' shrinks are independent and, with the tokens split over the ranks, each fills only a part
            # of the GPU: one stream each, so that they run side by side
            shrink_fork.record(stream)
            for i in range(n_proj):
                if row_count:
                    shrink_streams[i].wait_event(shrink_fork)
                    ab.lora_shrink_tiles(descs[k][i], row_begin, row_count, ws_sym["ptrs"][i], shrink_streams[i])
                    shrink_join[i].record(shrink_streams[i])
                    stream.wait_event(shrink_join[i])
            mark()
            ws_sym["handles"][0].barrier(channel=1)          # every rank's tiles are in every rank's scratch
            mark()
        if pushed:
            dd = descs_reuse[k] if sharded_shrink else descs[k]
            for i in range(n_proj):
                v = ab.nvfp4_lora_linear(dd[i], stream)
                if push_proj[i]:
                    push_events[k][i].record(stream)
                    push(k, i)
                if mlp_h and i == max(mlp_h["gate"], mlp_h["up"]):
                    swiglu_and_push(k)
            mark()
            for o, s_ in enumerate(sides):
                push_joins[k][o].record(s_)
                stream.wait_event(push_joins[k][o])
            mark()
            sym_sets[k]["handles"][0].barrier(channel=0)     # every rank's columns have landed in every buffer
            mark()
            return v
        if sharded_shrink:
            for i in range(n_proj):
                v = ab.nvfp4_lora_linear(descs_reuse[k][i], stream)
            mark()
            sym_sets[k]["handles"][0].barrier(channel=0)     # every rank's output tiles have landed in every buffer
            mark()
            return v
        for i in range(n_proj):
            v = ab.nvfp4_lora_linear(descs[k][i], stream)
            if tp > 1 and not fused:
                dist.all_gather_into_tensor(y_all[i].view(tp * M, dw.n_local[i]), y_loc[i] if not work.fused_out else y_loc[i].contiguous())
        if fused:
            sym_sets[k]["handles"][0].barrier(channel=0)     # every rank's tiles have landed in every buffer
        return v

    def barrier():
        if tp > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if fused:
        for s in sym_sets:
            for b in s["bufs"]:
                b.view(torch.int16).fill_(0x7FC0)       # NaN pattern: the warm-up must overwrite all of it
    variant = None
    for _ in range(max(args.warmup, 2 * len(descs))):
        flush.fill_(1)
        variant = step()
    barrier()
    launch_shape = ab.last_launch_shape()
    status = ab.device_status()
    if status != 0:
        raise RuntimeError(f"device status word {status:#x} after warm-up")
    if variant != ab.VARIANT_TCGEN05 and work.nvfp4:
        raise RuntimeError("the tcgen05 path did not run for this workload")

    # ---- the gathered result, checked: every rank's buffers must equal the concatenation of the ranks' own
    #      (unplaced) shard results, bit for bit; the shards travel by NCCL for this check only ----
    if tp > 1:
        for i in range(n_proj):
            ab.nvfp4_lora_linear(descs_plain[i], stream)
            mine = y_loc[i].contiguous()
            dist.all_gather_into_tensor(y_all[i].view(tp * M, dw.n_local[i]), mine)
        torch.cuda.synchronize()
        if fused:
            for s in sym_sets:
                for i in range(n_proj):
                    got = s["bufs"][0][:, int(full_cols0[i]):int(full_cols0[i + 1])] if work.fused_out else s["bufs"][i]
                    want = y_all[i].permute(1, 0, 2).reshape(M, tp * dw.n_local[i])
                    if i in local_only:                  # only the rank's own columns of gate / up are kept
                        lo_, hi_ = rank * dw.n_local[i], (rank + 1) * dw.n_local[i]
                        got, want = got[:, lo_:hi_], want[:, lo_:hi_]
                    if not torch.equal(got.contiguous().view(torch.int16), want.contiguous().view(torch.int16)):
                        raise RuntimeError(f"rank {rank}: gathered buffer of projection {i} differs from the ranks' own shard results")
            if mlp_h:
                # h on every rank = SwiGLU of the ranks' own gate / up shards, gathered (by NCCL for this check)
                gi_, ui_ = mlp_h["gate"], mlp_h["up"]
                n_loc = dw.n_local[gi_]
                h_loc = torch.empty((M, n_loc), dtype=torch.bfloat16, device=dev)
                ab.silu_mul(y_loc[gi_].contiguous(), y_loc[ui_].contiguous(), h_loc, M, n_loc, stream=stream)
                h_all = torch.empty((tp, M, n_loc), dtype=torch.bfloat16, device=dev)
                dist.all_gather_into_tensor(h_all.view(tp * M, n_loc), h_loc)
                torch.cuda.synchronize()
                want = h_all.permute(1, 0, 2).reshape(M, tp * n_loc).contiguous().view(torch.int16)
                for hb in mlp_h["bufs"]:
                    if not torch.equal(hb.view(torch.int16), want):
                        raise RuntimeError(f"rank {rank}: gathered h differs from SwiGLU of the ranks' own gate / up shards")

    # ---- device-timed steps ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for a, b in ev:
        flush.fill_(1)
        a.record(stream)
        step()
        b.record(stream)
    barrier()
    step_ms = float(np.mean([a.elapsed_time(b) for a, b in ev]))

    # ---- the phases of a step at N > 1 (token-sharded shrink, its barrier, the projections, what is left of the exchange) ----
    phase_ms = None
    if tp > 1 and sharded_shrink:
        rows_ = []
        for _ in range(min(args.steps, 10)):
            flush.fill_(1)
            mk = []
            step(mk)
            rows_.append(mk)
        barrier()
        names_ = (["shrink (this rank's tokens)", "barrier", "projections", "push tail", "barrier"] if pushed else
                  ["shrink (this rank's tokens)", "barrier", "projections + peer stores", "barrier"])
        pm = torch.tensor([float(np.mean([r[i].elapsed_time(r[i + 1]) for r in rows_])) for i in range(len(names_))],
                          dtype=torch.float64, device=dev)
        dist.all_reduce(pm, op=dist.ReduceOp.MAX)
        phase_ms = [{"phase": n_, "ms": float(v_)} for n_, v_ in zip(names_, pm.tolist())]

    # ---- per projection (fused call = shrink + main kernel), then the dominant kernel instance alone with the
    #      shrink result reused: the roofline's kernel ----
    n_sub = min(args.steps, 20)
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(n_proj + 1)] for _ in range(n_sub)]
    for row in marks:
        flush.fill_(1)
        row[0].record(stream)
        for i in range(n_proj):
            ab.nvfp4_lora_linear(descs_plain[i], stream)
            row[i + 1].record(stream)
    barrier()
    proj_ms = [float(np.mean([row[i].elapsed_time(row[i + 1]) for row in marks])) for i in range(n_proj)]
    works_local = [algorithmic_work(c) for c in dw.local_cases]
    dom = int(np.argmax([w["flops"] for w in works_local]))
    desc_main_only = build_descs(mode | ab.FLAG_REUSE_SHRINK)[dom]
    ab.nvfp4_lora_linear(descs_plain[dom], stream)      # the scratch holds this projection's own tiles again
    ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_sub)]
    for a, b in ev2:
        flush.fill_(1)
        a.record(stream)
        ab.nvfp4_lora_linear(desc_main_only, stream)
        b.record(stream)
    barrier()
    main_ms = float(np.mean([a.elapsed_time(b) for a, b in ev2]))
    dom_shape = ab.last_launch_shape()
    dom_kernel = ("nvfp4_lora_linear_tc_persistent_kernel" if dom_shape.get("persistent_tiles_per_pass") else
                  ("nvfp4_lora_linear_tc_kernel" if work.nvfp4 else "dense_bf16_linear_tc_kernel"))

    # ---- the same step in the other activation mode (no collective), a secondary figure ----
    other_ms = float("nan")
    other = 0 if mode else ab.FLAG_ACT_FP4
    have_other = work.nvfp4 and all(c.K % 256 == 0 for c in work.projections) and not args.no_other_mode
    if have_other:
        descs_other = build_descs(other)
        for _ in range(3):
            for d in descs_other:
                ab.nvfp4_lora_linear(d, stream)
        ev3 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_sub)]
        for a, b in ev3:
            flush.fill_(1)
            a.record(stream)
            for d in descs_other:
                ab.nvfp4_lora_linear(d, stream)
            b.record(stream)
        barrier()
        other_ms = float(np.mean([a.elapsed_time(b) for a, b in ev3]))

    # ---- end to end through the C ABI with host buffers: every step copies its inputs (every activation tensor and
    #      seq_slot) from pinned host memory and copies its results back.  With N > 1 every rank uploads its own rows of
    #      the (replicated) activations, the ranks all-gather them over NVLink, and every rank reads back its own column
    #      shard of every result: the host traffic of the job is spread over the ranks' PCIe links. ----
    e2e_ms = e2e_serial_ms = float("nan")
    h2d = sum(int(v.size) * 2 for v in work.inputs.values()) + int(work.seq_slot.size) * 4
    d2h = sum(M * n * 2 for n in dw.n_local)
    if not args.no_e2e:
        x_host = {k: torch.from_numpy(v.view(np.int16)).pin_memory() for k, v in work.inputs.items()}
        slot_host = torch.from_numpy(work.seq_slot.astype(np.int32)).pin_memory()
        y_host = [torch.empty((M, n), dtype=torch.int16).pin_memory() for n in dw.n_local]

        def results(k):
            if not fused:
                return y_loc
            s = sym_sets[k]
            if work.fused_out:
                return [s["bufs"][0][:, int(full_cols0[i]) + rank * dw.n_local[i]: int(full_cols0[i]) + (rank + 1) * dw.n_local[i]] for i in range(n_proj)]
            return [s["bufs"][i][:, rank * dw.n_local[i]:(rank + 1) * dw.n_local[i]] for i in range(n_proj)]
        e2e_steps = max(3, min(args.steps, 10))
        shard_h2d = tp > 1 and M % tp == 0
        r0, r1 = (rank * (M // tp), (rank + 1) * (M // tp)) if shard_h2d else (0, M)
        if shard_h2d:
            h2d = sum((r1 - r0) * int(v.shape[1]) * 2 for v in work.inputs.values()) + int(work.seq_slot.size) * 4
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            if shard_h2d:
                # every rank uploads its own rows of each activation tensor over its own PCIe link; the ranks then
                # exchange the rows over NVLink (in-place all-gather: plumbing, NCCL)
                for k_, t_ in dw.inputs.items():
                    t_[r0:r1].copy_(x_host[k_][r0:r1], non_blocking=True)
                    dist.all_gather_into_tensor(t_.view(torch.bfloat16), t_[r0:r1].view(torch.bfloat16))
            else:
                for k_, t_ in dw.inputs.items():
                    t_.copy_(x_host[k_], non_blocking=True)
            dw.seq_slot.copy_(slot_host, non_blocking=True)
            k = step_no[0] % len(descs)
            step()
            for i, r_ in enumerate(results(k)):
                y_host[i].copy_(r_.view(torch.int16), non_blocking=True)
            barrier()
        e2e_ms = e2e_serial_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps

        # N > 1, as a serving loop would run it: the read-back of step i's results (set k of the rotating result buffers)
        # runs on its own stream while step i+1 uploads, gathers and computes into the other set; a step waits for the
        # read-back that last used the set it is about to overwrite.  Uploads and read-backs share no direction of PCIe.
        if tp > 1:
            def upload():
                if shard_h2d:
                    for k_, t_ in dw.inputs.items():
                        t_[r0:r1].copy_(x_host[k_][r0:r1], non_blocking=True)
                        dist.all_gather_into_tensor(t_.view(torch.bfloat16), t_[r0:r1].view(torch.bfloat16))
                else:
                    for k_, t_ in dw.inputs.items():
                        t_.copy_(x_host[k_], non_blocking=True)
                dw.seq_slot.copy_(slot_host, non_blocking=True)
            n_set = len(descs)
            s_out = torch.cuda.Stream(device=dev)
            ev_step = [torch.cuda.Event() for _ in range(n_set)]
            ev_out = [torch.cuda.Event() for _ in range(n_set)]
            y_hosts = [[torch.empty((M, n), dtype=torch.int16).pin_memory() for n in dw.n_local] for _ in range(n_set)]
            e2e_steps = max(6, min(args.steps, 16))
            barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                k = step_no[0] % n_set
                upload()
                # Set k is about to be overwritten — by this rank and, through their stores, by its peers: every rank's
                # read-back of set k must have finished first.  Each rank waits for its own, then the ranks meet (the
                # token-sharded shrink's barrier at the head of the step is that meeting; otherwise one is added).
                stream.wait_event(ev_out[k])
                if fused and not sharded_shrink:
                    sym_sets[k]["handles"][0].barrier(channel=2)
                step()
                ev_step[k].record(stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_step[k])
                    for i, r_ in enumerate(results(k)):
                        y_hosts[k][i].copy_(r_.view(torch.int16), non_blocking=True)
                    ev_out[k].record(s_out)
            barrier()
            # (a batch of a few hundred tokens is over before the second stream has been set up: the plain loop is then
            #  the faster way to run it, and the one reported)
            e2e_ms = min(e2e_serial_ms, (time.perf_counter() - t0) * 1e3 / e2e_steps)
            for i in range(n_proj):
                if not torch.equal(y_hosts[0][i], y_host[i]) or not torch.equal(y_hosts[-1][i], y_host[i]):
                    raise RuntimeError("the overlapped end-to-end loop read back something else than the serial one")

        # The same as a serving loop would run it on one GPU: two sets of device buffers, the copy of step i+1's
        # inputs and of step i-1's results on their own streams while step i computes.  Every step still carries
        # its own H2D and D2H copies inside the timed region; what changes is that the three overlap.
        if tp == 1:
            n_buf = 2
            e2e_steps = max(6, min(args.steps, 16))
            xs = [{k_: torch.empty_like(t_) for k_, t_ in dw.inputs.items()} for _ in range(n_buf)]
            slots = [torch.empty_like(dw.seq_slot) for _ in range(n_buf)]
            outs = [make_outputs()[0] for _ in range(n_buf)]
            y_hosts = [[torch.empty((M, n), dtype=torch.int16).pin_memory() for n in dw.n_local] for _ in range(n_buf)]
            dsets = [build_descs(mode, outs=outs[b], x_of=xs[b], seq_slot=slots[b]) for b in range(n_buf)]
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            ev_in = [torch.cuda.Event() for _ in range(n_buf)]
            ev_done = [torch.cuda.Event() for _ in range(n_buf)]
            ev_out = [torch.cuda.Event() for _ in range(n_buf)]
            barrier()
            t0 = time.perf_counter()
            for it in range(e2e_steps):
                b = it % n_buf
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_done[b])            # the step that last read these input buffers has finished
                    for k_ in xs[b]:
                        xs[b][k_].copy_(x_host[k_], non_blocking=True)
                    slots[b].copy_(slot_host, non_blocking=True)
                    ev_in[b].record(s_in)
                stream.wait_event(ev_in[b])
                stream.wait_event(ev_out[b])               # the copies that last read these output buffers have finished
                for d in dsets[b]:
                    ab.nvfp4_lora_linear(d, stream)
                ev_done[b].record(stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[b])
                    for i in range(n_proj):
                        y_hosts[b][i].copy_(outs[b][i].view(torch.int16), non_blocking=True)
                    ev_out[b].record(s_out)
            torch.cuda.synchronize()
            e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
            for i in range(n_proj):
                if not torch.equal(y_hosts[0][i], y_hosts[1][i]):
                    raise RuntimeError("the two buffer sets of the end-to-end loop disagree")
    clocks = sampler.stop()

    t = torch.tensor([step_ms, main_ms, e2e_ms, other_ms, e2e_serial_ms] + proj_ms, dtype=torch.float64, device=dev)
    if tp > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    vals = [float(v) for v in t.tolist()]
    step_ms, main_ms, e2e_ms, other_ms, e2e_serial_ms = vals[:5]
    proj_ms = vals[5:]

    names_p = [c.name.split("/")[-1] for c in work.projections]
    pushed_names = [n_ for i_, n_ in enumerate(names_p) if push_proj[i_]]
    stored_names = [n_ for i_, n_ in enumerate(names_p) if not push_proj[i_] and i_ not in local_only]
    mover = "the copy engines" if by_copy_engines else "a push kernel"
    if not fused:
        args.collective_used = "NCCL all-gather per projection"
    else:
        parts = []
        if stored_names:
            parts.append("tiles of " + ",".join(stored_names) + " stored into every rank's buffer by the kernel" + (" under its next tile" if pushed else ""))
        if pushed_names:
            parts.append("columns of " + ",".join(pushed_names) + f" copied into every rank's buffer by {mover} on a second stream beside the next "
                         "projection's kernels")
        if mlp_h:
            parts.append(f"gate and up stay on their rank: h = silu(gate) * up of the rank's columns is gathered instead ({mover})")
        parts.append("one device barrier per step")
        if sharded_shrink:
            parts.append("shrink sharded by tokens, its tiles stored into every rank's scratch + one device barrier")
        args.collective_used = "; ".join(parts)
    if rank == 0:
        hbm_gbs, bf16_burst, bf16_sustained, peak_kind = peaks()
        work_all = total_work(work.projections)
        dom_work = works_local[dom]
        # What bounds the dominant kernel: exact-BF16 activations run at the BF16 tensor rate, so a prefill tile is tensor-bound
        # against the measured BF16 GEMM peak of a kernel timed alone; a decode batch streams weights and is HBM-bound.  With FP4
        # activations the tensor peak is the nominal NVFP4 figure (no measured one on this pool).
        tensor_peak = FP4_PEAK_TFLOPS if mode else bf16_burst
        t_hbm = dom_work["main_kernel"] / (hbm_gbs * 1e9)
        t_tensor = dom_work["flops"] / (tensor_peak * 1e12)
        traffic = NCU_TRAFFIC_BYTES.get((args.workload, work.projections[dom].name.split("/")[-1], args.activations)) if tp == 1 else None
        if t_tensor > t_hbm:
            achieved = dom_work["flops"] / (main_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                    "peak_kind": ("nominal dense NVFP4" if mode else f"{peak_kind} dense BF16 GEMM, kernel timed alone"),
                    "algorithmic_flops": dom_work["flops"], "hbm_gbs": dom_work["main_kernel"] / (main_ms * 1e-3) / 1e9}
        else:
            achieved = dom_work["main_kernel"] / (main_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                    "peak_kind": f"{peak_kind} HBM copy", "tflops": dom_work["flops"] / (main_ms * 1e-3) / 1e12}
        roof.update({"traffic": traffic, "kernel": f"{dom_kernel}, projection '{work.projections[dom].name.split('/')[-1]}' (per rank)",
                     "kernel_ms": main_ms, "algorithmic_bytes": dom_work["main_kernel"], "launch_shape": dom_shape})
        t_roof = max(work_all["flops"] / (FP4_PEAK_TFLOPS * 1e12), work_all["total"] / (hbm_gbs * 1e9))
        t_roof_bf16 = max(work_all["flops"] / (bf16_sustained * 1e12), work_all["total"] / (hbm_gbs * 1e9))
        per_step_launches = sum((1 if c.seq_slot is not None else 0) + 1 + (1 if mode and i_ not in dw.shares_x_with else 0) for i_, c in enumerate(work.projections)) + (1 if fused else 0) + (0 if by_copy_engines else sum(1 for p_ in push_proj if p_)) + ((1 if by_copy_engines else 2) if mlp_h else 0)
        line = {
            "metric": METRIC, "value": M / (step_ms * 1e-3), "unit": "tokens/s", "n_gpus": tp,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": work.config(args, tp),
            "tflops": work_all["flops"] / (step_ms * 1e-3) / 1e12,
            "roofline": roof,
            "layer_roofline": {"time_us": t_roof * 1e6, "frac": t_roof / (step_ms * 1e-3),
                               "rule": "max(flops / 9 PFLOP/s nominal NVFP4, algorithmic bytes / measured HBM GB/s), single GPU",
                               "algorithmic_bytes": work_all["total"], "flops": work_all["flops"],
                               "exact_activation_ceiling": {"time_us": t_roof_bf16 * 1e6, "frac": t_roof_bf16 / (step_ms * 1e-3),
                                                            "rule": "the same with flops / measured sustained dense BF16 TFLOP/s: what exact BF16 "
                                                                    "activations can reach at most, since they run at the BF16 tensor rate"}},
            "projections": [{"name": c.name.split("/")[-1], "ms": proj_ms[i],
                             "tflops": works_local[i]["flops"] / (proj_ms[i] * 1e-3) / 1e12} for i, c in enumerate(work.projections)],
            "e2e": {"value": M / (e2e_ms * 1e-3) if e2e_ms == e2e_ms else None, "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "serial_ms_per_step": e2e_serial_ms,
                    "note": ("value: copies of neighbouring steps overlap the compute (two buffer sets, three streams); "
                             "serial_ms_per_step: copy in, compute, copy out, one step at a time") if tp == 1 else
                            "per rank: copy this rank's rows of the activations in, all-gather them over NVLink, compute + exchange, "
                            "copy this rank's column shard of every result out; value: the read-back of step i overlaps step i+1 "
                            "(two result buffer sets), serial_ms_per_step: one step at a time; byte counts are per rank"},
            "launch_shape": launch_shape,
            "gpu_launches": args.steps * per_step_launches + n_sub * (per_step_launches - (1 if fused else 0)) + n_sub * (2 if mode else 1),
            "clocks": clocks,
        }
        if collective_note:
            line["collective_note"] = collective_note
        if phase_ms:
            line["step_phases"] = phase_ms
        if have_other:
            line["other_activation_mode"] = {
                "activations": "bf16" if mode else "fp4", "ms_per_step": other_ms, "value": M / (other_ms * 1e-3),
                "unit": "tokens/s", "layer_roofline_frac": t_roof / (other_ms * 1e-3),
                "note": "layer kernels only, no collective; fp4 = activations quantised to NVFP4 before the base product "
                        "(the reference's opt-in W4A4 arm), outside the BF16-activation tolerance by construction"}
        if not args.no_cpu_baseline and tp == 1:
            cstep, rows, cores = cpu_sample(work, args.cpu_rows or default_cpu_rows(work))
            ct = cstep()
            line["cpu_baseline"] = {"value": rows / ct, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"first {rows} of {M} tokens x all outputs of all {n_proj} projections, one pass ({ct:.1f} s)"}
        print(json.dumps(line), flush=True)
    if tp > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
