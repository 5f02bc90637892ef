#!/usr/bin/env python
"""Benchmark of the fused NVFP4 + multi-LoRA linear layer.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload config1] [--impl reference]

One step = one pass of the layer over one synthetic batch.  The default workload is benchmark
configuration 1 (NVFP4 base K=5120 N=17408, 256 tokens, 16 adapters of rank 32, 10 % of the tokens
adapter-less).  With N > 1 (launched by torch.distributed.run, one rank per GPU) the same layer is
split column-parallel over the ranks — W, its scales and every B_s by output rows; x and A_s
replicated: strong scaling.  Every rank's kernel stores its output tiles straight into all ranks' gathered
[M, N] buffers over NVLink (peer mappings from torch's symmetric memory), so the exchange overlaps the
compute tile by tile and what remains of the collective is one device-side barrier; `--collective nccl`
(or a box where the peer mapping cannot be made) runs the layer followed by one NCCL all-gather instead.

Rank 0 prints one JSON line.  `value` is device-timed (CUDA events on the launching stream, L2
flushed between steps, inputs resident in HBM); `e2e` runs the same call with host buffers, with the
H2D copy of the step's inputs and the D2H copy of its result inside the timed region.
`--impl reference` times the CPU oracle (a scalar restatement of the reference's arithmetic — the
reference itself is Rust + GB10 CUDA and has no CPU build of this path) on a bounded sample.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the tcgen05 kernel, from the ncu captures
# summarised under profiles/ (per workload; None where no capture exists)
NCU_TRAFFIC_BYTES = {"config1": 72.9e6}
WORKLOADS = {"config0": 0, "config1": 1, "config2": 2, "config3": 3, "config4": 4}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def algorithmic_work(case):
    """Bytes and flops of one pass, each tensor counted once (adapters at their true rank)."""
    M, N, K = case.M, case.N, case.K
    w_bytes = N * K * 2 if case.w_bf16 is not None else N * K * (0.5 + 1.0 / 16.0)
    hit = sorted(set(int(s) for s in case.seq_slot if s >= 0))
    a_bytes = sum(case.adapters[s].rank * K * 2 for s in hit)
    b_bytes = sum(case.adapters[s].rank * N * 2 for s in hit)
    x_bytes, y_bytes, slot_bytes = M * K * 2, M * N * 2, 4 * M
    flops = 2.0 * M * N * K + 2.0 * sum(case.adapters[int(s)].rank * (K + N) for s in case.seq_slot if s >= 0)
    return dict(w=w_bytes, a=a_bytes, b=b_bytes, x=x_bytes, y=y_bytes, slot=slot_bytes,
                total=w_bytes + a_bytes + b_bytes + x_bytes + y_bytes + slot_bytes, flops=flops,
                main_kernel=w_bytes + b_bytes + x_bytes + y_bytes + slot_bytes)


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
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------------
# CPU arm: the oracle on host cores
# --------------------------------------------------------------------------------------------------
def cpu_sample(case, budget_rows=None):
    """Time the reference's launch sequence (base linear, then staged routed LoRA) on a row sample."""
    from oracle import oracle_ctypes as oc
    import copy
    rows = budget_rows or max(1, min(case.M, int(2.5e10 / (case.N * case.K))))  # ~ 5-20 s of host work per pass
    sub = copy.copy(case)
    sub.M, sub.x, sub.seq_slot = rows, case.x[:rows].copy(), case.seq_slot[:rows].copy()
    pool = oc.HostPool(case.K, case.N, case.max_rank, case.max_loras)
    for s, ad in enumerate(case.adapters):
        if ad is not None:
            pool.pack(s, ad.a, ad.b, ad.scale)
    kw = dict(packed=case.packed, scales=case.scales, scale2=case.scale2, w_bf16=case.w_bf16,
              seq_slot=sub.seq_slot, pool=pool)

    def step():
        t0 = time.perf_counter()
        oc.reference_sequence(sub.x, rows, case.N, case.K, **kw)
        return time.perf_counter() - t0
    return step, rows, oc.num_threads()


def run_reference_arm(args, case):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # size the per-step sample so that the whole run stays near two minutes on this host
    probe, probe_rows, _ = cpu_sample(case, budget_rows=min(4, case.M))
    per_row = probe() / probe_rows
    budget_rows = int(120.0 / max(args.steps + min(args.warmup, 1), 1) / max(per_row, 1e-9))
    step, rows, cores = cpu_sample(case, budget_rows=max(1, min(case.M, budget_rows)))
    for _ in range(min(args.warmup, 1)):
        step()
    times = [step() for _ in range(args.steps)]
    t = float(np.mean(times))
    tok_s = rows / t
    sample = f"first {rows} of {case.M} tokens x all {case.N} outputs, every step"
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": t * 1e3 * case.M / rows,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, case, 1),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, case, tp):
    hit = len(set(int(s) for s in case.seq_slot if s >= 0))
    return {"workload": args.workload, "M": case.M, "K": case.K, "N": case.N, "base": "nvfp4" if case.packed is not None else "bf16",
            "adapters": sum(a is not None for a in case.adapters), "adapters_hit": hit, "max_rank": case.max_rank,
            "adapter_less_rows": int((case.seq_slot < 0).sum()), "activation_mode": "A4 (x quantised to NVFP4)" if getattr(args, "activations", "bf16") == "fp4" else "A16 (exact BF16 x)",
            "parallelism": (f"column-parallel tp{tp}, " + getattr(args, "collective_used", "all-gather")) if tp > 1 else "single GPU",
            "l2": "flushed between timed steps"}


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="config1", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="atlas_b200", choices=["atlas_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--collective", default="fused", choices=["fused", "nccl"],
                    help="N > 1: fused = the kernel's epilogue stores into every rank's buffer; nccl = all-gather after it")
    ap.add_argument("--activations", default="bf16", choices=["bf16", "fp4"],
                    help="bf16: the layer as specified (exact activations); fp4: the opt-in W4A4 mode as the timed step")
    args = ap.parse_args()

    from atlas_b200 import synth
    case = synth.baseline_config(WORKLOADS[args.workload])

    if args.impl == "reference":
        run_reference_arm(args, case)
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

    # ---- this rank's column shard, resident in HBM ----
    from atlas_b200 import tp as tpmod
    shard = tpmod.DeviceShard(torch, ab, case, tp, rank)
    M, N, K, n_loc = case.M, case.N, case.K, shard.n_local
    y_loc = torch.empty((M, n_loc), dtype=torch.bfloat16, device=dev)
    y_all = torch.empty((tp, M, n_loc), dtype=torch.bfloat16, device=dev) if tp > 1 else None
    # fused collective: every rank's [M, N] result buffer, mapped into every process
    y_sym, sym_handle, collective_note = None, None, None
    if tp > 1 and args.collective == "fused":
        try:
            import torch.distributed._symmetric_memory as symm_mem
            if hasattr(symm_mem, "enable_symm_mem_for_group"):
                try:
                    symm_mem.enable_symm_mem_for_group(dist.group.WORLD.group_name)
                except Exception:
                    pass
            y_sym = symm_mem.empty((M, N), dtype=torch.bfloat16, device=dev)
            sym_handle = symm_mem.rendezvous(y_sym, dist.group.WORLD)
            peer_ptrs = [int(p) for p in sym_handle.buffer_ptrs]
            assert len(peer_ptrs) == tp and all(peer_ptrs)
        except Exception as e:                     # no peer mapping on this box: the NCCL path still measures the layer
            collective_note = f"peer mapping unavailable ({type(e).__name__}: {e}); NCCL all-gather used"
            y_sym, sym_handle = None, None
        ok = torch.tensor([1 if sym_handle is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            y_sym, sym_handle = None, None
    fused = sym_handle is not None
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # > L2 (126 MB)
    mode = ab.FLAG_ACT_FP4 if args.activations == "fp4" else 0
    place = dict(y_dest=peer_ptrs, y_col_offset=rank * n_loc, out_row_stride=N) if fused else {}
    desc = shard.desc(y_loc, extra_flags=mode, **place)
    desc_main_only = shard.desc(y_loc, extra_flags=mode | ab.FLAG_REUSE_SHRINK, **place)
    # the other activation mode, timed beside the headline as a secondary figure
    other = 0 if mode else ab.FLAG_ACT_FP4
    desc_other = shard.desc(y_loc, extra_flags=other) if case.packed is not None and K % 256 == 0 else None
    stream = torch.cuda.current_stream()

    def step():
        v = ab.nvfp4_lora_linear(desc, stream)
        if fused:
            sym_handle.barrier(channel=0)          # every rank's tiles have landed in every buffer
        elif tp > 1:
            dist.all_gather_into_tensor(y_all.view(tp * M, n_loc), y_loc)
        return v

    def barrier():
        if tp > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if fused:
        y_sym.view(torch.int16).fill_(0x7FC0)       # NaN pattern: the warm-up must overwrite all of it
    variant = None
    for _ in range(args.warmup):
        flush.fill_(1)
        variant = step()
    barrier()
    launch_shape = ab.last_launch_shape()
    status = ab.device_status()
    if status != 0:
        raise RuntimeError(f"device status word {status:#x} after warm-up")
    if variant != ab.VARIANT_TCGEN05 and case.packed is not None:
        raise RuntimeError("the tcgen05 path did not run for this workload")
    if fused and not bool(torch.isfinite(y_sym.float()).all()):
        raise RuntimeError("the gathered buffer still holds unwritten elements after the warm-up")

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

    # ---- the dominant kernel alone (shrink result reused), for the roofline ----
    ev2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in ev2:
        flush.fill_(1)
        a.record(stream)
        ab.nvfp4_lora_linear(desc_main_only, stream)
        b.record(stream)
    barrier()
    main_ms = float(np.mean([a.elapsed_time(b) for a, b in ev2]))

    # ---- the same step in the other activation mode (no collective), a secondary figure ----
    other_ms = float("nan")
    if desc_other is not None:
        for _ in range(3):
            ab.nvfp4_lora_linear(desc_other, stream)
        ev3 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(min(args.steps, 100))]
        for a, b in ev3:
            flush.fill_(1)
            a.record(stream)
            ab.nvfp4_lora_linear(desc_other, stream)
            b.record(stream)
        barrier()
        other_ms = float(np.mean([a.elapsed_time(b) for a, b in ev3]))

    # ---- end to end through the C ABI with host buffers ----
    x_host = torch.from_numpy(case.x.view(np.int16).copy()).pin_memory()
    slot_host = torch.from_numpy(case.seq_slot.copy()).pin_memory()
    y_host = torch.empty((tp, M, n_loc) if tp > 1 else (M, n_loc), dtype=torch.int16).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        shard.x.view(torch.int16).copy_(x_host, non_blocking=True)
        shard.seq_slot.copy_(slot_host, non_blocking=True)
        step()
        if rank == 0:
            y_host.view(-1).copy_((y_sym if fused else (y_all if tp > 1 else y_loc)).view(torch.int16).view(-1), non_blocking=True)
        barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    e2e_serial_ms = e2e_ms

    # The same, as a serving loop would run it on one GPU: two sets of device buffers, the copy of step i+1's
    # inputs and of step i-1's result on their own streams while step i computes.  Every step still carries its
    # own H2D and D2H copy inside the timed region; what changes is that the three overlap.
    if tp == 1:
        n_buf = 2
        e2e_steps = max(8, min(args.steps, 40))
        xs = [torch.empty_like(shard.x) for _ in range(n_buf)]
        slots = [torch.empty_like(shard.seq_slot) for _ in range(n_buf)]
        ys = [torch.empty((M, n_loc), dtype=torch.bfloat16, device=dev) for _ in range(n_buf)]
        y_hosts = [torch.empty((M, n_loc), dtype=torch.int16).pin_memory() for _ in range(n_buf)]
        descs = []
        for b in range(n_buf):
            db = shard.desc(ys[b], extra_flags=mode)
            db.x, db.seq_slot = xs[b].data_ptr(), slots[b].data_ptr()
            descs.append(db)
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(n_buf)]
        ev_done = [torch.cuda.Event() for _ in range(n_buf)]
        ev_out = [torch.cuda.Event() for _ in range(n_buf)]
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            b = i % n_buf
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_done[b])            # the step that last read these input buffers has finished
                xs[b].view(torch.int16).copy_(x_host, non_blocking=True)
                slots[b].copy_(slot_host, non_blocking=True)
                ev_in[b].record(s_in)
            stream.wait_event(ev_in[b])
            stream.wait_event(ev_out[b])               # the copy that last read this output buffer has finished
            ab.nvfp4_lora_linear(descs[b], stream)
            ev_done[b].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                y_hosts[b].copy_(ys[b].view(torch.int16), non_blocking=True)
                ev_out[b].record(s_out)
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        if not np.array_equal(y_hosts[0].numpy(), y_hosts[1].numpy()):
            raise RuntimeError("the two buffer sets of the end-to-end loop disagree")
    clocks = sampler.stop()

    t = torch.tensor([step_ms, main_ms, e2e_ms, other_ms], dtype=torch.float64, device=dev)
    if tp > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms, main_ms, e2e_ms, other_ms = [float(v) for v in t.tolist()]

    args.collective_used = "tiles stored into every rank's buffer by the kernel + device barrier" if fused else "NCCL all-gather"
    if rank == 0:
        hbm_gbs, peak_kind = peaks()
        work = algorithmic_work(case)
        shard_work = algorithmic_work(shard.local_case)
        achieved = shard_work["main_kernel"] / (main_ms * 1e-3) / 1e9
        t_roof = max(work["flops"] / (FP4_PEAK_TFLOPS * 1e12), work["total"] / (hbm_gbs * 1e9))
        line = {
            "metric": METRIC, "value": M / (step_ms * 1e-3), "unit": "tokens/s", "n_gpus": tp,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args, case, tp),
            "tflops": work["flops"] / (step_ms * 1e-3) / 1e12,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload) if tp == 1 else None, "peak_kind": peak_kind,
                         "kernel": "nvfp4_lora_linear_tc_kernel (per rank)", "kernel_ms": main_ms,
                         "algorithmic_bytes": shard_work["main_kernel"]},
            "layer_roofline": {"time_us": t_roof * 1e6, "frac": t_roof / (step_ms * 1e-3),
                               "rule": "max(flops / 9 PFLOP/s nominal NVFP4, algorithmic bytes / measured HBM GB/s), single GPU",
                               "algorithmic_bytes": work["total"], "flops": work["flops"]},
            "e2e": {"value": M / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(x_host.numel() * 2 + slot_host.numel() * 4),
                    "d2h_bytes_per_step": int(y_host.numel() * 2), "ms_per_step": e2e_ms,
                    "serial_ms_per_step": e2e_serial_ms,
                    "note": "value: copies of neighbouring steps overlap the compute (two buffer sets, three streams); "
                            "serial_ms_per_step: copy in, compute, copy out, one step at a time" if tp == 1 else
                            "copy in, compute + collective, copy out, one step at a time"},
            "launch_shape": launch_shape,
            "gpu_launches": args.steps * (3 if mode else 2) + args.steps * (2 if mode else 1),
            "clocks": clocks,
        }
        if collective_note:
            line["collective_note"] = collective_note
        if desc_other is not None:
            line["other_activation_mode"] = {
                "activations": "bf16" if mode else "fp4", "ms_per_step": other_ms, "value": M / (other_ms * 1e-3),
                "unit": "tokens/s", "layer_roofline_frac": t_roof / (other_ms * 1e-3),
                "note": "layer kernels only, no collective; fp4 = activations quantised to NVFP4 before the base product "
                        "(the reference's opt-in W4A4 arm), outside the BF16-activation tolerance by construction"}
        if not args.no_cpu_baseline and tp == 1:
            cstep, rows, cores = cpu_sample(case)
            ct = cstep()
            line["cpu_baseline"] = {"value": rows / ct, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"first {rows} of {M} tokens x all {N} outputs, one pass ({ct:.1f} s)"}
        print(json.dumps(line), flush=True)
    if tp > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
