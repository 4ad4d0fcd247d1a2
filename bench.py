#!/usr/bin/env python
"""Benchmark of the varlen QK^T + row-softmax hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One step = one pass of the fused scores+softmax operator over one synthetic
packed batch (default workload: the molecular-graph batch -- 4096 graphs,
n ~ clip(round(N(25,10)),2,128), 8 heads, d = 64, fp16).  With N > 1 (launched
under torchrun, one rank per GPU) the batch holds N times the segments, split
into N contiguous ranges of balanced cost; a rank generates and processes only
its own range and there is no collective on the data path (weak scaling).

Prints ONE JSON line on rank 0.  `value` is whole-job TFLOP/s (algorithmic
2*H*d*sum(n^2) flops per step) with inputs resident in HBM; `roofline` rates the
same launches against the measured HBM copy bandwidth; `e2e` is the same metric
through the public Python operator with pinned host buffers (H2D of q,k and D2H
of the probabilities inside the timed region); `cpu_baseline` times the CPU
oracle (the per-segment torch loop) on the host cores.

`--impl reference` times that CPU loop alone as the reference arm: the upstream
project has no CPU implementation of its own (its launchers reject non-CUDA
tensors), so the arm is the oracle port of its per-segment check loop.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="molecular")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--segments", type=int, default=0,
                    help="segments per GPU (default: the workload's own count); a smaller batch for profiler captures")
    ap.add_argument("--nbuf", type=int, default=3, help="input/output buffer sets rotated between steps")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--gather", action="store_true", help="also time the optional NCCL all-gather of the output")
    return ap.parse_args()


# --------------------------------------------------------------------------
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p.get("bf16_tflops", 1590.0)),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", 1400.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs."""

    def __init__(self, index: int, period: float = 0.02):
        self.index, self.period = index, period
        self.samples, self.stop_flag, self.thread, self.ok = [], threading.Event(), None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def _one(self):
        nv = self.nv
        mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
        try:
            reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        self.samples.append((time.perf_counter(), mhz, reasons))

    def _loop(self):
        while not self.stop_flag.is_set():
            try:
                self._one()
            except Exception:
                pass
            self.stop_flag.wait(self.period)

    def start(self):
        if self.ok:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self):
        if self.thread:
            self.stop_flag.set()
            self.thread.join()

    def summary(self, t0: float, t1: float) -> dict:
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or [min(self.samples, key=lambda s: abs(s[0] - t1))]
        nv = self.nv
        names = {
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        bits = 0
        for s in inside:
            bits |= s[2]
        return {"sm_mhz": float(np.median([s[1] for s in inside])), "sm_max_mhz": float(self.max_mhz),
                "reasons": [k for k, b in names.items() if bits & b], "samples": len(inside)}


# --------------------------------------------------------------------------
def cpu_reference_pass(w, sample_segments: int, threads: int, seed: int):
    """Times the CPU oracle on the first `sample_segments` segments of workload w."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import blk_oracle as O
    torch.set_num_threads(threads)
    ws = w.slice(0, min(sample_segments, w.S))
    q, k = ws.make_inputs("cpu", seed=seed)[:2]
    q, k = q.float(), k.float()
    t0 = time.perf_counter()
    if ws.softmax:
        O.block_scores(q, k, ws.M, ws.N, ws.K, scale=ws.scale)
    else:
        O.block_gemm(q, k, ws.M, ws.N, ws.K, scale=ws.scale)
    dt = time.perf_counter() - t0
    fl = 2.0 * ws.H * float((ws.M * ws.N * ws.K).sum())
    return dt, fl, ws.S


def base_line(args, w, unit="TFLOP/s"):
    return {
        "metric": "varlen QK^T+softmax throughput (algorithmic 2*H*d*sum(n^2) flop per step)",
        "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": str(w.dtype).split(".")[-1],
        "data": "synthetic",
        "config": {"workload": w.name, "note": w.note, "segments_per_gpu": None, "heads": w.H,
                   "d": int(w.K[0]) if w.S else 0, "seed": args.seed,
                   "l2": f"inputs+outputs of one step exceed L2 and {args.nbuf} buffer sets rotate between steps"},
    }


def run_reference(args):
    """Reference arm: the CPU per-segment loop on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import torch
    from blockedattention_b200.synth import workload
    w = workload(args.workload, seed=args.seed, segments=args.segments or None)
    threads = os.cpu_count() or 1
    # bounded sample per step: at most 1024 segments or ~2e10 flop of the workload
    budget = 2e10
    per_seg = 2.0 * w.H * (w.M * w.N * w.K).astype(np.float64)
    cum = np.cumsum(per_seg)
    sample = int(min(w.S, max(1, np.searchsorted(cum, budget) + 1), 1024))
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_pass(w, sample, threads, args.seed)
    t = fl = 0.0
    for _ in range(args.steps):
        dt, f, _ = cpu_reference_pass(w, sample, threads, args.seed)
        t += dt
        fl += f
    val = fl / t / 1e12
    line = base_line(args, w)
    line.update({
        "impl": "reference", "value": val, "ms_per_step": t / args.steps * 1e3,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"first {sample} of {w.S} segments of {w.name} per step, fp32 torch per-segment "
                                   "loop (matmul + softmax); upstream has no CPU implementation"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    line["config"]["segments_per_gpu"] = sample
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------
def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from blockedattention_b200 import blockAttention, blockAttnScores, blockAttnScoresHost, blockGEMM, partition
    from blockedattention_b200.plan import AttentionPlan, GemmPlan
    from blockedattention_b200.synth import workload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()

    # ---- workload and this rank's shard -----------------------------------
    base = workload(args.workload, seed=args.seed, segments=args.segments or None)
    seg_per_gpu = args.segments or base.S
    wg = workload(args.workload, seed=args.seed, segments=seg_per_gpu * world) if world > 1 else base
    cost = partition.segment_cost(wg.M, wg.N, wg.K, wg.H)
    bounds = partition.partition_contiguous(cost, world)
    w = wg.slice(int(bounds[rank]), int(bounds[rank + 1]))
    imb = partition.imbalance(cost, bounds)

    fused_attn = bool(w.extra.get("fused_attention"))
    if fused_attn:
        plan = AttentionPlan(w.M, w.N, w.H, w.dtype, device=dev, d=int(w.K[0]) if w.S else 64)
    else:
        plan = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, w.out_dtype, False, False, w.softmax, device=dev)
    plan_pv = None
    if w.d_v and not fused_attn:
        dv = np.full_like(w.N, w.d_v)
        plan_pv = GemmPlan(w.M, dv, w.N, w.H, w.out_dtype, w.out_dtype, False, True, False, device=dev)
    nbuf = max(1, args.nbuf)
    sets = []
    for i in range(nbuf):
        ins = w.make_inputs(dev, seed=1000 * rank + i + args.seed)
        out = None if fused_attn else torch.empty((w.H, plan.Dout), dtype=w.out_dtype, device=dev)
        o2 = torch.empty((w.H, int(w.M.sum()) * w.d_v), dtype=w.out_dtype, device=dev) if w.d_v else None
        sets.append((ins, out, o2))
    launches_per_step = plan.summary["launches"] + (plan_pv.summary["launches"] if plan_pv else 0)

    def step(i):
        ins, out, o2 = sets[i % nbuf]
        if fused_attn:
            plan.run(ins[0], ins[1], ins[2], out=o2, scale=w.scale)
            return
        plan.run(ins[0], ins[1], out=out, scale=w.scale)
        if plan_pv is not None:
            plan_pv.run(out, ins[2], out=o2)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    barrier()
    t_wall1 = time.perf_counter()
    ms = ev0.elapsed_time(ev1)
    plan.check()
    clocks = sampler.summary(t_wall0, t_wall1)

    tms = torch.tensor([ms], dtype=torch.float64, device=dev)
    tot = torch.tensor([w.flops(), w.bytes()], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms_max = float(tms.item())
    flops_all, bytes_all = float(tot[0].item()), float(tot[1].item())
    ms_per_step = ms_max / args.steps
    value = flops_all / (ms_per_step * 1e-3) / 1e12

    # roofline of this rank's launches (rank 0 reports its own device)
    my_ms_per_step = ms / args.steps
    achieved = w.bytes() / (my_ms_per_step * 1e-3) / 1e9
    s = plan.summary
    small_kernel = "blk_scores_pipe_kernel" if s["packs"] else "blk_scores_small_kernel"
    kernel = max(((small_kernel, s["small_items"]), ("blk_gemm_tile_kernel", s["tile_items"]),
                  ("blk_gemm_umma_kernel", s["umma_items"]), ("blk_gemm_simt_kernel", s["simt_items"])),
                 key=lambda kv: kv[1])[0]
    if fused_attn and not s["packs"]:
        kernel = "blk_attn_umma_kernel"
    t_hbm = w.bytes() / (peaks["hbm_gbs"] * 1e9)
    t_tc = w.flops() / (peaks["bf16_tflops"] * 1e12)
    if t_tc > t_hbm:
        ach_tf = w.flops() / (my_ms_per_step * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": ach_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": ach_tf / peaks["bf16_tflops"], "traffic": None, "peak_source": peaks["source"],
                    "kernel": kernel, "launches_per_step": launches_per_step,
                    "algorithmic_flops_per_step": w.flops()}
    else:
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                    "kernel": kernel, "launches_per_step": launches_per_step,
                    "algorithmic_bytes_per_step": w.bytes()}

    # DRAM traffic of one step from the committed ncu capture of this workload (profiles/), where there is one
    if args.workload == "molecular" and world == 1 and args.seed == 0:
        roofline["traffic"] = 245.0e6  # dram__bytes_read.sum + dram__bytes_write.sum of the step's one launch
        roofline["traffic_source"] = "profiles/blk_scores_pipe_kernel_molecular.md"

    # ---- end to end through the public operator with host buffers ----------
    e2e = None
    if not args.no_e2e:
        nh = 2
        host = []
        for i in range(nh):
            ins = sets[i % nbuf][0]
            host.append(tuple(t.cpu().pin_memory() for t in ins))
        h_out = None if fused_attn else torch.empty((w.H, plan.Dout), dtype=w.out_dtype).pin_memory()
        h_o2 = torch.empty((w.H, int(w.M.sum()) * w.d_v), dtype=w.out_dtype).pin_memory() if w.d_v else None
        dl = np.full_like(w.N, w.d_v) if w.d_v else None

        def e2e_step(i):
            hin = host[i % nh]
            if w.softmax and not w.d_v:
                # host operands in, host probabilities out: head groups pipelined over three streams
                blockAttnScoresHost(hin[0], hin[1], w.M, w.N, w.K, scale=w.scale, out=h_out, out_dtype=w.out_dtype,
                                    device=dev)
                return
            q = hin[0].to(dev, non_blocking=True)
            k = hin[1].to(dev, non_blocking=True)
            if fused_attn:
                v = hin[2].to(dev, non_blocking=True)
                h_o2.copy_(blockAttention(q, k, v, w.M, w.N, scale=w.scale), non_blocking=True)
                return
            if w.softmax:
                p = blockAttnScores(q, k, w.M, w.N, w.K, scale=w.scale, out_dtype=w.out_dtype)
            else:
                p = blockGEMM(q, k, None, None, None, w.M, w.N, w.K, scale=w.scale, out_dtype=w.out_dtype)
            if w.d_v:
                v = hin[2].to(dev, non_blocking=True)
                o = blockGEMM(p, v, None, None, None, w.M, dl, w.N, False, True)
                h_o2.copy_(o, non_blocking=True)
            else:
                h_out.copy_(p, non_blocking=True)

        e2e_steps = max(3, min(args.steps, 20))
        for i in range(3):
            e2e_step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(e2e_steps):
            e2e_step(i)
        e1.record()
        barrier()
        ems = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ems, op=dist.ReduceOp.MAX)
        e_ms = float(ems.item()) / e2e_steps
        h2d = sum(t.numel() * t.element_size() for t in host[0])
        d2h = (h_o2 if w.d_v else h_out).numel() * (h_o2 if w.d_v else h_out).element_size()
        e2e = {"value": flops_all / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms,
               "steps": e2e_steps, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "api": ("blockedattention_b200.blockAttention with explicit copies of pinned host tensors" if fused_attn else
                       "blockedattention_b200.blockAttnScoresHost on pinned host tensors (per rank)"
                       if w.softmax and not w.d_v else
                       "blockedattention_b200.blockGEMM / blockAttnScores with explicit copies of pinned host tensors")}
    sampler.stop()

    gather = None
    if args.gather and world > 1:
        # optional: every rank ends with the whole packed output (H strips of unequal length per rank)
        outs = sets[0][1]
        sizes = torch.tensor([outs.numel()], device=dev)
        all_sizes = [torch.zeros_like(sizes) for _ in range(world)]
        dist.all_gather(all_sizes, sizes)
        bufs = [torch.empty(int(s.item()), dtype=outs.dtype, device=dev) for s in all_sizes]
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        dist.all_gather(bufs, outs.reshape(-1))
        g1.record()
        barrier()
        gather = {"ms": g0.elapsed_time(g1), "bytes_per_rank": int(outs.numel() * outs.element_size())}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        budget = 2e10
        per_seg = 2.0 * base.H * (base.M * base.N * base.K).astype(np.float64)
        sample = int(min(base.S, max(1, np.searchsorted(np.cumsum(per_seg), budget) + 1)))
        cpu_reference_pass(base, min(sample, 64), threads, args.seed)  # warm the thread pool
        t = fl = 0.0
        reps = 0
        while t < 10.0 and reps < 20:
            dt, f, _ = cpu_reference_pass(base, sample, threads, args.seed)
            t += dt; fl += f; reps += 1
        cpu = {"value": fl / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"first {sample} of {base.S} segments of {base.name}, {reps} passes, fp32 torch "
                         "per-segment loop (matmul + softmax) = the oracle; upstream has no CPU implementation"}

    if rank == 0:
        line = base_line(args, base)
        line.update({"value": value, "ms_per_step": ms_per_step, "roofline": roofline, "cpu_baseline": cpu,
                     "e2e": e2e, "gpu_launches": launches_per_step * args.steps * world, "clocks": clocks,
                     "hbm_gbs_all_gpus": bytes_all / (ms_per_step * 1e-3) / 1e9,
                     "partition": {"kind": "contiguous, balanced max(flops/peak, bytes/peak)",
                                   "imbalance": imb, "collective": "none"},
                     "plan": plan.summary})
        if gather:
            line["gather"] = gather
        line["config"]["segments_per_gpu"] = seg_per_gpu
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
