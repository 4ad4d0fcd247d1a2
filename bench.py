#!/usr/bin/env python
"""Benchmark of the varlen QK^T + row-softmax hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One step = one pass of the fused scores+softmax operator over one synthetic
packed batch.  Default workload: the long-tail batch (512 segments, n
log-uniform in [16, 2048], 4 heads, d = 64, bf16), the largest QK^T+softmax
configuration that fits one GPU.  With N > 1 (launched under torchrun, one rank
per GPU) that same fixed batch is split over the ranks by balanced cost (strong
scaling): a rank generates and processes only the segments it owns and there is
no collective on the data path; `--gather` additionally times the optional
gather of the packed result onto every rank.

Prints ONE JSON line on rank 0.  `value` is whole-job TFLOP/s (algorithmic
2*H*d*sum(n^2) flops per step) with inputs resident in HBM; `roofline` rates the
same launches against the measured HBM copy bandwidth (or the measured bf16
tensor throughput where that binds); `e2e` is the same metric through the public
Python operator with pinned host buffers (H2D of q,k and D2H of the
probabilities inside the timed region); `cpu_baseline` times the CPU oracle (the
per-segment torch loop) on the host cores; `configs` carries one sub-record per
other configuration (device time and roofline only); `reference_gpu` times the
upstream project's own CUDA kernels on the one batch they are known to run
cleanly on.

`--impl reference` times the CPU per-segment loop alone as the reference arm:
the upstream project has no CPU implementation of its own (its launchers reject
non-CUDA tensors), so the arm is the oracle port of its per-segment check loop.
That arm never imports the product package.
"""
from __future__ import annotations

import argparse
import glob
import importlib.util
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DEFAULT_WORKLOAD = "long_tail"
SUB_WORKLOADS = ("molecular", "general_gemm", "full_forward", "large_k", "long_tail_attention",
                 "full_forward_attention", "long_tail_softmax")
MIN_TIMED_MS = 200.0          # every device-timed region lasts at least this long, whatever --steps says
CPU_SAMPLE_FLOPS = 2e10       # algorithmic flops of the segment sample one CPU pass works through


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--segments", type=int, default=0,
                    help="segments of the batch (default: the workload's own count); a smaller batch for profiler captures")
    ap.add_argument("--nbuf", type=int, default=3, help="input/output buffer sets rotated between steps")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the sub-records of the other configurations")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the upstream project's own kernels")
    ap.add_argument("--min-ms", type=float, default=MIN_TIMED_MS)
    ap.add_argument("--gather", action="store_true", help="also time the optional gather of the output onto every rank")
    return ap.parse_args()


# --------------------------------------------------------------------------
def load_synth():
    """The workload generators, loaded by path: importing the package would load the product library, which the
    reference arm must not do."""
    spec = importlib.util.spec_from_file_location("_blk_synth", os.path.join(ROOT, "blockedattention_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["_blk_synth"] = mod
    spec.loader.exec_module(mod)
    return mod


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p.get("bf16_tflops", 1590.0)),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", 1400.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_traffic():
    """DRAM bytes per launch read from ncu captures, recorded beside the profile summaries."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


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
        self.smi = None      # fallback when the NVML binding is not importable: nvidia-smi in a loop

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
            return
        import shutil
        import subprocess
        if shutil.which("nvidia-smi"):
            q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
            try:
                self.smi = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                             "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                            stderr=subprocess.DEVNULL, text=True)
            except Exception:
                self.smi = None

    def stop(self):
        if self.thread:
            self.stop_flag.set()
            self.thread.join()

    def _smi_summary(self) -> dict:
        self.smi.terminate()            # our own child, by handle
        try:
            text = self.smi.communicate(timeout=5)[0]
        except Exception:
            text = ""
        rows = [[c.strip() for c in ln.split(",")] for ln in text.splitlines() if ln.count(",") >= 5]
        mhz = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # under load only: the sampler also sees the idle stretches around the timed region
        busy = [m for m in mhz if m >= 0.5 * max(mhz)]
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(rows[0][1]),
                "reasons": [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)],
                "samples": len(mhz), "source": "nvidia-smi -lms 100 over the whole run"}

    def summary(self, t0: float, t1: float) -> dict:
        if not self.ok and self.smi is not None:
            return self._smi_summary()
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
# CPU legs (the oracle is the checker and the reported baseline, never the product)
# --------------------------------------------------------------------------
def cpu_sample(w, seed: int):
    """A seeded sample of w's segments worth about CPU_SAMPLE_FLOPS (all of w if it is smaller)."""
    per_seg = 2.0 * w.H * (w.M * w.N * w.K).astype(np.float64)
    if per_seg.sum() <= CPU_SAMPLE_FLOPS:
        return w, f"all {w.S} segments of {w.name}"
    order = np.random.RandomState(seed + 12345).permutation(w.S)
    take = int(np.searchsorted(np.cumsum(per_seg[order]), CPU_SAMPLE_FLOPS) + 1)
    idx = np.sort(order[:take])
    frac = per_seg[idx].sum() / per_seg.sum()
    return w.take(idx), (f"seeded sample of {len(idx)} of {w.S} segments of {w.name} carrying {100 * frac:.1f} % of its "
                         "multiply-adds; throughput is flops of the sample / time of the sample")


def cpu_reference_pass(ws, inputs, threads: int):
    """One pass of the CPU oracle over workload ws; returns (seconds, algorithmic flops)."""
    import torch
    if os.path.join(ROOT, "oracle") not in sys.path:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import blk_oracle as O
    torch.set_num_threads(threads)
    q, k = inputs
    t0 = time.perf_counter()
    if ws.softmax:
        O.block_scores(q, k, ws.M, ws.N, ws.K, scale=ws.scale)
    else:
        O.block_gemm(q, k, ws.M, ws.N, ws.K, scale=ws.scale)
    dt = time.perf_counter() - t0
    return dt, 2.0 * ws.H * float((ws.M * ws.N * ws.K).sum())


def base_line(args, w, unit="TFLOP/s"):
    return {
        "metric": "varlen QK^T+softmax throughput (algorithmic 2*H*d*sum(n^2) flop per step)",
        "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": str(w.dtype).split(".")[-1],
        "data": "synthetic",
        "config": {"workload": w.name, "note": w.note, "segments": int(w.S), "heads": w.H,
                   "d": int(w.K[0]) if w.S else 0, "seed": args.seed,
                   "l2": f"inputs+outputs of one step exceed L2 and {args.nbuf} buffer sets rotate between steps"},
    }


def run_reference(args):
    """Reference arm: the CPU per-segment loop on the host cores (rank 0 only, product library never loaded)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    synth = load_synth()
    w = synth.workload(args.workload, seed=args.seed, segments=args.segments or None)
    threads = os.cpu_count() or 1
    ws, what = cpu_sample(w, args.seed)
    q, k = ws.make_inputs("cpu", seed=args.seed)[:2]
    inputs = (q.float(), k.float())
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_pass(ws, inputs, threads)
    t = fl = 0.0
    for _ in range(args.steps):
        dt, f = cpu_reference_pass(ws, inputs, threads)
        t += dt
        fl += f
    val = fl / t / 1e12
    line = base_line(args, w)
    with open("/proc/self/maps") as f:
        product_loaded = "libblkattn" in f.read()
    line.update({
        "impl": "reference", "value": val, "ms_per_step": t / args.steps * 1e3,
        "product_library_loaded": product_loaded,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": what + "; fp32 torch per-segment loop (matmul + softmax); upstream has no CPU "
                                          "implementation"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------
# device timing
# --------------------------------------------------------------------------
class Runner:
    """Plans, rotating buffer sets and the step function of one workload on one device."""

    def __init__(self, w, dev, nbuf: int, seed: int):
        import torch
        from blockedattention_b200.plan import AttentionPlan, GemmPlan
        self.w, self.dev = w, dev
        self.fused_attn = bool(w.extra.get("fused_attention"))
        self.softmax_only = bool(w.extra.get("softmax_only"))
        t0 = time.perf_counter()
        if self.softmax_only:
            from blockedattention_b200.plan import SoftmaxPlan
            self.plan = SoftmaxPlan(w.M, w.N, w.H, w.dtype, device=dev)
            self.plan_pv = None
            g = torch.Generator(device=dev)
            g.manual_seed(seed)
            self.sets = []
            for i in range(max(1, nbuf)):
                src = (torch.randn((w.H, self.plan.D), generator=g, device=dev, dtype=torch.float32) * w.std).to(w.dtype)
                self.sets.append(((src,), torch.empty_like(src), None))
            self.plan_ms_first = (time.perf_counter() - t0) * 1e3
            self.launches_per_step = self.plan.summary["launches"] or 1
            return
        if self.fused_attn:
            self.plan = AttentionPlan(w.M, w.N, w.H, w.dtype, device=dev, d=int(w.K[0]) if w.S else 64)
        else:
            self.plan = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, w.out_dtype, False, False, w.softmax, device=dev)
        self.plan_ms_first = (time.perf_counter() - t0) * 1e3
        self.plan_pv = None
        if w.d_v and not self.fused_attn:
            dv = np.full_like(w.N, w.d_v)
            self.plan_pv = GemmPlan(w.M, dv, w.N, w.H, w.out_dtype, w.out_dtype, False, True, False, device=dev)
        self.sets = []
        for i in range(max(1, nbuf)):
            ins = w.make_inputs(dev, seed=seed + i)
            out = None if self.fused_attn else torch.empty((w.H, self.plan.Dout), dtype=w.out_dtype, device=dev)
            o2 = torch.empty((w.H, int(w.M.sum()) * w.d_v), dtype=w.out_dtype, device=dev) if w.d_v else None
            self.sets.append((ins, out, o2))
        self.launches_per_step = self.plan.summary["launches"] + (self.plan_pv.summary["launches"] if self.plan_pv else 0)

    def step(self, i):
        w = self.w
        ins, out, o2 = self.sets[i % len(self.sets)]
        if self.softmax_only:
            self.plan.run(ins[0], out=out, scale=w.scale)
            return
        if self.fused_attn:
            self.plan.run(ins[0], ins[1], ins[2], out=o2, scale=w.scale)
            return
        self.plan.run(ins[0], ins[1], out=out, scale=w.scale)
        if self.plan_pv is not None:
            self.plan_pv.run(out, ins[2], out=o2)

    def kernel_name(self):
        s = self.plan.summary
        if self.softmax_only:
            return "blk_softmax_pipe_kernel"
        if self.fused_attn:
            return "blk_attn_umma_kernel" if s["umma_items"] else "blk_scores_pipe_kernel"
        small = "blk_scores_pipe_kernel" if s["packs"] else "blk_scores_small_kernel"
        return max(((small, s["small_items"]), ("blk_gemm_tile_kernel", s["tile_items"]),
                    ("blk_gemm_umma_kernel", s["umma_items"]), ("blk_gemm_simt_kernel", s["simt_items"])),
                   key=lambda kv: kv[1])[0]

    def check(self):
        self.plan.check()
        if self.plan_pv is not None:
            self.plan_pv.check()


def cold_plan_ms(w, run, dev, reps: int = 5):
    """Median wall time of creating the plan(s) of one step from the lists: host schedule, one pooled allocation and
    one upload each, synchronised on both sides."""
    import torch
    from blockedattention_b200.plan import AttentionPlan, GemmPlan
    if run.softmax_only:
        return None
    ts = []
    for _ in range(reps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if run.fused_attn:
            p = AttentionPlan(w.M, w.N, w.H, w.dtype, device=dev, d=int(w.K[0]) if w.S else 64)
        else:
            p = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, w.out_dtype, False, False, w.softmax, device=dev)
        q = None
        if run.plan_pv is not None:
            q = GemmPlan(w.M, np.full_like(w.N, w.d_v), w.N, w.H, w.out_dtype, w.out_dtype, False, True, False, device=dev)
        torch.cuda.synchronize()
        ts.append((time.perf_counter() - t0) * 1e3)
        del p, q
    return float(np.median(ts))


def timed_region(fn, steps: int, warmup: int, min_ms: float, barrier, allmax):
    """W warm-up steps, then `repeats` x `steps` steps between two events; returns (ms per step on this rank,
    repeats).  `repeats` is the same on every rank and makes the region last at least min_ms."""
    import torch
    for i in range(max(warmup, 3)):
        fn(i)
    barrier()
    # estimate a step from three more
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(3):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    est = allmax(max(e0.elapsed_time(e1) / 3.0, 1e-3))
    repeats = max(1, int(math.ceil(min_ms / (est * steps))))
    barrier()
    e0.record()
    for i in range(steps * repeats):
        fn(i)
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / (steps * repeats), repeats


def roofline_of(w, ms_per_step: float, peaks, kernel: str, launches: int, traffic_table, world: int):
    t_hbm = w.bytes() / (peaks["hbm_gbs"] * 1e9)
    t_tc = w.flops() / (peaks["bf16_tflops"] * 1e12)
    if t_tc > t_hbm:
        ach = w.flops() / (ms_per_step * 1e-3) / 1e12
        r = {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
             "frac": ach / peaks["bf16_tflops"], "algorithmic_flops_per_step": w.flops()}
    else:
        ach = w.bytes() / (ms_per_step * 1e-3) / 1e9
        r = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
             "algorithmic_bytes_per_step": w.bytes()}
    r.update({"traffic": None, "peak_source": peaks["source"], "kernel": kernel, "launches_per_step": launches})
    t = traffic_table.get(w.name)
    if t and world == 1 and int(t.get("segments", w.S)) == w.S:
        r["traffic"] = float(t["dram_bytes_per_step"])
        r["traffic_source"] = t.get("source")
    return r


def reference_gpu_leg(dev):
    """The upstream project's own kernels (compiled unmodified into oracle/_ref by oracle/build_ref.py), GEMM launch
    then softmax launch with their host tiling and synchronisations, on the one batch they are known to run without
    faulting: the molecular batch with every n rounded to a multiple of 8 (all offsets 16-byte aligned), 8 heads,
    fp16, buffers padded by a tile.  Timed beside the fused kernel of this library on the same batch."""
    import torch
    so = glob.glob(os.path.join(ROOT, "oracle", "_ref", "blk_ref_ext*.so"))
    if not so:
        return {"unavailable": "oracle/_ref is not built on this machine"}
    sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
    import blk_ref_ext as ref
    from blockedattention_b200 import blockAttnScores
    from blockedattention_b200.synth import workload
    w = workload("molecular", seed=0)
    n = np.maximum(8, (np.round(w.M / 8) * 8).astype(np.int64))
    K = np.full_like(n, 64)
    H = 8
    g = torch.Generator().manual_seed(0)
    A = (torch.randn((H, int((n * K).sum())), generator=g) * 0.125).half()
    B = torch.randn((H, int((n * K).sum())), generator=g).half()

    def padded(t):
        buf = torch.zeros(t.numel() + (1 << 19), dtype=t.dtype, device=dev)
        buf[:t.numel()] = t.reshape(-1).to(dev)
        return buf[:t.numel()].view(t.shape)

    a1 = np.concatenate([[0], np.cumsum(n * K)])
    ao = np.concatenate([[0], np.cumsum(n * n)])
    tn, tk, t1, to = (torch.as_tensor(x, device=dev) for x in (n, K, a1, ao))
    Ad, Bd = padded(A), padded(B)

    def ref_step():
        s = ref.gemm_launch(Ad, Bd, t1, t1, to, tn, tn, tk, False, False)
        return ref.softmax_launch(s, to, tn, tn)

    def ours_step():
        return blockAttnScores(Ad, Bd, n, n, K, scale=1.0)

    def timeit(f, it):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(it):
            f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / it

    p_ref, p_our = ref_step(), ours_step()
    torch.cuda.synchronize()
    diff = float((p_ref.float() - p_our.float()).abs().max())
    t_ref, t_our = timeit(ref_step, 30), timeit(ours_step, 300)
    fl = 2.0 * H * 64 * float((n.astype(np.float64) ** 2).sum())
    return {"ms": t_ref, "value": fl / t_ref / 1e9, "unit": "TFLOP/s",
            "ours_ms": t_our, "ours_value": fl / t_our / 1e9, "max_abs_diff": diff,
            "batch": "molecular (seed 0) with every n rounded to a multiple of 8, 8 heads, d=64, fp16, scale folded "
                     "into q; upstream GEMM launch + softmax launch incl. its host tiling and syncs (oracle/_ref), "
                     "ours = one fused launch on a cached plan"}


# --------------------------------------------------------------------------
def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from blockedattention_b200 import (blockAttention, blockAttnScores, blockAttnScoresHost, blockGEMM,
                                       clear_plan_cache, partition)
    from blockedattention_b200.plan import GemmPlan
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
    traffic = load_traffic()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allmax(x: float) -> float:
        if world == 1:
            return float(x)
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def allsum(x: float) -> float:
        if world == 1:
            return float(x)
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- workload and this rank's shard of the one fixed batch ----------------
    base = workload(args.workload, seed=args.seed, segments=args.segments or None)
    ei = torch.empty((), dtype=base.dtype).element_size()
    eo = torch.empty((), dtype=base.out_dtype).element_size()
    owner, pinfo = partition.shard(base.M, base.N, base.K, base.H, world, ei, eo,
                                   peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9)
    mine = np.nonzero(owner == rank)[0]
    w = base.take(mine) if world > 1 else base

    run = Runner(w, dev, args.nbuf, seed=args.seed + 1000 * rank)
    if run.softmax_only:   # a device-side line only: this workload has no operands to bring from the host
        args.no_e2e = args.no_cpu = True
    sampler = ClockSampler(local)
    sampler.start()
    t_wall0 = time.perf_counter()
    my_ms, repeats = timed_region(run.step, args.steps, args.warmup, args.min_ms, barrier, allmax)
    t_wall1 = time.perf_counter()
    run.check()
    plan_summary = run.plan.summary
    clocks = sampler.summary(t_wall0, t_wall1)
    ms_per_step = allmax(my_ms)
    flops_all, bytes_all = base.flops(), base.bytes()
    value = flops_all / (ms_per_step * 1e-3) / 1e12
    launches_all = int(allsum(run.launches_per_step))
    roofline = roofline_of(w, my_ms, peaks, run.kernel_name(), run.launches_per_step, traffic, world)

    # ---- cost of a new list set: cold plan creation (host schedule + allocation + upload) ------------
    plan_ms = None
    if not run.fused_attn and not run.softmax_only:
        ts = []
        for _ in range(5):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            p = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, w.out_dtype, False, False, w.softmax, device=dev)
            torch.cuda.synchronize()
            ts.append((time.perf_counter() - t0) * 1e3)
            del p
        plan_ms = float(np.median(ts))

    # ---- end to end through the public operator with host buffers ----------
    e2e = None
    h2d_probe = None
    if not args.no_e2e:
        fused_attn = run.fused_attn
        nh = 2
        host = [tuple(t.cpu().pin_memory() for t in run.sets[i % len(run.sets)][0]) for i in range(nh)]
        h_out = None if fused_attn else torch.empty((w.H, run.plan.Dout), dtype=w.out_dtype).pin_memory()
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

        def e2e_cold_step(i):
            clear_plan_cache()       # a new list set every step: schedule, upload and staging are rebuilt
            e2e_step(i)

        e2e_steps = max(3, min(args.steps, 20))
        my_e, _ = timed_region(e2e_step, e2e_steps, 3, 0.0, barrier, allmax)
        e_ms = allmax(my_e)
        my_c, _ = timed_region(e2e_cold_step, 5, 3, 0.0, barrier, allmax)
        c_ms = allmax(my_c)
        h2d = sum(t.numel() * t.element_size() for t in host[0])
        res = h_o2 if w.d_v else h_out
        d2h = res.numel() * res.element_size()
        api = ("blockedattention_b200.blockAttention with explicit copies of pinned host tensors" if fused_attn else
               "blockedattention_b200.blockAttnScoresHost on pinned host tensors (per rank)"
               if w.softmax and not w.d_v else
               "blockedattention_b200.blockGEMM / blockAttnScores with explicit copies of pinned host tensors")
        e2e = {"value": flops_all / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms,
               "steps": e2e_steps, "h2d_bytes_per_step": int(allsum(h2d)), "d2h_bytes_per_step": int(allsum(d2h)),
               "api": api,
               "cold": {"value": flops_all / (c_ms * 1e-3) / 1e12, "ms_per_step": c_ms, "steps": 5,
                        "what": "the plan cache is cleared before every step, so each step also builds the schedule, "
                                "uploads it and sets up the staging buffers, as a batch with new lists would"}}

        # what the box's host<->device path delivers with every rank copying at once and no kernels: the
        # ceiling of the end-to-end number (copies in both directions run on separate engines)
        d_in = [torch.empty_like(t, device=dev) for t in host[0]]
        d_res = torch.empty(res.shape, dtype=res.dtype, device=dev)
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        def probe(i):
            cur = torch.cuda.current_stream(dev)
            s_in.wait_stream(cur)
            s_out.wait_stream(cur)
            with torch.cuda.stream(s_in):
                for d, h in zip(d_in, host[i % nh]):
                    d.copy_(h, non_blocking=True)
            with torch.cuda.stream(s_out):
                res.copy_(d_res, non_blocking=True)
            cur.wait_stream(s_in)
            cur.wait_stream(s_out)

        my_p, _ = timed_region(probe, 5, 3, 0.0, barrier, allmax)
        p_ms = allmax(my_p)
        numa = len(glob.glob("/sys/devices/system/node/node[0-9]*")) or None
        h2d_probe = {"ms_per_step": p_ms, "h2d_gbs_all_ranks": allsum(h2d) / (p_ms * 1e-3) / 1e9,
                     "d2h_gbs_all_ranks": allsum(d2h) / (p_ms * 1e-3) / 1e9, "numa_nodes": numa,
                     "e2e_over_copy_ceiling": e_ms / p_ms,
                     "what": "plain pinned cudaMemcpyAsync of one step's operands (H2D) and result (D2H) on two "
                             "streams, all ranks at once, no kernels"}
        del d_in, d_res, host, h_out, h_o2
    sampler.stop()

    gather = None
    if args.gather and world > 1 and not run.fused_attn and not run.softmax_only and not w.d_v:
        outs = run.sets[0][1]
        full = torch.empty((base.H, base.Dout), dtype=outs.dtype, device=dev)
        partition.gather_output(outs, base.M * base.N, owner, base.H, out=full)   # warm-up (connections)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        partition.gather_output(outs, base.M * base.N, owner, base.H, out=full)
        g1.record()
        barrier()
        g_ms = allmax(g0.elapsed_time(g1))
        gather = {"ms": g_ms, "bytes_result": int(full.numel() * full.element_size()),
                  "gbs_received_per_rank": (full.numel() - outs.numel()) * full.element_size() / (g_ms * 1e-3) / 1e9,
                  "what": "partition.gather_output: grouped NCCL send/recv of every rank's strips into the final "
                          "(H, Dout) buffer on every rank; not part of ms_per_step"}
        del full

    # ---- rank 0 alone: CPU baseline, the other configurations, the upstream kernels ------------
    cpu = None
    configs = None
    ref_gpu = None
    if rank == 0 and world == 1:
        if not args.no_cpu:
            threads = os.cpu_count() or 1
            ws, what = cpu_sample(base, args.seed)
            q, k = ws.make_inputs("cpu", seed=args.seed)[:2]
            inputs = (q.float(), k.float())
            cpu_reference_pass(ws, inputs, threads)  # warm the thread pool
            t = fl = 0.0
            reps = 0
            while t < 10.0 and reps < 20:
                dt, f = cpu_reference_pass(ws, inputs, threads)
                t += dt
                fl += f
                reps += 1
            cpu = {"value": fl / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                   "sample": f"{what}, {reps} passes, fp32 torch per-segment loop (matmul + softmax) = the oracle; "
                             "upstream has no CPU implementation"}
        if not args.no_configs:
            del run
            torch.cuda.empty_cache()
            configs = []
            for name in SUB_WORKLOADS:
                if name == args.workload:
                    continue
                try:
                    wc = workload(name, seed=args.seed)
                    rc = Runner(wc, dev, 2, seed=args.seed + 7)
                    ms_c, rep_c = timed_region(rc.step, max(3, min(args.steps, 20)), 3, args.min_ms, barrier, allmax)
                    rc.check()
                    rec = {"workload": name, "note": wc.note, "ms_per_step": ms_c, "repeats": rep_c,
                           "value": wc.flops() / (ms_c * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "roofline": roofline_of(wc, ms_c, peaks, rc.kernel_name(), rc.launches_per_step, traffic, 1),
                           "launches_per_step": rc.launches_per_step, "plan": rc.plan.summary}
                    try:  # what a new set of lists costs on the host before the first launch
                        rec["plan_ms"] = cold_plan_ms(wc, rc, dev)
                    except Exception as exc:
                        rec["plan_ms_error"] = f"{type(exc).__name__}: {exc}"
                    configs.append(rec)
                    del rc
                except Exception as exc:  # a sub-record must not take the headline down with it
                    configs.append({"workload": name, "error": f"{type(exc).__name__}: {exc}"})
                torch.cuda.empty_cache()
        if not args.no_ref_gpu:
            try:
                ref_gpu = reference_gpu_leg(dev)
            except Exception as exc:
                ref_gpu = {"unavailable": f"{type(exc).__name__}: {exc}"}

    if rank == 0:
        line = base_line(args, base)
        line.update({"value": value, "ms_per_step": ms_per_step, "repeats": repeats, "roofline": roofline,
                     "cpu_baseline": cpu, "e2e": e2e, "h2d_probe": h2d_probe, "plan_ms": plan_ms,
                     "gpu_launches": launches_all * args.steps * repeats, "clocks": clocks,
                     "hbm_gbs_all_gpus": bytes_all / (ms_per_step * 1e-3) / 1e9,
                     "partition": {**{k: v for k, v in pinfo.items() if k != "bounds"},
                                   "what": "one fixed batch; segments split over the ranks by balanced "
                                           "max(flops/peak, bytes/peak), measured peaks", "collective": "none"},
                     "plan": plan_summary, "configs": configs, "reference_gpu": ref_gpu})
        if gather:
            line["gather"] = gather
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
