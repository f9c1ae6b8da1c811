#!/usr/bin/env python
"""Benchmark of the AM-Simulator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload conv3|...]
    python bench.py --impl reference ...       # the reference's CPU op path

Prints ONE JSON line (rank 0).  For N > 1 it is launched by torchrun, one rank
per GPU; every rank processes its own batch shard (weak scaling).

Workload ``conv3`` — the AMConv2D microbenchmark: NHWC FP32 tensors ~N(0,1)
from a seed, 3x3 stride 1 SAME, shapes A (N64 56x56 64->64) and B (N64 14x14
256->256), LUT MBM_7; one step = forward + input gradient + filter gradient of
both shapes = 6 x 7.399 GMAC.  `value` is GMAC/s with all tensors resident in
HBM; `e2e` is the same step through the op interface starting from pinned host
buffers, host<->device copies inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LUT_DIR = os.path.join(ROOT, "tests", "golden", "lut")
N_SM = 148
LANES_PER_CLK_PER_SM = 32  # one warp-wide shared-memory table lookup per clock per SM

CONV3_SHAPES = {
    # name: (N, H, W, C, KH, KW, K)
    "A": (64, 56, 56, 64, 3, 3, 64),
    "B": (64, 14, 14, 256, 3, 3, 256),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "sm_max_mhz": float(d["sm_max_mhz"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "sm_max_mhz": 1965.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
def conv3_work():
    """MACs and algorithmic HBM bytes per direction for each shape."""
    out = {}
    for name, (n, h, w, c, kh, kw, k) in CONV3_SHAPES.items():
        macs = n * h * w * k * kh * kw * c
        elems = n * h * w * c + kh * kw * c * k + n * h * w * k
        out[name] = {"macs": macs, "bytes": 4 * elems}
    return out


def run_conv3_gpu(args, rank, world):
    import torch
    import torch.distributed as dist
    from approxtrain_b200 import ops

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    lut = os.path.join(LUT_DIR, args.lut + ".bin")
    peaks = measured_peaks()
    work = conv3_work()

    host, devt = {}, {}
    for name, (n, h, w, c, kh, kw, k) in CONV3_SHAPES.items():
        g = torch.Generator().manual_seed(1000 * rank + ord(name))
        host[name] = {
            "x": torch.randn((n, h, w, c), generator=g).pin_memory(),
            "w": torch.randn((kh, kw, c, k), generator=g).pin_memory(),
            "dy": torch.randn((n, h, w, k), generator=g).pin_memory(),
        }
        devt[name] = {kk: v.to(dev) for kk, v in host[name].items()}
    kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=lut, deterministic=args.deterministic)

    OPS = []  # (label, shape, fn)
    for name in CONV3_SHAPES:
        t = devt[name]
        OPS.append((f"fwd_{name}", name, lambda t=t: ops.convam(t["x"], t["w"], **kw_)))
        OPS.append((f"input_grad_{name}", name, lambda t=t: ops.convam_input_grad(t["x"].shape, t["w"], t["dy"], **kw_)))
        OPS.append((f"filter_grad_{name}", name, lambda t=t: ops.convam_filter_grad(t["w"].shape, t["x"], t["dy"], **kw_)))
    launches_per_step = 0
    from approxtrain_b200 import _lib
    for label, name, _ in OPS:
        launches_per_step += 1
        if label.startswith("filter_grad"):
            n, h, w, c, kh, kw, k = CONV3_SHAPES[name]
            if _lib.lib.amsim_conv2d_bwd_filter_workspace(n, h, w, c, kh, kw, k, h, w, 1 if args.deterministic else 0):
                launches_per_step += 1  # split-K reduction kernel

    def step(record=None):
        for i, (label, name, fn) in enumerate(OPS):
            if record is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                record.append((i, e0, e1))
            else:
                fn()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    rec = []
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        step(rec)
    t1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t0.elapsed_time(t1)
    if world > 1:
        tt = torch.tensor([total_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms = float(tt.item())
    per_op_ms = [0.0] * len(OPS)
    for i, e0, e1 in rec:
        per_op_ms[i] += e0.elapsed_time(e1)
    per_op_ms = [v / args.steps for v in per_op_ms]

    step_macs = sum(work[name]["macs"] for _, name, _ in OPS)
    value = world * step_macs * args.steps / (total_ms * 1e-3) / 1e9  # GMAC/s, all ranks

    # ---- end to end through the op interface from pinned host memory ----------------------
    def e2e_step():
        outs = []
        for name in CONV3_SHAPES:
            hx = host[name]
            x = hx["x"].to(dev, non_blocking=True)
            w = hx["w"].to(dev, non_blocking=True)
            dy = hx["dy"].to(dev, non_blocking=True)
            y = ops.convam(x, w, **kw_)
            dx = ops.convam_input_grad(x.shape, w, dy, **kw_)
            dw = ops.convam_filter_grad(w.shape, x, dy, **kw_)
            outs += [y, dx, dw]
        return [o.to("cpu", non_blocking=True) for o in outs]

    e2e_steps = max(1, min(args.steps, 5))
    e2e_step()
    barrier()
    w0 = time.perf_counter()
    for _ in range(e2e_steps):
        res = e2e_step()
    torch.cuda.synchronize()
    barrier()
    e2e_s = time.perf_counter() - w0
    if world > 1:
        tt = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
    h2d = sum(v.numel() * 4 for name in CONV3_SHAPES for v in host[name].values())
    d2h = sum(r.numel() * 4 for r in res)
    e2e_value = world * step_macs * e2e_steps / e2e_s / 1e9

    if rank != 0:
        return None
    # ---- roofline of the dominant kernel -------------------------------------------------------
    clk_mhz = peaks["sm_max_mhz"]
    issue_peak = LANES_PER_CLK_PER_SM * N_SM * clk_mhz * 1e6 / 1e12  # TMAC/s
    kernels = []
    for (label, name, _), ms in zip(OPS, per_op_ms):
        macs, byts = work[name]["macs"], work[name]["bytes"]
        t_issue = macs / (issue_peak * 1e12)
        t_hbm = byts / (peaks["hbm_gbs"] * 1e9)
        kernels.append({
            "op": label, "ms": round(ms, 4), "gmacs": round(macs / (ms * 1e-3) / 1e9, 1),
            "frac_of_roofline": round(max(t_issue, t_hbm) / (ms * 1e-3), 4),
            "hbm_gbs_algorithmic": round(byts / (ms * 1e-3) / 1e9, 1),
        })
    dom = max(range(len(OPS)), key=lambda i: per_op_ms[i])
    dlabel, dname, _ = OPS[dom]
    achieved = work[dname]["macs"] / (per_op_ms[dom] * 1e-3) / 1e12
    obs_clk = clocks.get("sm_mhz") if clocks else None
    roofline = {
        "kernel": ("fgrad_gemm" if dlabel.startswith("filter_grad") else "gather_gemm") + f" ({dlabel})",
        "bound": "lut-issue",
        "achieved": round(achieved, 4), "peak": round(issue_peak, 4), "unit": "TMAC/s",
        "frac": round(achieved / issue_peak, 4),
        "peak_def": f"32 lookups/clk/SM x {N_SM} SM x sm_max_mhz {clk_mhz:.0f} ({peaks['source']}); "
                    f"the HBM bound ({work[dname]['bytes'] / 1e6:.1f} MB at {peaks['hbm_gbs']:.0f} GB/s of {peaks['source']}) "
                    "is ~50x lower for these shapes",
        "frac_at_observed_clock": (round(achieved / (LANES_PER_CLK_PER_SM * N_SM * obs_clk * 1e6 / 1e12), 4) if obs_clk else None),
        "algorithmic_bytes": work[dname]["bytes"],
        "traffic": None,
    }
    return {
        "metric": "am_lut_gemm_throughput", "value": round(value, 1), "unit": "GMAC/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(total_ms / args.steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "conv3: AMConv2D 3x3 s1 SAME, shapes A N64 56x56 64->64 and B N64 14x14 256->256, "
                               "fwd + input-grad + filter-grad, per GPU",
                   "lut": args.lut, "mode": "deterministic" if args.deterministic else "fast",
                   "l2": "inputs larger than L2: one step touches ~260 MB, L2 is 126 MB"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": "GMAC/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": roofline,
        "kernels": kernels,
    }


# ------------------------------------------------------------------------------------------------
def cpu_conv3(sample_batch: int, repeats: int = 1):
    """The reference's CPU op path (exact multiply, serial loops: convam.cc:452-491,
    :639-686, :910-954) restated in oracle/amsim_oracle.c, on a batch-reduced
    sample of the conv3 step.  Returns (GMAC/s, seconds, description)."""
    import numpy as np
    from oracle.oracle import Oracle
    o = Oracle.get()
    macs = 0
    secs = 0.0
    for name, (n, h, w, c, kh, kw, k) in CONV3_SHAPES.items():
        nb = sample_batch
        rng = np.random.default_rng(ord(name))
        x = rng.standard_normal((nb, h, w, c)).astype(np.float32)
        wt = rng.standard_normal((kh, kw, c, k)).astype(np.float32)
        dy = rng.standard_normal((nb, h, w, k)).astype(np.float32)
        g = o.geometry(nb, h, w, c, kh, kw, k, 1, 1, "SAME")
        for _ in range(repeats):
            t0 = time.perf_counter()
            o.cpu_conv2d_fwd(g, x, wt)
            o.cpu_conv2d_bwd_input(g, wt, dy)
            o.cpu_conv2d_bwd_filter(g, x, dy)
            secs += time.perf_counter() - t0
            macs += 3 * nb * h * w * k * kh * kw * c
    return macs / secs / 1e9, secs, f"conv3 step at batch {sample_batch} of 64 (both shapes, 3 directions), 1 thread"


def run_reference(args, rank, world):
    """--impl reference: the reference's own CPU implementation of the path.  Its
    TensorFlow op cannot be built here (no TensorFlow), so the serial loop nests
    of its CPU functors are timed as restated in the oracle (kind "port")."""
    if rank != 0:
        return None
    gm = []
    secs = 0.0
    for _ in range(args.warmup and 1):
        cpu_conv3(1)
    for _ in range(max(1, min(args.steps, 3))):
        v, s, desc = cpu_conv3(args.cpu_sample_batch)
        gm.append(v)
        secs += s
    value = statistics.mean(gm)
    return {
        "impl": "reference", "metric": "am_lut_gemm_throughput", "value": round(value, 3), "unit": "GMAC/s",
        "n_gpus": world, "steps": len(gm), "warmup": 1 if args.warmup else 0,
        "ms_per_step": round(1e3 * secs / len(gm), 1), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "conv3: AMConv2D 3x3 s1 SAME, shapes A and B, fwd + input-grad + filter-grad"},
        "cpu_baseline": {"value": round(value, 3), "unit": "GMAC/s", "cores": 1, "host_cores": os.cpu_count(),
                         "kind": "port", "sample": desc},
        "e2e": {"value": round(value, 3), "unit": "GMAC/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="conv3", choices=["conv3"])
    ap.add_argument("--lut", default="MBM_7")
    ap.add_argument("--deterministic", action="store_true")
    ap.add_argument("--cpu-sample-batch", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "ours" and args.warmup < 3:
        args.warmup = 3
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    import torch
    import torch.distributed as dist
    if world > 1:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl")
    try:
        line = run_conv3_gpu(args, rank, world)
        if rank == 0:
            if world == 1 and not args.no_cpu_baseline:
                v, s, desc = cpu_conv3(args.cpu_sample_batch)
                line["cpu_baseline"] = {"value": round(v, 3), "unit": "GMAC/s", "cores": 1, "host_cores": os.cpu_count(),
                                        "kind": "port", "sample": desc, "seconds": round(s, 2)}
            else:
                line["cpu_baseline"] = None
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
