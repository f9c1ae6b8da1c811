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
    args.lut = args.lut or "MBM_7"
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
TRAIN_WORKLOADS = {
    # name: (metric, unit, per-GPU batch, LUT, description)
    "resnet50": ("resnet50_am_train_throughput", "img/s", 32, "MBM_7",
                 "ResNet-50 v1 bottleneck, every Conv2D -> AMConv2D and the FC -> denseam, 224x224x3 NHWC ~N(0,1), "
                 "uniform labels 0..999, He-normal init, SGD train step"),
    "transformer": ("transformer_am_train_throughput", "tokens/s", 64, "MIT_7",
                    "Transformer encoder-decoder 6+6 layers, d_model 512, 8 heads, FFN 2048, seq 128, vocab 8000, "
                    "AMMHA + MatMulAM + denseam, teacher-forced SGD train step"),
    "lenet5": ("lenet5_am_train_throughput", "img/s", 128, "MIT_7", "LeNet-5 AMConv2D + denseam, 28x28x1, SGD train step"),
    "lenet300100": ("lenet300100_am_train_throughput", "img/s", 256, "MBM_7", "LeNet-300-100 denseam, 784 inputs, SGD train step"),
}


class OpTimer:
    """Wraps the op functions so every call is bracketed by CUDA events on the
    current stream and attributed its product count."""

    def __init__(self, ops_mod, torch):
        self.ops, self.torch = ops_mod, torch
        self.records = []  # (kernel, macs, e0, e1)
        self.enabled = False
        self.launches = 0
        self._orig = {}

    def _wrap(self, name, kernel, macs_fn, launches_fn=lambda *a, **k: 1):
        orig = getattr(self.ops, name)
        self._orig[name] = orig

        def f(*a, **k):
            if not self.enabled:
                return orig(*a, **k)
            e0 = self.torch.cuda.Event(enable_timing=True)
            e1 = self.torch.cuda.Event(enable_timing=True)
            e0.record()
            out = orig(*a, **k)
            e1.record()
            self.records.append((kernel, macs_fn(out, *a, **k), e0, e1))
            self.launches += launches_fn(out, *a, **k)
            return out
        setattr(self.ops, name, f)

    def install(self):
        def conv_macs(out, x, w, **k):
            return out.numel() * w.shape[0] * w.shape[1] * w.shape[2]

        def igrad_macs(out, sizes, w, dy, **k):
            return dy.numel() * w.shape[0] * w.shape[1] * w.shape[2]

        def fgrad_macs(out, sizes, x, dy, **k):
            return dy.numel() * sizes[0] * sizes[1] * sizes[2]

        self._wrap("convam", "gather_gemm", conv_macs)
        self._wrap("convam_input_grad", "gather_gemm", igrad_macs)
        self._wrap("convam_filter_grad", "fgrad_gemm", fgrad_macs, lambda *a, **k: 2)
        self._wrap("denseam", "gather_gemm", lambda out, x, w, *a, **k: out.numel() * x.shape[1])
        self._wrap("denseam_grad", "dense_grad(gather+fgrad)", lambda out, g, x, w, *a, **k: 2 * x.numel() * w.shape[1],
                   lambda *a, **k: 3)
        self._wrap("matmulam", "gather_gemm", lambda out, a, b, **k: out.numel() * a.shape[-1 if not k.get("transpose_a") else -2])

    def summary(self, steps):
        agg = {}
        for kernel, macs, e0, e1 in self.records:
            a = agg.setdefault(kernel, [0, 0.0, 0])
            a[0] += macs
            a[1] += e0.elapsed_time(e1)
            a[2] += 1
        return {k: {"macs_per_step": v[0] // steps, "ms_per_step": v[1] / steps, "calls_per_step": v[2] // steps} for k, v in agg.items()}


def build_train_workload(name, lut, dev, rank, torch, deterministic):
    from approxtrain_b200 import nets
    metric, unit, batch, _, _ = TRAIN_WORKLOADS[name]
    torch.manual_seed(0)  # identical weights on every rank
    g = torch.Generator().manual_seed(1000 + rank)  # different data shard per rank
    if name == "resnet50":
        model = nets.ResNet50AM(lut, deterministic=deterministic).to(dev)
        hx = torch.randn(batch, 224, 224, 3, generator=g).pin_memory()
        hy = torch.randint(0, 1000, (batch,), generator=g).pin_memory()
        units = batch

        def loss_fn(x, y):
            return torch.nn.functional.cross_entropy(model(x), y)
    elif name == "transformer":
        model = nets.TransformerAM(lut, deterministic=deterministic).to(dev)
        hx = torch.randint(1, 8000, (batch, 128), generator=g).pin_memory()
        hy = torch.randint(1, 8000, (batch, 129), generator=g).pin_memory()
        units = batch * 128

        def loss_fn(x, y):
            logits = model(x, y[:, :-1])
            return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), y[:, 1:].reshape(-1))
    elif name == "lenet5":
        model = nets.LeNet5(lut, deterministic=deterministic).to(dev)
        hx = torch.rand(batch, 28, 28, 1, generator=g).pin_memory()
        hy = torch.randint(0, 10, (batch,), generator=g).pin_memory()
        units = batch

        def loss_fn(x, y):
            return torch.nn.functional.cross_entropy(model(x), y)
    else:
        model = nets.LeNet300100(lut, deterministic=deterministic).to(dev)
        hx = torch.rand(batch, 28, 28, 1, generator=g).pin_memory()
        hy = torch.randint(0, 10, (batch,), generator=g).pin_memory()
        units = batch

        def loss_fn(x, y):
            return torch.nn.functional.cross_entropy(model(x), y)
    return model, hx, hy, units, loss_fn


def run_train_gpu(args, rank, world):
    import torch
    import torch.distributed as dist
    from approxtrain_b200 import ops
    from approxtrain_b200.dp import DataParallelSGD

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    metric, unit, batch, default_lut, desc = TRAIN_WORKLOADS[args.workload]
    lut_name = args.lut or default_lut
    lut = os.path.join(LUT_DIR, lut_name + ".bin")
    peaks = measured_peaks()
    timer = OpTimer(ops, torch)
    timer.install()
    model, hx, hy, units, loss_fn = build_train_workload(args.workload, lut, dev, rank, torch, args.deterministic)
    trainer = DataParallelSGD(model, lr=1e-3)
    dx, dy = hx.to(dev), hy.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        trainer.step(lambda: loss_fn(dx, dy))
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    timer.enabled = True
    barrier()
    t0.record()
    for _ in range(args.steps):
        loss = trainer.step(lambda: loss_fn(dx, dy))
    t1.record()
    barrier()
    timer.enabled = False
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t0.elapsed_time(t1)
    if world > 1:
        tt = torch.tensor([total_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms = float(tt.item())
    value = world * units * args.steps / (total_ms * 1e-3)

    # ---- end to end: this step's batch starts in pinned host memory, the loss comes back to the host
    e2e_steps = max(1, min(args.steps, 5))
    barrier()
    w0 = time.perf_counter()
    for _ in range(e2e_steps):
        x = hx.to(dev, non_blocking=True)
        y = hy.to(dev, non_blocking=True)
        host_loss = float(trainer.step(lambda: loss_fn(x, y)).item())
    barrier()
    e2e_s = time.perf_counter() - w0
    if world > 1:
        tt = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
    if rank != 0:
        return None
    issue_peak = LANES_PER_CLK_PER_SM * N_SM * peaks["sm_max_mhz"] * 1e6 / 1e12
    summ = timer.summary(args.steps)
    am_ms = sum(v["ms_per_step"] for v in summ.values())
    am_macs = sum(v["macs_per_step"] for v in summ.values())
    dom = max(summ, key=lambda k: summ[k]["ms_per_step"]) if summ else None
    roofline = None
    if dom:
        ach = summ[dom]["macs_per_step"] / (summ[dom]["ms_per_step"] * 1e-3) / 1e12
        roofline = {"kernel": dom, "bound": "lut-issue", "achieved": round(ach, 4), "peak": round(issue_peak, 4),
                    "unit": "TMAC/s", "frac": round(ach / issue_peak, 4),
                    "peak_def": f"32 lookups/clk/SM x {N_SM} SM x sm_max_mhz {peaks['sm_max_mhz']:.0f} ({peaks['source']})",
                    "launches_per_step": summ[dom]["calls_per_step"], "traffic": None,
                    "note": "aggregate over all launches of this kernel in a step (many layer shapes); per-shape figures: --workload conv3"}
    return {
        "metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(total_ms / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {desc}", "per_gpu_batch": batch, "global_batch": batch * world,
                   "lut": lut_name, "mode": "deterministic" if args.deterministic else "fast",
                   "parallelism": f"dp{world}: batch sharded, NCCL all-reduce of {trainer.gradient_bytes() / 1e6:.1f} MB of gradients per step",
                   "l2": "inputs larger than L2: a step streams activations and gradients far beyond 126 MB" if args.workload in ("resnet50", "transformer") else "working set smaller than L2 (launch-bound network)"},
        "clocks": clocks,
        "e2e": {"value": round(world * units * e2e_steps / e2e_s, 2), "unit": unit,
                "h2d_bytes_per_step": hx.numel() * hx.element_size() + hy.numel() * hy.element_size(),
                "d2h_bytes_per_step": 4, "steps": e2e_steps, "loss": host_loss},
        "gpu_launches": timer.launches,
        "roofline": roofline,
        "am_ops": {"ms_per_step": round(am_ms, 3), "gmac_per_step": round(am_macs / 1e9, 2),
                   "share_of_step": round(am_ms / (total_ms / args.steps), 3), "by_kernel": {k: {kk: (round(vv, 3) if isinstance(vv, float) else vv) for kk, vv in v.items()} for k, v in summ.items()}},
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
    ap.add_argument("--workload", default="conv3", choices=["conv3"] + list(TRAIN_WORKLOADS))
    ap.add_argument("--lut", default=None)
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
        line = run_conv3_gpu(args, rank, world) if args.workload == "conv3" else run_train_gpu(args, rank, world)
        if rank == 0:
            if args.workload != "conv3":
                line["cpu_baseline"] = None
            elif world == 1 and not args.no_cpu_baseline:
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
