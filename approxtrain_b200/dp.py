"""Batch-sharded data-parallel training: one process per GPU, gradients
all-reduced over NCCL (NVLink / NVSwitch) in buckets that overlap the backward
pass, replicated SGD update.

The reference is single-GPU; this wrapper is what lets the AM ops train on the
GPUs of one box.  The AM forward and input-gradient ops are independent per
sample and the filter / weight gradients are sums over the batch, so sharding
the batch needs exactly one collective per step: all-reduce(sum) of the
gradients, divided by the world size (each rank's loss is a mean over its own
shard).  Batch-norm statistics stay per replica.

Gradients live in flat bucket buffers (``param.grad`` are views into them), so
the all-reduce runs on the memory autograd accumulated into, without a staging
copy.  A bucket is reduced as soon as all its gradients are ready.
Works with any ``torch.distributed`` backend (``nccl`` on GPUs, ``gloo`` in
the CPU tests) and degenerates to plain SGD without a process group.
"""
from __future__ import annotations

from typing import Callable, List

import torch
import torch.distributed as dist


class DataParallelSGD:
    def __init__(self, model: torch.nn.Module, lr: float, bucket_bytes: int = 32 << 20, process_group=None):
        self.model = model
        self.lr = lr
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.params: List[torch.nn.Parameter] = [p for p in model.parameters() if p.requires_grad]
        if self.world > 1:
            for t in list(model.parameters()) + list(model.buffers()):
                dist.broadcast(t.data, src=0, group=process_group)
        # Buckets in reverse registration order: backward produces gradients roughly last layer first.
        self.buckets = []      # list of dict(flat, params, pending)
        cur, cur_bytes = [], 0
        for p in reversed(self.params):
            cur.append(p)
            cur_bytes += p.numel() * p.element_size()
            if cur_bytes >= bucket_bytes:
                self._close_bucket(cur)
                cur, cur_bytes = [], 0
        if cur:
            self._close_bucket(cur)
        self._handles = []
        self._defer_allreduce = False   # while a step is being captured into a CUDA graph
        self._expect = None             # per parameter: gradient reports per step (learned on the first step)
        self._late = False
        # Gradient kernels of the AM layers write straight into the bucket memory (layers.GradSink):
        # no per-parameter accumulate kernel, and NCCL reduces the memory the kernels wrote.
        from .layers import GradSink
        self._sinks = []
        for bi, b in enumerate(self.buckets):
            hook = self._make_hook(bi) if self.world > 1 else None
            for p in b["params"]:
                if self.world > 1:
                    p.register_post_accumulate_grad_hook(hook)
                p.amsim_grad_sink = GradSink(p.grad, hook)
                self._sinks.append(p.amsim_grad_sink)

    def _close_bucket(self, params):
        n = sum(p.numel() for p in params)
        flat = torch.zeros(n, dtype=params[0].dtype, device=params[0].device)
        off = 0
        for p in params:
            p.grad = flat[off:off + p.numel()].view_as(p)
            off += p.numel()
        self.buckets.append({"flat": flat, "params": params, "pending": len(params), "fired": {}, "launched": False})

    def _make_hook(self, bi):
        def hook(param):
            # Called when a gradient contribution of `param` is in place: by autograd after it
            # accumulated one, and by an AM layer that wrote the gradient into the bucket itself
            # (layers.GradSink).  A parameter may be reported several times per step: a shared
            # parameter once per use, and a directly written one a second time by autograd, which
            # fires its post-accumulate hook even for a gradient function that returned None
            # (torch 2.11).  So the first step only counts the reports per parameter (its buckets
            # are reduced after backward); from then on a parameter is complete at its last
            # expected report, and a bucket is reduced when all its parameters are.
            b = self.buckets[bi]
            n = b["fired"].get(id(param), 0) + 1
            b["fired"][id(param)] = n
            if self._expect is None or self._defer_allreduce:
                return
            want = self._expect.get(id(param), 0)
            if n == want:
                b["pending"] -= 1
                if b["pending"] == 0 and not b["launched"]:
                    b["launched"] = True
                    self._handles.append(dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            elif n > want and b["launched"]:
                self._late = True   # a contribution after the bucket went out: the graph changed
        return hook

    def zero_grad(self):
        for b in self.buckets:
            b["flat"].zero_()
            b["fired"] = {}
            b["launched"] = False
            b["pending"] = (sum(1 for p in b["params"] if self._expect.get(id(p), 0) > 0)
                            if self._expect is not None else len(b["params"]))
        for s in self._sinks:
            s.reset()
        self._handles = []
        self._late = False

    def _finish_allreduce(self):
        """After backward: wait for the overlapped reductions, reduce the buckets that have not gone out
        (first step; parameters that received no gradient), remember how often each parameter reports."""
        for h in self._handles:
            h.wait()
        if self.world > 1:
            if self._late:
                raise RuntimeError("a parameter received a gradient contribution after its bucket had been "
                                   "all-reduced: the autograd graph changed between steps")
            for b in self.buckets:
                if not b["launched"]:
                    dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group)
                    b["launched"] = True
            fired = {}
            for b in self.buckets:
                fired.update(b["fired"])
            if self._expect is None or any(fired.get(k, 0) != v for k, v in self._expect.items()):
                # first step, or a step that used the parameters differently: the next step starts
                # from these counts (this one was reduced correctly: every late report raises above,
                # and a bucket whose parameters reported less often than expected went out just now)
                self._expect = {id(p): fired.get(id(p), 0) for p in self.params}

    def step(self, loss_fn: Callable[[], torch.Tensor]) -> torch.Tensor:
        """zero grads, ``loss = loss_fn()``, backward (all-reduce overlapped), SGD update."""
        self.zero_grad()
        loss = loss_fn()
        loss.backward()
        self._finish_allreduce()
        self._update()
        return loss.detach()

    def _update(self):
        """Replicated SGD update p -= lr * mean-over-ranks(grad), all parameters in a few multi-tensor launches."""
        scale = self.lr / self.world
        with torch.no_grad():
            torch._foreach_add_(self.params, [p.grad for p in self.params], alpha=-scale)

    def capture(self, loss_fn: Callable[[], torch.Tensor], warmup: int = 3):
        """Record one train step into CUDA graphs and return ``replay() -> loss``: replaying removes
        the per-launch host cost of the several hundred small exact kernels around the AM ops
        (normalisation, activations, pooling, bias gradients), which is what bounds the launch-bound
        LeNet configurations and costs the large networks a few percent.  The tensors ``loss_fn``
        reads must be static (copy new batches into them).

        Single process: one graph holds zero-grads, forward, backward and the SGD update.
        With a process group: one graph holds zero-grads, forward and backward; the gradient
        buckets are then all-reduced by ordinary (not captured) collective calls and a second graph
        applies the update.  The all-reduce no longer overlaps the backward pass; on NVLink it is
        well under a millisecond for the ~100 MB of a ResNet-50."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):   # also triggers every lazy one-time set-up outside the capture
                self.step(loss_fn)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if self.world == 1:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                loss = self.step(loss_fn)

            def replay():
                graph.replay()
                return loss
            replay.graph = graph
            return replay

        fwd_bwd, update = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        self._defer_allreduce = True
        try:
            with torch.cuda.graph(fwd_bwd):
                self.zero_grad()
                loss = loss_fn()
                loss.backward()
                loss = loss.detach()
            with torch.cuda.graph(update, pool=fwd_bwd.pool()):
                self._update()
        finally:
            self._defer_allreduce = False

        def replay():
            fwd_bwd.replay()
            handles = [dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True) for b in self.buckets]
            for h in handles:
                h.wait()
            update.replay()
            return loss
        replay.graph = fwd_bwd
        return replay

    def gradient_bytes(self) -> int:
        return sum(b["flat"].numel() * b["flat"].element_size() for b in self.buckets)
