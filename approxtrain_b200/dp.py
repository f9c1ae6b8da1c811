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
        self.buckets.append({"flat": flat, "params": params, "pending": len(params)})

    def _make_hook(self, bi):
        def hook(_param):
            b = self.buckets[bi]
            b["pending"] -= 1
            if b["pending"] == 0 and not self._defer_allreduce:
                self._handles.append(dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        return hook

    def zero_grad(self):
        for b in self.buckets:
            b["flat"].zero_()
            b["pending"] = len(b["params"])
        for s in self._sinks:
            s.reset()
        self._handles = []

    def step(self, loss_fn: Callable[[], torch.Tensor]) -> torch.Tensor:
        """zero grads, ``loss = loss_fn()``, backward (all-reduce overlapped), SGD update."""
        self.zero_grad()
        loss = loss_fn()
        loss.backward()
        for h in self._handles:
            h.wait()
        if self.world > 1:
            # a parameter that received no gradient never fires its hook: reduce what is left
            for b in self.buckets:
                if b["pending"] != 0:
                    dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group)
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
