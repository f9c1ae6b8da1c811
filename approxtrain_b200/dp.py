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
        if self.world > 1:
            for bi, b in enumerate(self.buckets):
                for p in b["params"]:
                    p.register_post_accumulate_grad_hook(self._make_hook(bi))

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
            if b["pending"] == 0:
                self._handles.append(dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        return hook

    def zero_grad(self):
        for b in self.buckets:
            b["flat"].zero_()
            b["pending"] = len(b["params"])
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
        scale = self.lr / self.world
        with torch.no_grad():
            for p in self.params:
                p.add_(p.grad, alpha=-scale)
        return loss.detach()

    def capture(self, loss_fn: Callable[[], torch.Tensor], warmup: int = 3):
        """Record one whole train step (zero grads, forward, backward, SGD update) into a
        CUDA graph and return ``replay() -> loss``.  For launch-bound networks (the LeNet
        configurations: ~60-100 kernels of a few microseconds each) replaying the graph
        removes the per-launch host cost.  The tensors ``loss_fn`` reads must be static
        (copy new batches into them).  Single process only: the hook-driven all-reduce
        is not captured."""
        if self.world > 1:
            raise RuntimeError("capture() supports a single process; use step() with a process group")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):   # also triggers every lazy one-time set-up outside the capture
                self.step(loss_fn)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            loss = self.step(loss_fn)

        def replay():
            graph.replay()
            return loss
        replay.graph = graph
        return replay

    def gradient_bytes(self) -> int:
        return sum(b["flat"].numel() * b["flat"].element_size() for b in self.buckets)
