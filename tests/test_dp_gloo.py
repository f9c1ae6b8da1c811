"""Data-parallel wrapper on CPU ranks (gloo, world size 2): the bucketed,
hook-driven all-reduce must give every rank the gradient of the full batch and
keep the replicas identical.  The AM ops need a GPU, so the model here is a
plain torch MLP: what is tested is the host-side sharding/collective logic."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _model():
    torch.manual_seed(5)
    return torch.nn.Sequential(torch.nn.Linear(12, 16), torch.nn.ReLU(), torch.nn.Linear(16, 16), torch.nn.ReLU(),
                               torch.nn.Linear(16, 3))


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from approxtrain_b200.dp import DataParallelSGD
    model = _model()
    if rank == 1:  # replicas start different: the wrapper must broadcast rank 0's weights
        with torch.no_grad():
            for p in model.parameters():
                p.add_(1.0)
    tr = DataParallelSGD(model, lr=0.1, bucket_bytes=100)  # tiny buckets: several collectives per step
    assert len(tr.buckets) > 2
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, 12, generator=g)
    y = torch.randint(0, 3, (8,), generator=g)
    xs, ys = x[rank * 4:(rank + 1) * 4], y[rank * 4:(rank + 1) * 4]
    for _ in range(3):
        tr.step(lambda: torch.nn.functional.cross_entropy(model(xs), ys))
    torch.save([p.detach().clone() for p in model.parameters()], os.path.join(out, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_matches_full_batch_sgd(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "rank0.pt")
    r1 = torch.load(tmp_path / "rank1.pt")
    for a, b in zip(r0, r1):
        assert torch.equal(a, b), "replicas diverged"
    # single-process reference: plain SGD on the full batch (mean loss)
    model = _model()
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, 12, generator=g)
    y = torch.randint(0, 3, (8,), generator=g)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for _ in range(3):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    for a, p in zip(r0, model.parameters()):
        assert torch.allclose(a, p.detach(), atol=1e-6, rtol=1e-5)


def test_single_process_is_plain_sgd():
    from approxtrain_b200.dp import DataParallelSGD
    m1, m2 = _model(), _model()
    tr = DataParallelSGD(m1, lr=0.05)
    opt = torch.optim.SGD(m2.parameters(), lr=0.05)
    x = torch.randn(6, 12)
    y = torch.randint(0, 3, (6,))
    for _ in range(2):
        tr.step(lambda: torch.nn.functional.cross_entropy(m1(x), y))
        opt.zero_grad()
        torch.nn.functional.cross_entropy(m2(x), y).backward()
        opt.step()
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.allclose(a, b, atol=1e-7)


# ---- the same through the AM layers' direct gradient writes (layers.GradSink) -------------------
# The AM ops need a GPU; here exact torch stand-ins take their place, so what runs is the layers'
# backward wiring (gradient kernels writing into the all-reduce buckets, the trainer's hooks called
# from the layer instead of from autograd) on CPU ranks.
def _install_cpu_ops():
    from approxtrain_b200 import ops

    def denseam_bias_act(x, w, b, activation=None, mant_mul_lut="", deterministic=False):
        y = x @ w
        if b is not None:
            y = y + b
        return torch.relu(y) if activation == "relu" else y

    def denseam_grad(g, x, w, lut="", deterministic=False, out_weights=None, weights_stream=None):
        dw = x.t() @ g
        if out_weights is not None:
            out_weights.copy_(dw)
            dw = out_weights
        return g @ w.t(), dw

    def bias_grad(g, out=None):
        db = g.reshape(-1, g.shape[-1]).sum(0)
        if out is not None:
            out.copy_(db)
            db = out
        return db

    ops.denseam_bias_act, ops.denseam_grad, ops.bias_grad = denseam_bias_act, denseam_grad, bias_grad


class _SinkMLP(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(5)
        self.w = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(i, o) * 0.3) for i, o in ((12, 16), (16, 16), (16, 3))])
        self.b = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(o) * 0.1) for o in (16, 16, 3)])

    def forward(self, x):
        from approxtrain_b200.layers import _DenseamBiasActFn
        for i in range(3):
            x = _DenseamBiasActFn.apply(x, self.w[i], self.b[i], "relu" if i < 2 else None, "", False)
        return x


def _sink_worker(rank, world, port, out, bucket_bytes):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _install_cpu_ops()
    from approxtrain_b200.dp import DataParallelSGD
    model = _SinkMLP()
    tr = DataParallelSGD(model, lr=0.1, bucket_bytes=bucket_bytes)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, 12, generator=g)
    y = torch.randint(0, 3, (8,), generator=g)
    xs, ys = x[rank * 4:(rank + 1) * 4], y[rank * 4:(rank + 1) * 4]
    for _ in range(3):
        tr.step(lambda: torch.nn.functional.cross_entropy(model(xs), ys))
    torch.save([p.detach().clone() for p in model.parameters()], os.path.join(out, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("bucket_bytes", [100, 32 << 20], ids=["many-buckets", "one-bucket"])
def test_two_rank_gloo_with_direct_gradient_writes(tmp_path, bucket_bytes):
    mp.spawn(_sink_worker, args=(2, _free_port(), str(tmp_path), bucket_bytes), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "rank0.pt")
    r1 = torch.load(tmp_path / "rank1.pt")
    for a, b in zip(r0, r1):
        assert torch.equal(a, b), "replicas diverged"
    model = _SinkMLP()
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, 12, generator=g)
    y = torch.randint(0, 3, (8,), generator=g)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for _ in range(3):
        opt.zero_grad()
        h = x
        for i in range(3):
            h = h @ model.w[i] + model.b[i]
            if i < 2:
                h = torch.relu(h)
        torch.nn.functional.cross_entropy(h, y).backward()
        opt.step()
    for a, p in zip(r0, model.parameters()):
        assert torch.allclose(a, p.detach(), atol=1e-6, rtol=1e-5)


# ---- a parameter used twice in the graph reports twice per step --------------------------------
class _SharedMLP(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(9)
        self.a, self.shared, self.c = torch.nn.Linear(12, 16), torch.nn.Linear(16, 16), torch.nn.Linear(16, 3)

    def forward(self, x):
        h = torch.relu(self.a(x))
        h = torch.relu(self.shared(h))
        h = torch.relu(self.shared(h))   # same weights again: two gradient contributions per step
        return self.c(h)


def _shared_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from approxtrain_b200.dp import DataParallelSGD
    model = _SharedMLP()
    tr = DataParallelSGD(model, lr=0.1, bucket_bytes=100)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, 12, generator=g)
    y = torch.randint(0, 3, (8,), generator=g)
    xs, ys = x[rank * 4:(rank + 1) * 4], y[rank * 4:(rank + 1) * 4]
    for _ in range(3):
        tr.step(lambda: torch.nn.functional.cross_entropy(model(xs), ys))
    torch.save([p.detach().clone() for p in model.parameters()], os.path.join(out, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_with_a_shared_parameter(tmp_path):
    mp.spawn(_shared_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "rank0.pt")
    r1 = torch.load(tmp_path / "rank1.pt")
    for a, b in zip(r0, r1):
        assert torch.equal(a, b), "replicas diverged"
    model = _SharedMLP()
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, 12, generator=g)
    y = torch.randint(0, 3, (8,), generator=g)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for _ in range(3):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    for a, p in zip(r0, model.parameters()):
        assert torch.allclose(a, p.detach(), atol=1e-6, rtol=1e-5)
