"""Data-parallel training with the AM ops on two GPUs (NCCL): a batch sharded over
two ranks must give the update of the full batch on one GPU, within the FP32
reduction-order tolerance, for the networks without batch statistics: LeNet-300-100
(denseam layers) and LeNet-5 (AMConv2D filter gradients cross the all-reduce too).
The NCCL cases are skipped where fewer than two GPUs are visible; the same check also
runs with both ranks on ONE GPU over gloo (the ranks' kernels never wait on one another:
the exchange is a host-side collective), so a single-GPU box covers the trainer with the
real AM kernels too."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import lut_path

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _data(which):
    g = torch.Generator().manual_seed(3)
    shape = (64, 784) if which == "lenet300100" else (64, 28, 28, 1)
    return torch.rand(*shape, generator=g), torch.randint(0, 10, (64,), generator=g)


def _net(which, dev):
    from approxtrain_b200.nets import LeNet5, LeNet300100
    torch.manual_seed(0)
    if which == "lenet300100":
        return LeNet300100(lut_path("MBM_7")).to(dev)
    return LeNet5(lut_path("MIT_7")).to(dev)


def _worker(rank, world, port, out, which, graph=False, one_gpu=False, bucket_bytes=32 << 20):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(0 if one_gpu else rank)
    dist.init_process_group("gloo" if one_gpu else "nccl", rank=rank, world_size=world)
    from approxtrain_b200.dp import DataParallelSGD
    dev = torch.device("cuda", 0 if one_gpu else rank)
    net = _net(which, dev)
    tr = DataParallelSGD(net, lr=0.05, bucket_bytes=bucket_bytes)
    x, y = _data(which)
    n = x.shape[0] // world
    xs, ys = x[rank * n:(rank + 1) * n].to(dev), y[rank * n:(rank + 1) * n].to(dev)
    fn = lambda: torch.nn.functional.cross_entropy(net(xs), ys)
    if graph:
        # one eager warm-up step, then the step replayed from CUDA graphs (forward + backward captured,
        # all-reduce between the graphs, update captured): two steps in all, like the eager run
        replay = tr.capture(fn, warmup=1)
        replay()
    else:
        for _ in range(2):
            tr.step(fn)
    torch.cuda.synchronize()
    torch.save([p.detach().cpu() for p in net.parameters()], os.path.join(out, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


# (network, replay from CUDA graphs, bucket size): the small buckets split LeNet-5's ten parameters over
# several all-reduces that start while backward is still running on both of the layers' streams
CASES = [("lenet300100", False, 32 << 20), ("lenet5", False, 32 << 20), ("lenet5", True, 32 << 20), ("lenet5", False, 4096),
         ("lenet300100", False, 100000)]
IDS = ["lenet300100", "lenet5", "lenet5-graphs", "lenet5-small-buckets", "lenet300100-small-buckets"]


@pytest.mark.parametrize("which,graph,bucket_bytes", CASES, ids=IDS)
def test_two_gpus_give_the_full_batch_update(tmp_path, which, graph, bucket_bytes):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _check(tmp_path, which, graph, False, bucket_bytes)


@pytest.mark.parametrize("which,graph,bucket_bytes", CASES, ids=IDS)
def test_two_ranks_on_one_gpu_give_the_full_batch_update(tmp_path, which, graph, bucket_bytes):
    _check(tmp_path, which, graph, True, bucket_bytes)


def _check(tmp_path, which, graph, one_gpu, bucket_bytes):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), which, graph, one_gpu, bucket_bytes), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "rank0.pt")
    r1 = torch.load(tmp_path / "rank1.pt")
    for a, b in zip(r0, r1):
        assert torch.equal(a, b), "replicas diverged"
    # one GPU, whole batch, plain SGD on the mean loss
    from approxtrain_b200.dp import DataParallelSGD
    dev = torch.device("cuda", 0)
    net = _net(which, dev)
    tr = DataParallelSGD(net, lr=0.05)
    x, y = _data(which)
    x, y = x.to(dev), y.to(dev)
    for _ in range(2):
        tr.step(lambda: torch.nn.functional.cross_entropy(net(x), y))
    worst = 0.0
    for a, p in zip(r0, net.parameters()):
        worst = max(worst, float((a - p.detach().cpu()).abs().max()))
        assert torch.allclose(a, p.detach().cpu(), atol=1e-6, rtol=1e-4)
    print(f"{which}{' (CUDA graphs)' if graph else ''}: replicas identical on {'one GPU, 2 gloo ranks' if one_gpu else '2 GPUs'}; "
          f"max |sharded - full batch| over all parameters {worst:.3e}")
