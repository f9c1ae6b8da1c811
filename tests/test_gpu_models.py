"""GPU tests of the layers / networks built on the AM ops: gradient wiring
against the oracle (bit-exact in deterministic mode, operands captured from the
running network), and train-step sanity for the configured networks."""
import numpy as np
import pytest

from conftest import lut_path, rel_l2

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def beq(a, b):
    return np.array_equal(np.ascontiguousarray(a, np.float32).view(np.uint32), np.ascontiguousarray(b, np.float32).view(np.uint32))


def test_lenet300100_step_against_oracle(oracle, luts):
    """Benchmark configuration 1 (LeNet-300-100): 784-300-100-10, batch 256, x ~ U[0,1), MBM_7, one
    forward + backward + SGD step.  Logits are bit-exact vs the oracle; each
    layer's gradients are bit-exact given the upstream gradient torch produced."""
    from approxtrain_b200.nets import LeNet300100
    from approxtrain_b200.dp import DataParallelSGD
    lut, m = luts["MBM_7"]
    torch.manual_seed(0)
    net = LeNet300100(lut_path("MBM_7"), deterministic=True).cuda()
    g = torch.Generator().manual_seed(0)
    x = torch.rand(256, 28, 28, 1, generator=g).cuda()
    y = torch.randint(0, 10, (256,), generator=g).cuda()
    W = [p.detach().cpu().numpy().copy() for p in (net.fc1.kernel, net.fc2.kernel, net.fc3.kernel)]
    B = [p.detach().cpu().numpy().copy() for p in (net.fc1.bias, net.fc2.bias, net.fc3.bias)]
    # oracle forward
    h0 = x.cpu().numpy().reshape(256, -1)
    z1 = oracle.dense_fwd(h0, W[0], lut, m) + B[0]
    h1 = np.maximum(z1, 0)
    z2 = oracle.dense_fwd(h1, W[1], lut, m) + B[1]
    h2 = np.maximum(z2, 0)
    z3 = oracle.dense_fwd(h2, W[2], lut, m) + B[2]
    logits = net(x)
    assert beq(logits.detach().cpu().numpy(), z3)
    loss = torch.nn.functional.cross_entropy(logits, y)
    loss.backward()
    # upstream gradient as torch computed it, then the oracle's backward chain
    p = torch.softmax(logits.detach(), -1)
    p[torch.arange(256), y] -= 1
    g3 = (p / 256).cpu().numpy()
    assert rel_l2(net.fc3.bias.grad.cpu().numpy(), g3.sum(0)) < 1e-5
    dW3 = oracle.dense_bwd_weight(h2, g3, lut, m)
    assert rel_l2(net.fc3.kernel.grad.cpu().numpy(), dW3) < 1e-5
    dh2 = oracle.dense_bwd_input(W[2], g3, lut, m)
    g2 = dh2 * (z2 > 0)
    assert rel_l2(net.fc2.kernel.grad.cpu().numpy(), oracle.dense_bwd_weight(h1, g2, lut, m)) < 1e-5
    g1 = oracle.dense_bwd_input(W[1], g2, lut, m) * (z1 > 0)
    assert rel_l2(net.fc1.kernel.grad.cpu().numpy(), oracle.dense_bwd_weight(h0, g1, lut, m)) < 1e-5
    # SGD through the wrapper lowers the loss on the same batch
    net.zero_grad(set_to_none=True)
    tr = DataParallelSGD(net, lr=0.1)
    l0 = float(tr.step(lambda: torch.nn.functional.cross_entropy(net(x), y)))
    for _ in range(5):
        l1 = float(tr.step(lambda: torch.nn.functional.cross_entropy(net(x), y)))
    assert l1 < l0


def test_conv_layer_gradient_wiring_bit_exact(oracle, luts):
    """Convam -> (ConvamInputGrad, ConvamFilterGrad) as in python/ops/amnn_ops.py:220-244."""
    from approxtrain_b200.layers import amconv2d
    lut, m = luts["MIT_7"]
    rng = np.random.default_rng(2)
    x = torch.from_numpy(rng.standard_normal((3, 9, 9, 6)).astype(np.float32)).cuda().requires_grad_()
    w = torch.from_numpy(rng.standard_normal((5, 5, 6, 16)).astype(np.float32)).cuda().requires_grad_()
    y = amconv2d(x, w, [1, 2, 2, 1], "SAME", lut_path("MIT_7"), True)
    dy = torch.from_numpy(rng.standard_normal(tuple(y.shape)).astype(np.float32)).cuda()
    y.backward(dy)
    g = oracle.geometry(3, 9, 9, 6, 5, 5, 16, 2, 2, "SAME")
    xn, wn, dyn = x.detach().cpu().numpy(), w.detach().cpu().numpy(), dy.cpu().numpy()
    assert beq(y.detach().cpu().numpy(), oracle.conv2d_fwd(g, xn, wn, lut, m))
    assert beq(x.grad.cpu().numpy(), oracle.conv2d_bwd_input(g, wn, dyn, lut, m))
    assert beq(w.grad.cpu().numpy(), oracle.conv2d_bwd_filter(g, xn, dyn, lut, m))


def test_matmul_gradient_wiring(oracle, luts):
    """dA = MatMulAM(g, B^T), dB = MatMulAM(A^T, g), rank-4 attention-shaped operands."""
    from approxtrain_b200.layers import ammatmul
    lut, m = luts["MIT_7"]
    rng = np.random.default_rng(6)
    a = torch.from_numpy(rng.standard_normal((2, 3, 8, 5)).astype(np.float32)).cuda().requires_grad_()
    b = torch.from_numpy(rng.standard_normal((2, 3, 5, 7)).astype(np.float32)).cuda().requires_grad_()
    c = ammatmul(a, b, lut_path("MIT_7"), True)
    g = torch.from_numpy(rng.standard_normal(tuple(c.shape)).astype(np.float32)).cuda()
    c.backward(g)
    an, bn, gn = (t.detach().cpu().numpy().reshape(6, *t.shape[-2:]) for t in (a, b, g))
    assert beq(c.detach().cpu().numpy().reshape(6, 8, 7), oracle.matmul(an, bn, lut, m))
    assert beq(a.grad.cpu().numpy().reshape(6, 8, 5), oracle.matmul(gn, np.ascontiguousarray(bn.transpose(0, 2, 1)), lut, m))
    assert beq(b.grad.cpu().numpy().reshape(6, 5, 7), oracle.matmul(np.ascontiguousarray(an.transpose(0, 2, 1)), gn, lut, m))


@pytest.mark.parametrize("sa,sb", [((1, 8, 5), (4, 5, 7)), ((4, 8, 5), (1, 5, 7)), ((8, 5), (4, 5, 7)), ((4, 8, 5), (5, 7))])
def test_matmul_gradient_of_a_broadcast_operand(oracle, luts, sa, sb):
    """An operand that MatMulAM broadcasts over the batch (rank 2, or rank 3 with batch 1) gets the
    sum of the per-batch gradients, in its own shape."""
    from approxtrain_b200.layers import ammatmul
    lut, m = luts["MBM_7"]
    rng = np.random.default_rng(26)
    an, bn = rng.standard_normal(sa).astype(np.float32), rng.standard_normal(sb).astype(np.float32)
    a = torch.from_numpy(an).cuda().requires_grad_()
    b = torch.from_numpy(bn).cuda().requires_grad_()
    c = ammatmul(a, b, lut_path("MBM_7"), True)
    gn = rng.standard_normal(tuple(c.shape)).astype(np.float32)
    c.backward(torch.from_numpy(gn).cuda())
    assert a.grad.shape == a.shape and b.grad.shape == b.shape
    nb = gn.shape[0]
    af = np.broadcast_to(an.reshape(-1, *an.shape[-2:]), (nb, *an.shape[-2:])).copy()
    bf = np.broadcast_to(bn.reshape(-1, *bn.shape[-2:]), (nb, *bn.shape[-2:])).copy()
    T = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1))
    da = torch.from_numpy(oracle.matmul(gn, T(bf), lut, m))
    db = torch.from_numpy(oracle.matmul(T(af), gn, lut, m))
    want_a = da.sum(0).reshape(sa) if (len(sa) == 2 or sa[0] == 1) else da
    want_b = db.sum(0).reshape(sb) if (len(sb) == 2 or sb[0] == 1) else db
    assert rel_l2(a.grad.cpu().numpy(), want_a.numpy()) <= 1e-6
    assert rel_l2(b.grad.cpu().numpy(), want_b.numpy()) <= 1e-6


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
def test_matmul_gradient_wiring_with_transposes_and_alpha(oracle, luts, ta, tb):
    """The four transpose cases of the reference's MatMulAM gradient (math_ops.py:127-157),
    alpha applied to both gradients."""
    from approxtrain_b200.layers import ammatmul
    lut, m = luts["MIT_7"]
    rng = np.random.default_rng(16)
    M, K, N, al = 8, 5, 7, 0.25
    an = rng.standard_normal((6, K, M) if ta else (6, M, K)).astype(np.float32)
    bn = rng.standard_normal((6, N, K) if tb else (6, K, N)).astype(np.float32)
    a = torch.from_numpy(an).cuda().requires_grad_()
    b = torch.from_numpy(bn).cuda().requires_grad_()
    c = ammatmul(a, b, lut_path("MIT_7"), True, transpose_a=ta, transpose_b=tb, alpha=al)
    gn = rng.standard_normal((6, M, N)).astype(np.float32)
    c.backward(torch.from_numpy(gn).cuda())
    T = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1))
    opa, opb = (T(an) if ta else an), (T(bn) if tb else bn)
    assert beq(c.detach().cpu().numpy(), oracle.matmul(opa, opb, lut, m) * np.float32(al))
    if not ta:
        want_da = oracle.matmul(gn, T(opb), lut, m)
    else:
        want_da = oracle.matmul(opb, T(gn), lut, m)
    if not tb:
        want_db = oracle.matmul(T(opa), gn, lut, m)
    else:
        want_db = oracle.matmul(T(gn), opa, lut, m)
    assert beq(a.grad.cpu().numpy(), want_da * np.float32(al))
    assert beq(b.grad.cpu().numpy(), want_db * np.float32(al))


def test_lenet5_trains_on_a_fixed_batch():
    """Benchmark configuration 2 (LeNet-5) shapes: batch 128 of 28x28x1, MIT_7, He-normal."""
    from approxtrain_b200.nets import LeNet5
    from approxtrain_b200.dp import DataParallelSGD
    torch.manual_seed(0)
    net = LeNet5(lut_path("MIT_7")).cuda()
    g = torch.Generator().manual_seed(0)
    x = torch.rand(128, 28, 28, 1, generator=g).cuda()
    y = torch.randint(0, 10, (128,), generator=g).cuda()
    tr = DataParallelSGD(net, lr=0.05)
    losses = [float(tr.step(lambda: torch.nn.functional.cross_entropy(net(x), y))) for _ in range(8)]
    assert np.isfinite(losses).all() and losses[-1] < losses[0]


def test_resnet50_am_step_runs():
    from approxtrain_b200.nets import ResNet50AM
    from approxtrain_b200.dp import DataParallelSGD
    torch.manual_seed(0)
    net = ResNet50AM(lut_path("MBM_7")).cuda()
    n_conv = sum(1 for mod in net.modules() if mod.__class__.__name__ == "AMConv2D")
    assert n_conv == 53
    x = torch.randn(2, 224, 224, 3, device="cuda")
    y = torch.randint(0, 1000, (2,), device="cuda")
    feats = {}
    def _shape_hook(mod, inp, out):
        feats["s2"] = tuple(out.shape)
    net.blocks[0].register_forward_hook(_shape_hook)
    tr = DataParallelSGD(net, lr=0.01)
    loss = tr.step(lambda: torch.nn.functional.cross_entropy(net(x), y))
    assert feats["s2"] == (2, 55, 55, 256)   # unpadded 3x3/2 max pool: 55x55 at stage 2
    assert torch.isfinite(loss)
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.parameters())


def test_transformer_am_small_step_runs():
    from approxtrain_b200.nets import TransformerAM
    from approxtrain_b200.dp import DataParallelSGD
    torch.manual_seed(0)
    net = TransformerAM(lut_path("MIT_7"), vocab=120, layers=2, d_model=64, heads=4, d_ff=128, d_k=64, d_v=64).cuda()
    src = torch.randint(1, 120, (4, 16), device="cuda")
    tgt = torch.randint(1, 120, (4, 16), device="cuda")
    src[0, 12:] = 0  # padding
    tr = DataParallelSGD(net, lr=0.01)
    l0 = float(tr.step(lambda: torch.nn.functional.cross_entropy(net(src, tgt[:, :-1]).reshape(-1, 120), tgt[:, 1:].reshape(-1))))
    for _ in range(6):
        l1 = float(tr.step(lambda: torch.nn.functional.cross_entropy(net(src, tgt[:, :-1]).reshape(-1, 120), tgt[:, 1:].reshape(-1))))
    assert np.isfinite(l1) and l1 < l0


class _ConvStack(torch.nn.Module):
    """Three 3x3 AMConv2D layers and a dense head, sized so that their forward / input-gradient launches
    share tiles between CTAs (balanced launches) inside a graph capture too."""

    def __init__(self, lut):
        super().__init__()
        from approxtrain_b200.layers import AMConv2D, denseam
        kw = dict(mant_mul_lut=lut, kernel_initializer="he_normal")
        self.c1 = AMConv2D(8, 32, 3, padding="same", activation="relu", **kw)
        self.c2 = AMConv2D(32, 64, 3, padding="same", activation="relu", **kw)
        self.c3 = AMConv2D(64, 64, 3, padding="same", activation="relu", **kw)
        self.f = denseam(64, 10, **kw)

    def forward(self, x):
        return self.f(self.c3(self.c2(self.c1(x))).mean((1, 2)))


@pytest.mark.parametrize("which", ["lenet5", "conv_stack"])
def test_cuda_graph_replay_matches_eager_steps(which):
    """The whole train step (ops, split-K reduction, cluster and balanced launches, SGD update) is
    capturable; replaying it gives the eager losses bit for bit.  In the capture the balanced launches
    park their partial tiles in the persistent scratch, whose tile counters the kernel itself leaves at
    zero for the next launch: a counter left dirty would show as a different (or missing) tile sum in
    the second replay."""
    from approxtrain_b200.nets import LeNet5
    from approxtrain_b200.dp import DataParallelSGD
    g = torch.Generator().manual_seed(3)
    if which == "lenet5":
        x = torch.rand(64, 28, 28, 1, generator=g).cuda()
    else:
        x = torch.rand(16, 24, 24, 8, generator=g).cuda()
    y = torch.randint(0, 10, (x.shape[0],), generator=g).cuda()

    def run(graphed):
        torch.manual_seed(1)
        net = (LeNet5(lut_path("MIT_7")) if which == "lenet5" else _ConvStack(lut_path("MBM_7"))).cuda()
        tr = DataParallelSGD(net, lr=0.05)
        fn = lambda: torch.nn.functional.cross_entropy(net(x), y)
        if not graphed:
            return [float(tr.step(fn)) for _ in range(3 + 4)]   # capture() runs 3 warm-up steps; recording does not execute
        replay = tr.capture(fn, warmup=3)
        return [float(replay()) for _ in range(4)]

    eager = run(False)
    graph = run(True)
    assert graph == eager[3:], (graph, eager)


def test_gradients_written_straight_into_the_buckets_equal_autograd_accumulation():
    """DataParallelSGD hands every parameter a view into its flat gradient bucket; the AM layers'
    gradient kernels (filter / weight gradient, bias gradient) write into that view directly.  The
    result must be the bits autograd's own accumulation gives (sinks removed), also for a layer
    that is applied twice in one step (shared weights: autograd sums the two contributions)."""
    from approxtrain_b200.layers import AMConv2D, denseam
    from approxtrain_b200.dp import DataParallelSGD

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            kw = dict(mant_mul_lut=lut_path("MBM_7"), kernel_initializer="he_normal")
            self.c1 = AMConv2D(4, 8, 3, padding="same", activation="relu", **kw)
            self.c2 = AMConv2D(8, 8, 3, padding="same", activation="relu", **kw)   # applied twice
            self.f = denseam(8 * 6 * 6, 10, **kw)

        def forward(self, x):
            y = self.c2(self.c2(self.c1(x)))
            return self.f(y.reshape(y.shape[0], -1))

    g = torch.Generator().manual_seed(4)
    x = torch.randn(16, 6, 6, 4, generator=g).cuda()
    y = torch.randint(0, 10, (16,), generator=g).cuda()

    def run(direct):
        torch.manual_seed(2)
        net = Net().cuda()
        tr = DataParallelSGD(net, lr=0.05)
        if not direct:
            for p in net.parameters():
                del p.amsim_grad_sink
            tr._sinks = []
        losses = [float(tr.step(lambda: torch.nn.functional.cross_entropy(net(x), y))) for _ in range(3)]
        used = [s.uses for s in tr._sinks]
        return losses, [p.detach().clone() for p in net.parameters()], used

    l_direct, p_direct, used = run(True)
    l_plain, p_plain, _ = run(False)
    assert sorted(used) == [1, 1, 1, 1, 2, 2]     # c1 and f (weight, bias) once each, c2 twice
    assert l_direct == l_plain
    for a, b in zip(p_direct, p_plain):
        assert torch.equal(a, b)


def test_bench_prints_one_complete_line_for_a_small_workload():
    """bench.py end to end on the smallest train workload: timed region, end-to-end leg, the
    instrumented step behind `am_ops` (event pairs around every op call, including the ones that
    write into gradient buckets), CUDA-graph replay, one JSON line with the keys the contract names."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "lenet5", "--steps", "5", "--warmup", "3",
                          "--no-cpu-baseline"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-3000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "dtype",
                "data", "config", "clocks", "e2e", "gpu_launches", "roofline", "am_ops"):
        assert key in d, key
    assert d["value"] > 0 and d["gpu_launches"] > 0 and d["e2e"]["value"] > 0 and d["e2e"]["h2d_bytes_per_step"] > 0
    assert d["am_ops"]["layers"] and d["roofline"]["frac"] > 0


def test_bench_single_layer_workload():
    """bench.py --workload layer: one AMConv2D layer's three ops timed in isolation, one JSON line."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "layer", "--shape", "4,14,14,32,3,3,64,1,SAME",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-3000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert [k["op"] for k in d["kernels"]] == ["fwd", "input_grad", "filter_grad"]
    assert d["value"] > 0 and all(k["ms"] > 0 and k["frac_of_roofline"] > 0 for k in d["kernels"])


def test_second_backward_stream_changes_no_bit():
    """A layer's parameter gradients run on a second stream beside its input gradient; with the switch off
    everything runs in order on one stream.  Same kernels, same operands: the parameters after three steps
    are bit-identical either way (a missing join between the streams would show here as a difference)."""
    from approxtrain_b200 import layers
    from approxtrain_b200.dp import DataParallelSGD
    g = torch.Generator().manual_seed(5)
    x = torch.rand(16, 24, 24, 8, generator=g).cuda()
    y = torch.randint(0, 10, (16,), generator=g).cuda()

    def run(two_streams):
        keep, layers.TWO_STREAM_BACKWARD = layers.TWO_STREAM_BACKWARD, two_streams
        try:
            torch.manual_seed(1)
            net = _ConvStack(lut_path("MBM_7")).cuda()
            tr = DataParallelSGD(net, lr=0.05)
            for _ in range(3):
                tr.step(lambda: torch.nn.functional.cross_entropy(net(x), y))
            torch.cuda.synchronize()
            return [p.detach().cpu() for p in net.parameters()]
        finally:
            layers.TWO_STREAM_BACKWARD = keep

    for a, b in zip(run(True), run(False)):
        assert torch.equal(a, b)
