"""Network-level parity: every AM op call of one train step of each benchmark network, with the
operands the running network produced, against the CPU oracle.

The op functions (`ops.convam`, `convam_bias_act`, `convam_input_grad`, `convam_filter_grad`,
`denseam`, `denseam_bias_act`, `denseam_grad`, `matmulam`, `bias_grad`) are wrapped for the
duration of one forward + backward + update; each call's arguments and result are kept, and every
call is then recomputed by the oracle from the same arguments:

* deterministic mode: every result bit-identical to the reference-order result;
* fast mode: every result within rel-L2 <= 1e-5 of it.

So the wiring (which tensor goes where, strides, paddings, transposes, the score scale, operand
roles in the gradients) is checked at every layer of LeNet-300-100 (batch 256), LeNet-5 (batch
128), ResNet-50 (batch 2 of 224x224x3: all 53 convolutions and the FC, forward and both
gradients) and the Transformer (6 + 6 layers, 2 x 128 tokens), not only op by op.
"""
import numpy as np
import pytest

from conftest import lut_path, rel_l2

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

OPS = ("convam", "convam_bias_act", "convam_input_grad", "convam_filter_grad", "denseam", "denseam_bias_act",
       "denseam_grad", "matmulam", "bias_grad")


class Recorder:
    def __init__(self, ops_mod):
        self.ops, self.calls, self._orig = ops_mod, [], {}

    def __enter__(self):
        for name in OPS:
            orig = getattr(self.ops, name)
            self._orig[name] = orig

            def wrapped(*a, __orig=orig, __name=name, **k):
                out = __orig(*a, **k)
                # a layer may have launched part of the op on its second stream (the weight gradient of
                # denseam_grad) and joins after the call returns: wait for the whole device before copying
                torch.cuda.synchronize()
                keep = lambda v: v.detach().cpu().numpy().copy() if isinstance(v, torch.Tensor) else v
                outs = tuple(keep(o) for o in out) if isinstance(out, tuple) else keep(out)
                self.calls.append((__name, tuple(keep(v) for v in a), {kk: keep(v) for kk, v in k.items() if kk not in ("out", "out_weights")}, outs))
                return out
            setattr(self.ops, name, wrapped)
        return self

    def __exit__(self, *exc):
        for name, orig in self._orig.items():
            setattr(self.ops, name, orig)


def _stride(k):
    st = k.get("strides") or [1, 1, 1, 1]
    return (st[1], st[2]) if len(st) == 4 else (st[0], st[-1])


def _oracle_result(o, luts_by_path, name, a, k):
    """The reference-order result of one recorded call (numpy)."""
    lut, m = luts_by_path[k["mant_mul_lut"]] if "mant_mul_lut" in k else (None, None)
    if name in ("convam", "convam_bias_act"):
        x, w = a[0], a[1]
        sh, sw = _stride(k)
        g = o.geometry(x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[0], w.shape[1], w.shape[3], sh, sw, k.get("padding", "VALID"))
        y = o.conv2d_fwd(g, x, w, lut, m)
        if name == "convam_bias_act":
            if k.get("scale") is not None:
                y = y * k["scale"]
            if a[2] is not None:
                y = y + a[2]
            if k.get("activation") == "relu":
                y = np.where(y < 0, np.float32(0), y)   # as the epilogue does it: only values below zero are replaced
        return y.astype(np.float32)
    if name == "convam_input_grad":
        sizes, w, dy = a
        sh, sw = _stride(k)
        g = o.geometry(sizes[0], sizes[1], sizes[2], sizes[3], w.shape[0], w.shape[1], w.shape[3], sh, sw, k.get("padding", "VALID"))
        return o.conv2d_bwd_input(g, w, dy, lut, m)
    if name == "convam_filter_grad":
        sizes, x, dy = a
        sh, sw = _stride(k)
        g = o.geometry(x.shape[0], x.shape[1], x.shape[2], x.shape[3], sizes[0], sizes[1], sizes[3], sh, sw, k.get("padding", "VALID"))
        return o.conv2d_bwd_filter(g, x, dy, lut, m)
    if name in ("denseam", "denseam_bias_act"):
        x, w = a[0], a[1]
        if name == "denseam":
            lut, m = luts_by_path[a[2] if len(a) > 2 else k["mant_mul_lut"]]
            return o.dense_fwd(x, w, lut, m)
        y = o.dense_fwd(x, w, lut, m)
        if a[2] is not None:
            y = y + a[2]
        if k.get("activation") == "relu":
            y = np.where(y < 0, np.float32(0), y)
        return y.astype(np.float32)
    if name == "denseam_grad":
        gy, x, w = a[0], a[1], a[2]
        lut, m = luts_by_path[a[3] if len(a) > 3 else k["mant_mul_lut"]]
        return (o.dense_bwd_input(w, gy, lut, m), o.dense_bwd_weight(x, gy, lut, m))
    if name == "matmulam":
        A, B = a[0], a[1]
        lead = A.shape[:-2]
        A3, B3 = A.reshape(-1, *A.shape[-2:]), B.reshape(-1, *B.shape[-2:])
        if k.get("transpose_a"):
            A3 = np.ascontiguousarray(A3.transpose(0, 2, 1))
        if k.get("transpose_b"):
            B3 = np.ascontiguousarray(B3.transpose(0, 2, 1))
        c = o.matmul(A3, B3, lut, m)
        if k.get("alpha") is not None:
            c = (c * np.float32(k["alpha"])).astype(np.float32)
        return c.reshape(*lead, *c.shape[-2:])
    raise KeyError(name)


def _build(which, lp, det):
    from approxtrain_b200 import nets
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(7)
    ce = torch.nn.functional.cross_entropy
    if which == "lenet300100":
        net = nets.LeNet300100(lp, deterministic=det).cuda()
        x, y = torch.rand(256, 28, 28, 1, generator=g).cuda(), torch.randint(0, 10, (256,), generator=g).cuda()
        return net, lambda: ce(net(x), y)
    if which == "lenet5":
        net = nets.LeNet5(lp, deterministic=det).cuda()
        x, y = torch.rand(128, 28, 28, 1, generator=g).cuda(), torch.randint(0, 10, (128,), generator=g).cuda()
        return net, lambda: ce(net(x), y)
    if which == "resnet50":
        net = nets.ResNet50AM(lp, deterministic=det).cuda()
        x, y = torch.randn(2, 224, 224, 3, generator=g).cuda(), torch.randint(0, 1000, (2,), generator=g).cuda()
        return net, lambda: ce(net(x), y)
    net = nets.TransformerAM(lp, deterministic=det).cuda()
    src = torch.randint(1, 8000, (2, 128), generator=g).cuda()
    tgt = torch.randint(1, 8000, (2, 129), generator=g).cuda()

    def loss():
        logits = net(src, tgt[:, :-1])
        return ce(logits.reshape(-1, logits.shape[-1]), tgt[:, 1:].reshape(-1))
    return net, loss


@pytest.mark.parametrize("det", [True, False], ids=["deterministic", "fast"])
@pytest.mark.parametrize("which,lut_name", [("lenet300100", "MBM_7"), ("lenet5", "MIT_7"), ("resnet50", "MBM_7"),
                                            ("transformer", "MIT_7")])
def test_every_am_op_call_of_a_train_step_matches_the_oracle(oracle, luts, which, lut_name, det):
    from approxtrain_b200 import ops
    from approxtrain_b200.dp import DataParallelSGD
    lp = lut_path(lut_name)
    net, loss_fn = _build(which, lp, det)
    tr = DataParallelSGD(net, lr=0.01)
    with Recorder(ops) as rec:
        loss = float(tr.step(loss_fn))
    assert np.isfinite(loss)
    luts_by_path = {lut_path(n): v for n, v in luts.items()}
    seen, worst = {}, 0.0
    for name, a, k, out in rec.calls:
        if name == "bias_grad":
            want = a[0].astype(np.float64).reshape(-1, a[0].shape[-1]).sum(0)
            scale = np.abs(a[0]).astype(np.float64).reshape(-1, a[0].shape[-1]).sum(0).clip(1e-30)
            assert (np.abs(out - want) / scale).max() <= 1e-6
            seen[name] = seen.get(name, 0) + 1
            continue
        want = _oracle_result(oracle, luts_by_path, name, a, k)
        pairs = zip(out, want) if isinstance(out, tuple) else [(out, want)]
        for got, ref in pairs:
            assert got.shape == ref.shape, (name, got.shape, ref.shape)
            if det:
                same = np.array_equal(got.view(np.uint32), ref.view(np.uint32))
                assert same, f"{which}: {name} call {seen.get(name, 0)} {[getattr(v, 'shape', v) for v in a]} is not bit-identical"
            else:
                r = rel_l2(got, ref)
                worst = max(worst, r)
                assert r <= 1e-5, f"{which}: {name} call {seen.get(name, 0)} {[getattr(v, 'shape', v) for v in a]} rel-L2 {r:.3e}"
        seen[name] = seen.get(name, 0) + 1
    print(f"{which} ({lut_name}, {'deterministic' if det else 'fast'}): calls checked {seen}"
          + ("" if det else f"; worst rel-L2 {worst:.3e}"))
    expect = {"lenet300100": 3, "lenet5": 5, "resnet50": 54, "transformer": 97}[which]
    fwd_calls = sum(seen.get(n, 0) for n in ("convam", "convam_bias_act", "denseam", "denseam_bias_act"))
    assert fwd_calls == expect, (fwd_calls, expect)
