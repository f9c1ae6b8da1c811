"""Full-size parity: the shapes the benchmark times, in the mode it times them,
against the CPU oracle's reference-order result.

The small-shape tests cover every index-map and launch variant; these cover what
only size can show: a filter gradient whose reduction runs over 200 704 (shape A)
or 401 408 (ResNet-50 stem) pixels, where a split sum and the reference's single
FP32 chain (cuda/gemm.cu:30-53 of the reference) differ by accumulated rounding.

Bars, as everywhere: AMSIM_DETERMINISTIC bit-exact; AMSIM_FAST rel-L2 <= 1e-5
against the reference-order result, max-abs printed.  Every case also appends a
line to the JSON-lines file named by the environment variable
AMSIM_PARITY_REPORT (when set), so a run can keep its measured figures.
"""
import json
import os

import numpy as np
import pytest

from conftest import lut_path, rel_l2

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-5

# name: (batch, in_h, in_w, in_c, f, out_c, stride, padding, seed)
CONV_CASES = {
    # AMConv2D microbenchmark shapes (3x3 stride 1 SAME)
    "A": (64, 56, 56, 64, 3, 64, 1, "SAME", 11),
    "B": (64, 14, 14, 256, 3, 256, 1, "SAME", 12),
    # ResNet-50 stem on the zero-padded 230x230 image, batch 32: filter-gradient reduction over 401 408 pixels
    "stem": (32, 230, 230, 3, 7, 64, 2, "VALID", 13),
    # first stride-2 1x1 projection of ResNet-50 (stage 3 entry), batch 32
    "proj": (32, 55, 55, 256, 1, 512, 2, "VALID", 14),
}


def _report(rec):
    path = os.environ.get("AMSIM_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(rec) + "\n")


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _check(got, want, what, deterministic, rec):
    got = np.asarray(got)
    r = rel_l2(got, want)
    mx = float(np.abs(got.astype(np.float64) - want).max())
    same = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
    print(f"{what}: rel-L2 {r:.3e} max-abs {mx:.3e} bit-identical {same}")
    _report(dict(rec, rel_l2=r, max_abs=mx, bit_identical=same, rms_ref=float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))))
    if deterministic:
        assert same, f"{what}: deterministic result is not bit-identical (rel-L2 {r:.3e})"
    else:
        assert r <= REL_L2_TOL, f"{what}: rel-L2 {r:.3e} above {REL_L2_TOL}"


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from approxtrain_b200 import ops as o
    return o


def _conv_inputs(case):
    n, h, w, c, f, k, s, pad, seed = CONV_CASES[case]
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, h, w, c), dtype=np.float32)
    wt = rng.standard_normal((f, f, c, k), dtype=np.float32)
    return x, wt, rng


# the microbenchmark shapes with a table LUT and an additive one; the ResNet-50 shapes with the network's LUT
CONV_PARAMS = [("A", "MBM_7"), ("A", "MIT_7"), ("B", "MBM_7"), ("B", "MIT_7"), ("stem", "MBM_7"), ("proj", "MBM_7")]


@pytest.mark.parametrize("case,lut_name", CONV_PARAMS)
def test_conv_full_size_all_directions(ops, oracle, luts, case, lut_name):
    """forward, input gradient and filter gradient at the benchmark's sizes, both modes."""
    n, h, w, c, f, k, s, pad, _ = CONV_CASES[case]
    lut, m = luts[lut_name]
    x, wt, rng = _conv_inputs(case)
    g = oracle.geometry(n, h, w, c, f, f, k, s, s, pad)
    dy = rng.standard_normal((n, g.out_h, g.out_w, k), dtype=np.float32)
    kw = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=lut_path(lut_name))
    dx_, dw_, ddy = _dev(x), _dev(wt), _dev(dy)
    directions = [
        ("fwd", lambda: oracle.conv2d_fwd(g, x, wt, lut, m), lambda det: ops.convam(dx_, dw_, deterministic=det, **kw)),
        ("filter_grad", lambda: oracle.conv2d_bwd_filter(g, x, dy, lut, m),
         lambda det: ops.convam_filter_grad(wt.shape, dx_, ddy, deterministic=det, **kw)),
    ]
    if case != "stem":  # the image needs no gradient; the stem's input gradient is covered at small size
        directions.append(("input_grad", lambda: oracle.conv2d_bwd_input(g, wt, dy, lut, m),
                           lambda det: ops.convam_input_grad(x.shape, dw_, ddy, deterministic=det, **kw)))
    for name, ref_fn, gpu_fn in directions:
        want = ref_fn()
        for det in (False, True):
            got = gpu_fn(det).cpu().numpy()
            _check(got, want, f"{case} {name} {lut_name} {'deterministic' if det else 'fast'}", det,
                   dict(case=case, op=name, lut=lut_name, mode="deterministic" if det else "fast"))


@pytest.mark.parametrize("which", ["scores", "context"])
def test_attention_matmuls_full_size(ops, oracle, luts, which):
    """The two batched products of one attention layer of the Transformer configuration:
    512 x (128x64 . 64x128) with K read transposed and the 1/sqrt(d_k) factor, and
    512 x (128x128 . 128x64) on softmax rows (MIT_7)."""
    lut, m = luts["MIT_7"]
    rng = np.random.default_rng(31 if which == "scores" else 32)
    lp = lut_path("MIT_7")
    if which == "scores":
        q = rng.standard_normal((512, 128, 64), dtype=np.float32)
        kk = rng.standard_normal((512, 128, 64), dtype=np.float32)
        alpha = np.float32(1.0) / np.sqrt(np.float32(512.0))
        want = oracle.matmul(q, np.ascontiguousarray(kk.transpose(0, 2, 1)), lut, m)
        want = (want * alpha).astype(np.float32)
        run = lambda det: ops.matmulam(_dev(q), _dev(kk), transpose_b=True, mant_mul_lut=lp, deterministic=det,
                                       alpha=float(alpha))
    else:
        p = rng.standard_normal((512, 128, 128), dtype=np.float32)
        p = np.exp(p - p.max(-1, keepdims=True))
        p = (p / p.sum(-1, keepdims=True)).astype(np.float32)
        v = rng.standard_normal((512, 128, 64), dtype=np.float32)
        want = oracle.matmul(p, v, lut, m)
        run = lambda det: ops.matmulam(_dev(p), _dev(v), mant_mul_lut=lp, deterministic=det)
    for det in (False, True):
        got = run(det).cpu().numpy()
        _check(got, want, f"attention {which} MIT_7 {'deterministic' if det else 'fast'}", det,
               dict(case="attention_" + which, op="matmul", lut="MIT_7", mode="deterministic" if det else "fast"))


def test_dense_head_full_size(ops, oracle, luts):
    """ResNet-50's final AM dense layer at batch 32 (2048 -> 1000) and the Transformer's
    vocabulary projection on all 8192 tokens of a step (512 -> the first 2000 of its 8000
    columns: columns are independent, the reduction lengths are the full ones): forward and
    both gradients."""
    for tag, lut_name, b, kin, u, seed in (("fc", "MBM_7", 32, 2048, 1000, 41), ("vocab", "MIT_7", 8192, 512, 2000, 42)):
        lut, m = luts[lut_name]
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((b, kin), dtype=np.float32)
        w = (rng.standard_normal((kin, u), dtype=np.float32) * np.float32(0.05))
        gy = rng.standard_normal((b, u), dtype=np.float32)
        lp = lut_path(lut_name)
        want_y = oracle.dense_fwd(x, w, lut, m)
        want_dx, want_dw = oracle.dense_bwd_input(w, gy, lut, m), oracle.dense_bwd_weight(x, gy, lut, m)
        for det in (False, True):
            mode = "deterministic" if det else "fast"
            y = ops.denseam(_dev(x), _dev(w), lp, deterministic=det).cpu().numpy()
            dx, dw = ops.denseam_grad(_dev(gy), _dev(x), _dev(w), lp, deterministic=det)
            _check(y, want_y, f"dense {tag} fwd {mode}", det, dict(case="dense_" + tag, op="fwd", lut=lut_name, mode=mode))
            _check(dx.cpu().numpy(), want_dx, f"dense {tag} input_grad {mode}", det,
                   dict(case="dense_" + tag, op="input_grad", lut=lut_name, mode=mode))
            _check(dw.cpu().numpy(), want_dw, f"dense {tag} weight_grad {mode}", det,
                   dict(case="dense_" + tag, op="weight_grad", lut=lut_name, mode=mode))
