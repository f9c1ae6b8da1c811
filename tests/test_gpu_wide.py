"""GPU parity of the wide-tile filter / weight gradient kernel (wide_fgrad: 16 x 8 or 16 x 9
register tiles, 256- or 288-row CTA tiles, cp.async staging).

By default it only takes launches large enough to fill the device a few times over (the
full-size tests reach it that way); here the switch AMSIM_WIDE=1 sends every eligible
fast-mode filter / weight gradient through it, so ragged tiles, padding edges, strides,
1x1 GEMM routing with swapped operand roles and both table kinds are compared with the CPU
oracle at sizes it finishes in a moment.  Bar: rel-L2 <= 1e-5 against the reference-order
result.
"""
import zlib

import numpy as np
import pytest

from conftest import lut_path, rel_l2, set_switch

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-5


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from approxtrain_b200 import ops as o
    return o


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(got, want, what):
    r = rel_l2(got, want)
    print(f"{what}: rel-L2 {r:.3e} max-abs {np.abs(np.asarray(got) - np.asarray(want)).max():.3e}")
    assert np.asarray(got).shape == np.asarray(want).shape
    assert r <= REL_L2_TOL, f"{what}: rel-L2 {r}"


def launches():
    from approxtrain_b200 import _lib
    return _lib.lib.amsim_debug_launch_count()


# (n, h, w, c, kh, kw, k, stride, padding): channel counts are multiples of 4 (128-bit gathers), which is
# what the wide kernel takes
WIDE_CONV = [
    (2, 9, 8, 8, 3, 3, 48, 1, "SAME"),       # one ragged 256-row tile, 144 of them valid
    (3, 17, 19, 12, 3, 2, 70, 1, "VALID"),   # several row tiles, ragged columns, asymmetric filter
    (2, 13, 13, 16, 3, 3, 64, 2, "SAME"),    # stride 2: input gradient runs one sub-convolution per phase
    (1, 20, 20, 32, 1, 1, 96, 1, "VALID"),   # 1x1: plain GEMM routing
    (2, 11, 11, 64, 1, 1, 256, 2, "VALID"),  # strided 1x1 projection
    (4, 10, 10, 32, 3, 3, 40, 1, "SAME"),    # filter gradient: 288 rows = one 9-rows-per-lane tile
    (2, 6, 6, 8, 5, 5, 36, 1, "SAME"),       # 5x5
]


@pytest.mark.parametrize("lname", ["MBM_7", "MIT_7", "MBM_5"])
@pytest.mark.parametrize("case", WIDE_CONV)
def test_wide_conv_all_directions(ops, oracle, luts, monkeypatch, case, lname):
    n, h, w, c, kh, kw, k, s, pad = case
    set_switch(monkeypatch, "AMSIM_WIDE", "1")
    lut, m = luts[lname]
    rng = np.random.default_rng(zlib.crc32(repr((case, lname)).encode()))
    x = rng.standard_normal((n, h, w, c)).astype(np.float32)
    x[x < -0.8] = 0.0                      # zeros as after a ReLU
    wt = rng.standard_normal((kh, kw, c, k)).astype(np.float32)
    g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
    dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
    dy[dy < -1.0] = 0.0
    kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=lut_path(lname))
    close(ops.convam(dev(x), dev(wt), **kw_).cpu().numpy(), oracle.conv2d_fwd(g, x, wt, lut, m), "wide fwd")
    close(ops.convam_input_grad(x.shape, dev(wt), dev(dy), **kw_).cpu().numpy(), oracle.conv2d_bwd_input(g, wt, dy, lut, m),
          "wide input-grad")
    close(ops.convam_filter_grad(wt.shape, dev(x), dev(dy), **kw_).cpu().numpy(), oracle.conv2d_bwd_filter(g, x, dy, lut, m),
          "wide filter-grad")


def test_wide_kernels_are_the_ones_that_ran(ops, oracle, luts, monkeypatch):
    """AMSIM_WIDE=0 and =1 give the same numbers within the bar through different kernels: the
    filter gradient's split count differs (2 vs 3 resident CTAs per multiprocessor), so the two
    results are close but not identical; with the switch off and on again the result repeats."""
    lut, m = luts["MBM_7"]
    rng = np.random.default_rng(8)
    x = rng.standard_normal((16, 40, 40, 32)).astype(np.float32)   # 25 600 pixels: room for 148 and for 296 splits
    dy = rng.standard_normal((16, 40, 40, 64)).astype(np.float32)
    kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=lut_path("MBM_7"))
    g = oracle.geometry(16, 40, 40, 32, 3, 3, 64, 1, 1, "SAME")
    want = oracle.conv2d_bwd_filter(g, x, dy, lut, m)
    out = {}
    for sw in ("0", "1", "0", "1"):
        set_switch(monkeypatch, "AMSIM_WIDE", sw)
        got = ops.convam_filter_grad((3, 3, 32, 64), dev(x), dev(dy), **kw_).cpu().numpy()
        close(got, want, f"filter-grad AMSIM_WIDE={sw}")
        if sw in out:
            assert np.array_equal(out[sw], got), "same switch, same kernel, same bits"
        out[sw] = got
    assert not np.array_equal(out["0"], out["1"]), "both settings ran the same kernel"


def test_wide_dense_weight_gradient(ops, oracle, luts, monkeypatch):
    set_switch(monkeypatch, "AMSIM_WIDE", "1")
    lut, m = luts["MBM_7"]
    lp = lut_path("MBM_7")
    rng = np.random.default_rng(12)
    for b, kin, u in ((300, 64, 72), (513, 128, 260), (40, 512, 1000)):
        x = rng.random((b, kin)).astype(np.float32)
        x[x < 0.3] = 0
        w = (rng.standard_normal((kin, u)) * 0.1).astype(np.float32)
        gy = (rng.standard_normal((b, u)) * 0.01).astype(np.float32)
        close(ops.denseam(dev(x), dev(w), lp).cpu().numpy(), oracle.dense_fwd(x, w, lut, m), f"wide dense fwd {b}x{kin}x{u}")
        dx, dw = ops.denseam_grad(dev(gy), dev(x), dev(w), lp)
        close(dx.cpu().numpy(), oracle.dense_bwd_input(w, gy, lut, m), "wide dense input-grad")
        close(dw.cpu().numpy(), oracle.dense_bwd_weight(x, gy, lut, m), "wide dense weight-grad")


# (n, h, w, c, kh, kw, k, stride, padding): channel counts that are NO multiple of 4 take the 160-row tile
# with element-wise staging (by default only for long reductions such as a 7x7x3 first layer)
TALL5_CONV = [
    (2, 30, 30, 3, 7, 7, 64, 2, "VALID"),    # the first layer of a ResNet: 147 rows in one 160-row tile
    (2, 12, 11, 6, 5, 5, 16, 1, "VALID"),    # LeNet-5's second convolution: 150 rows, 16 columns
    (3, 9, 9, 5, 3, 3, 70, 1, "SAME"),       # 45 rows of one tile, padding taps, ragged columns
    (1, 14, 14, 30, 3, 3, 33, 2, "SAME"),    # 270 rows: two tiles, the second ragged; stride 2
    (2, 10, 10, 1, 5, 5, 6, 1, "SAME"),      # one input channel
]


@pytest.mark.parametrize("lname", ["MBM_7", "MIT_7"])
@pytest.mark.parametrize("case", TALL5_CONV)
def test_filter_gradient_on_the_160_row_tile(ops, oracle, luts, monkeypatch, case, lname):
    n, h, w, c, kh, kw, k, s, pad = case
    lut, m = luts[lname]
    rng = np.random.default_rng(zlib.crc32(repr((case, lname)).encode()))
    x = rng.standard_normal((n, h, w, c)).astype(np.float32)
    x[x < -0.8] = 0.0
    g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
    dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
    dy[dy < -1.0] = 0.0
    want = oracle.conv2d_bwd_filter(g, x, dy, lut, m)
    kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=lut_path(lname))
    got = {}
    for sw in ("0", "1"):
        set_switch(monkeypatch, "AMSIM_WIDE", sw)
        got[sw] = ops.convam_filter_grad((kh, kw, c, k), dev(x), dev(dy), **kw_).cpu().numpy()
        close(got[sw], want, f"filter-grad AMSIM_WIDE={sw}")
    # an input tensor that is not 16-byte aligned takes the same tile (4-byte copies need no more)
    xo = torch.empty(x.size + 1, dtype=torch.float32, device="cuda")[1:].view(x.shape)
    xo.copy_(dev(x))
    close(ops.convam_filter_grad((kh, kw, c, k), xo, dev(dy), **kw_).cpu().numpy(), want, "filter-grad, unaligned input")
