"""GPU parity tests: the CUDA path, called through the C ABI (ctypes ->
libamsim.so), against the CPU oracle on the same seeded inputs.

Bars: the elementwise primitive and every AMSIM_DETERMINISTIC result are
bit-exact; AMSIM_FAST results are within rel-L2 <= 1e-5 of the oracle's
reference-order result (max-abs is printed)."""
import os

import numpy as np
import pytest

from conftest import BIG_LUT, GOLDEN, SMALL_LUTS, lut_path, rel_l2, set_switch

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


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def assert_bit_equal(got, want, what):
    got, want = np.asarray(got), np.asarray(want)
    bad = bits(got) != bits(want)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} differ, first {np.argwhere(bad)[0]}: " \
                          f"{got[bad][0]!r} vs {want[bad][0]!r}"


def assert_close(got, want, what):
    r = rel_l2(got, want)
    print(f"{what}: rel-L2 {r:.3e} max-abs {np.abs(np.asarray(got) - np.asarray(want)).max():.3e}")
    assert r <= REL_L2_TOL, f"{what}: rel-L2 {r}"


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", SMALL_LUTS)
def test_primitive_exhaustive(ops, oracle, luts, name):
    """all 2^(2m) mantissa pairs x exponent classes x signs, device vs oracle."""
    lut, m = luts[name]
    n = 1 << m
    ia, ib = np.meshgrid(np.arange(n, dtype=np.uint32), np.arange(n, dtype=np.uint32), indexing="ij")
    rng = np.random.default_rng(21)
    low = rng.integers(0, 1 << (23 - m), size=ia.shape, dtype=np.uint32)
    classes = [0, 1, 64, 126, 127, 128, 129, 200, 254, 255]
    ats, bts = [], []
    for ea in classes:
        for eb in classes:
            for sa, sb in ((0, 0), (1, 0), (1, 1)):
                ats.append(((np.uint32(sa) << 31) | (np.uint32(ea) << 23) | (ia << (23 - m)) | low).ravel())
                bts.append(((np.uint32(sb) << 31) | (np.uint32(eb) << 23) | (ib << (23 - m)) | (low ^ 1)).ravel())
    at, bt = np.concatenate(ats), np.concatenate(bts)
    got = ops.am_multiply(dev(at.view(np.float32)), dev(bt.view(np.float32)), lut_path(name)).cpu().numpy()
    want = oracle.mul(at.view(np.float32), bt.view(np.float32), lut, m)
    assert_bit_equal(got, want, f"AM primitive {name}")


def test_primitive_known_answers_from_reference(ops):
    kat = np.load(os.path.join(GOLDEN, "prim_kat.npz"))
    for name in SMALL_LUTS:
        got = ops.am_multiply(dev(kat["at"].view(np.float32)), dev(kat["bt"].view(np.float32)), lut_path(name))
        assert np.array_equal(got.cpu().numpy().view(np.uint32), kat["out_" + name]), name


def test_primitive_m11(ops, oracle):
    if not os.path.exists(BIG_LUT):
        pytest.skip("oracle/_ref/lut/MBM_11.bin not built")
    from oracle.oracle import load_lut
    lut, m = load_lut(BIG_LUT)
    rng = np.random.default_rng(5)
    a = rng.standard_normal(1 << 20).astype(np.float32)
    b = rng.standard_normal(1 << 20).astype(np.float32)
    a[::7] = 0
    got = ops.am_multiply(dev(a), dev(b), BIG_LUT).cpu().numpy()
    assert_bit_equal(got, oracle.mul(a, b, lut, m), "AM primitive m=11")


# ---------------------------------------------------------------------------------------
def _conv_case(rng, n, h, w, c, kh, kw, k, zeros=True, ints=False):
    if ints:
        x = rng.integers(-2, 2, size=(n, h, w, c)).astype(np.float32)
        wt = rng.integers(-2, 2, size=(kh, kw, c, k)).astype(np.float32)
    else:
        x = rng.standard_normal((n, h, w, c)).astype(np.float32)
        wt = rng.standard_normal((kh, kw, c, k)).astype(np.float32)
        if zeros:
            x[x < -0.4] = 0.0  # ReLU-like zeros
    return x, wt


# (n, h, w, c, kh, kw, k): vector path (c % 4 == 0) and scalar path, ragged tiles, 1x1, full-size filter
CONV_SHAPES = [
    (2, 9, 8, 8, 3, 3, 16),
    (1, 12, 12, 4, 3, 3, 70),      # K_out not a multiple of 64
    (2, 7, 7, 3, 3, 3, 5),         # c % 4 != 0 (scalar gather)
    (3, 10, 11, 1, 5, 5, 6),       # LeNet conv1-like
    (2, 6, 6, 6, 5, 5, 16),        # LeNet conv2-like
    (1, 8, 8, 16, 1, 1, 32),       # 1x1
    (2, 5, 5, 8, 5, 5, 8),         # filter as large as the input
    (5, 17, 19, 12, 3, 2, 24),     # > 1 pixel tile
]


@pytest.mark.parametrize("shape", CONV_SHAPES)
@pytest.mark.parametrize("stride", [1, 2])
@pytest.mark.parametrize("padding", ["SAME", "VALID"])
def test_conv_all_directions(ops, oracle, luts, shape, stride, padding):
    n, h, w, c, kh, kw, k = shape
    if padding == "VALID" and (kh > h or kw > w):
        pytest.skip("filter larger than input")
    lname = "MBM_7" if (n + h) % 2 else "MIT_5"
    lut, m = luts[lname]
    rng = np.random.default_rng(hash((shape, stride, padding)) % (2**32))
    x, wt = _conv_case(rng, n, h, w, c, kh, kw, k)
    g = oracle.geometry(n, h, w, c, kh, kw, k, stride, stride, padding)
    dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
    dy[dy < -1.0] = 0.0
    y_ref = oracle.conv2d_fwd(g, x, wt, lut, m)
    dw_ref = oracle.conv2d_bwd_filter(g, x, dy, lut, m)
    dx_ref = oracle.conv2d_bwd_input(g, wt, dy, lut, m)
    st = [1, stride, stride, 1]
    kw_ = dict(strides=st, padding=padding, mant_mul_lut=lut_path(lname))
    for det in (True, False):
        y = ops.convam(dev(x), dev(wt), deterministic=det, **kw_).cpu().numpy()
        dw = ops.convam_filter_grad(wt.shape, dev(x), dev(dy), deterministic=det, **kw_).cpu().numpy()
        dx = ops.convam_input_grad(x.shape, dev(wt), dev(dy), deterministic=det, **kw_).cpu().numpy()
        assert y.shape == y_ref.shape and dw.shape == dw_ref.shape and dx.shape == dx_ref.shape
        if det:
            assert_bit_equal(y, y_ref, "conv fwd (deterministic)")
            assert_bit_equal(dw, dw_ref, "conv filter-grad (deterministic)")
            assert_bit_equal(dx, dx_ref, "conv input-grad (deterministic)")
        else:
            assert_close(y, y_ref, "conv fwd (fast)")
            assert_close(dw, dw_ref, "conv filter-grad (fast)")
            assert_close(dx, dx_ref, "conv input-grad (fast)")


@pytest.mark.parametrize("name", SMALL_LUTS)
def test_conv_every_lut(ops, oracle, luts, name):
    lut, m = luts[name]
    rng = np.random.default_rng(99)
    x, wt = _conv_case(rng, 2, 10, 9, 8, 3, 3, 12)
    g = oracle.geometry(2, 10, 9, 8, 3, 3, 12, 1, 1, "SAME")
    dy = rng.standard_normal((2, g.out_h, g.out_w, 12)).astype(np.float32)
    kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=lut_path(name))
    for det in (True, False):
        chk = assert_bit_equal if det else assert_close
        chk(ops.convam(dev(x), dev(wt), deterministic=det, **kw_).cpu().numpy(), oracle.conv2d_fwd(g, x, wt, lut, m), f"fwd {name}")
        chk(ops.convam_filter_grad(wt.shape, dev(x), dev(dy), deterministic=det, **kw_).cpu().numpy(),
            oracle.conv2d_bwd_filter(g, x, dy, lut, m), f"fgrad {name}")
        chk(ops.convam_input_grad(x.shape, dev(wt), dev(dy), deterministic=det, **kw_).cpu().numpy(),
            oracle.conv2d_bwd_input(g, wt, dy, lut, m), f"igrad {name}")


def test_fast_forward_is_bit_exact_without_zero_operands(ops, oracle, luts, monkeypatch):
    """With no zero/denormal operand and no underflowing product the fast path
    computes the reference products exactly and, where one warp of one CTA owns an
    output's whole reduction (more than 32 output columns, plain grid), sums them in
    the reference order: VALID padding, N(0,1) data."""
    set_switch(monkeypatch, "AMSIM_BALANCED", "0")
    set_switch(monkeypatch, "AMSIM_FORCE_KSPLIT", "1")
    lut, m = luts["MBM_7"]
    rng = np.random.default_rng(17)
    x = rng.standard_normal((2, 12, 12, 8)).astype(np.float32)
    wt = rng.standard_normal((3, 3, 8, 48)).astype(np.float32)
    g = oracle.geometry(2, 12, 12, 8, 3, 3, 48, 1, 1, "VALID")
    y = ops.convam(dev(x), dev(wt), [1, 1, 1, 1], "VALID", mant_mul_lut=lut_path("MBM_7")).cpu().numpy()
    assert_bit_equal(y, oracle.conv2d_fwd(g, x, wt, lut, m), "fast fwd, no zeros")


def test_conv_reference_test_inputs_small_integers(ops, oracle, luts):
    """Inputs of the reference's own conv test: integers in [-2, 2)
    (test/convam_final_test.py:165-166) with the bf16-exact LUT; compared the
    way that test does (mean error <= 1e-7, :64) against the exact convolution,
    and bit for bit against the oracle in deterministic mode (0 x +-2 quirk)."""
    lut, m = luts["ACC_7"]
    rng = np.random.default_rng(3)
    x, wt = _conv_case(rng, 2, 8, 8, 3, 3, 3, 4, ints=True)
    g = oracle.geometry(2, 8, 8, 3, 3, 3, 4, 1, 1, "SAME")
    kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=lut_path("ACC_7"))
    exact = oracle.cpu_conv2d_fwd(g, x, wt)
    y_det = ops.convam(dev(x), dev(wt), deterministic=True, **kw_).cpu().numpy()
    y_fast = ops.convam(dev(x), dev(wt), **kw_).cpu().numpy()
    assert_bit_equal(y_det, oracle.conv2d_fwd(g, x, wt, lut, m), "ints fwd det")
    assert np.abs(y_det - exact).mean() <= 1e-7
    assert np.array_equal(y_fast, exact)  # the fast path drops the 0 x 2 residue: exactly the integer result


def test_conv_golden_fixture(ops):
    """Known answers committed under tests/golden (needs no oracle build)."""
    kat = np.load(os.path.join(GOLDEN, "ops_kat.npz"))
    for tag, lname in (("convA", "MBM_7"), ("convB", "MIT_5"), ("convC", "MBM_7")):
        n, h, w, c, kh, kw, k, s, same = [int(v) for v in kat[tag + "_geom"]]
        kw_ = dict(strides=[1, s, s, 1], padding="SAME" if same else "VALID", mant_mul_lut=lut_path(lname), deterministic=True)
        assert_bit_equal(ops.convam(dev(kat[tag + "_x"]), dev(kat[tag + "_w"]), **kw_).cpu().numpy(), kat[tag + "_y"], tag)
        assert_bit_equal(ops.convam_filter_grad((kh, kw, c, k), dev(kat[tag + "_x"]), dev(kat[tag + "_dy"]), **kw_).cpu().numpy(), kat[tag + "_dw"], tag)
        assert_bit_equal(ops.convam_input_grad((n, h, w, c), dev(kat[tag + "_w"]), dev(kat[tag + "_dy"]), **kw_).cpu().numpy(), kat[tag + "_dx"], tag)
    lut7 = lut_path("MBM_7")
    assert_bit_equal(ops.denseam(dev(kat["dense_x"]), dev(kat["dense_w"]), lut7, deterministic=True).cpu().numpy(), kat["dense_y"], "dense")
    dx, dw = ops.denseam_grad(dev(kat["dense_g"]), dev(kat["dense_x"]), dev(kat["dense_w"]), lut7, deterministic=True)
    assert_bit_equal(dx.cpu().numpy(), kat["dense_dx"], "dense dx")
    assert_bit_equal(dw.cpu().numpy(), kat["dense_dw"], "dense dw")
    assert_bit_equal(ops.matmulam(dev(kat["mm_a"]), dev(kat["mm_b"]), mant_mul_lut=lut7, deterministic=True).cpu().numpy(), kat["mm_c"], "matmul")


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("b,k,u", [(256, 784, 300), (256, 300, 100), (256, 100, 10), (7, 33, 5), (130, 64, 129), (1, 1, 1)])
def test_dense(ops, oracle, luts, b, k, u):
    lut, m = luts["MBM_7"]
    rng = np.random.default_rng(b * 1000 + k)
    x = rng.random((b, k)).astype(np.float32)
    x[x < 0.3] = 0
    w = (rng.standard_normal((k, u)) * 0.1).astype(np.float32)
    g = (rng.standard_normal((b, u)) * 0.01).astype(np.float32)
    p = lut_path("MBM_7")
    for det in (True, False):
        chk = assert_bit_equal if det else assert_close
        chk(ops.denseam(dev(x), dev(w), p, deterministic=det).cpu().numpy(), oracle.dense_fwd(x, w, lut, m), "dense fwd")
        dx, dw = ops.denseam_grad(dev(g), dev(x), dev(w), p, deterministic=det)
        chk(dx.cpu().numpy(), oracle.dense_bwd_input(w, g, lut, m), "dense input-grad")
        chk(dw.cpu().numpy(), oracle.dense_bwd_weight(x, g, lut, m), "dense weight-grad")


def test_dense_input_grad_operand_order(ops, oracle):
    """dx uses AM(w, g) (weight first): checked with a deliberately asymmetric LUT."""
    import tempfile
    rng = np.random.default_rng(8)
    m = 3
    lutb = rng.integers(0, 256, size=1 << (2 * m), dtype=np.uint8)
    lutb = ((lutb & 0x80) | (lutb & ((1 << m) - 1))).astype(np.uint8)  # carry | m mantissa bits, asymmetric
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ASYM_3.bin")
        lutb.tofile(path)
        x = rng.standard_normal((9, 20)).astype(np.float32)
        w = rng.standard_normal((20, 6)).astype(np.float32)
        g = rng.standard_normal((9, 6)).astype(np.float32)
        for det in (True, False):
            chk = assert_bit_equal if det else assert_close
            dx, dw = ops.denseam_grad(dev(g), dev(x), dev(w), path, deterministic=det)
            chk(dx.cpu().numpy(), oracle.dense_bwd_input(w, g, lutb, m), "asym dx")
            chk(dw.cpu().numpy(), oracle.dense_bwd_weight(x, g, lutb, m), "asym dw")
            chk(ops.denseam(dev(x), dev(w), path, deterministic=det).cpu().numpy(), oracle.dense_fwd(x, w, lutb, m), "asym y")


def test_lut_with_wide_mantissa_bytes(ops, oracle):
    """A LUT whose low 7 bits exceed 2^m (lut_gen never writes one, the format
    allows it): the reference adds (v & 0x7f) << (23 - m) as is."""
    import tempfile
    rng = np.random.default_rng(12)
    m = 5
    lutb = rng.integers(0, 256, size=1 << (2 * m), dtype=np.uint8)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "WIDE_5.bin")
        lutb.tofile(path)
        a = rng.standard_normal((6, 40)).astype(np.float32)
        b = rng.standard_normal((40, 8)).astype(np.float32)
        assert_bit_equal(ops.matmulam(dev(a), dev(b), mant_mul_lut=path, deterministic=True).cpu().numpy(),
                         oracle.matmul(a, b, lutb, m), "wide-mantissa LUT")
        assert_close(ops.matmulam(dev(a), dev(b), mant_mul_lut=path).cpu().numpy(), oracle.matmul(a, b, lutb, m), "wide fast")


@pytest.mark.parametrize("sa,sb", [((5, 7), (7, 3)), ((4, 5, 7), (4, 7, 3)), ((4, 5, 7), (7, 3)), ((5, 7), (4, 7, 3)),
                                   ((1, 5, 7), (4, 7, 3)), ((4, 5, 7), (1, 7, 3)), ((16, 128, 64), (16, 64, 128))])
def test_matmul_ranks_and_broadcast(ops, oracle, luts, sa, sb):
    lut, m = luts["MIT_7"]
    rng = np.random.default_rng(len(sa) * 10 + len(sb))
    a = rng.standard_normal(sa).astype(np.float32)
    b = rng.standard_normal(sb).astype(np.float32)
    want = oracle.matmul(a, b, lut, m)
    for det in (True, False):
        got = ops.matmulam(dev(a), dev(b), mant_mul_lut=lut_path("MIT_7"), deterministic=det).cpu().numpy()
        assert got.shape == want.shape
        (assert_bit_equal if det else assert_close)(got, want, f"matmul {sa}x{sb}")


def test_matmul_transpose_flags_and_errors(ops, oracle, luts):
    lut, m = luts["MIT_7"]
    rng = np.random.default_rng(4)
    q = rng.standard_normal((3, 6, 8)).astype(np.float32)
    k = rng.standard_normal((3, 5, 8)).astype(np.float32)
    got = ops.matmulam(dev(q), dev(k), transpose_b=True, mant_mul_lut=lut_path("MIT_7"), deterministic=True).cpu().numpy()
    assert_bit_equal(got, oracle.matmul(q, np.ascontiguousarray(k.transpose(0, 2, 1)), lut, m), "q k^T")
    with pytest.raises(ValueError, match="cols of mat a"):
        ops.matmulam(dev(q), dev(k), mant_mul_lut=lut_path("MIT_7"))
    with pytest.raises(ValueError, match="batch of mat a"):
        ops.matmulam(dev(q), dev(np.zeros((2, 8, 5), np.float32)), mant_mul_lut=lut_path("MIT_7"))
    with pytest.raises(ValueError, match="equal leading axes"):
        ops.matmulam(dev(np.zeros((2, 2, 2, 2), np.float32)), dev(np.zeros((2, 2), np.float32)), mant_mul_lut=lut_path("MIT_7"))
    with pytest.raises(ValueError, match="2 dimensional or 3 dimensional"):
        ops.matmulam(dev(np.zeros((2,), np.float32)), dev(np.zeros((2, 2), np.float32)), mant_mul_lut=lut_path("MIT_7"))


@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
def test_matmul_transposes_in_the_kernel_and_alpha(ops, oracle, luts, ta, tb):
    """transpose_a / transpose_b are index maps in the kernel (the reference materialises
    them in Python, math_ops.py:82-93): deterministic results are bit-identical to the
    oracle on the materialised operands, for batched, broadcast and rank-4 operands; alpha
    is one FP32 multiply of the finished sum."""
    lut, m = luts["MBM_7"]
    p7 = lut_path("MBM_7")
    rng = np.random.default_rng(12)
    for (M, K, N) in ((37, 70, 45), (40, 72, 48)):   # scalar staging; 128-bit staging along q or k
        _check_matmul_transposes(ops, oracle, lut, m, p7, rng, M, K, N, ta, tb)


def _check_matmul_transposes(ops, oracle, lut, m, p7, rng, M, K, N, ta, tb):
    def mk(batch, r, c, t):
        shp = (c, r) if t else (r, c)
        return rng.standard_normal(batch + shp).astype(np.float32)
    def mat(x, t):
        return np.ascontiguousarray(np.swapaxes(x, -1, -2)) if t else x
    for ba, bb in [((), ()), ((4,), (4,)), ((4,), ()), ((1,), (3,)), ((2, 3), (2, 3))]:
        a, b = mk(ba, M, K, ta), mk(bb, K, N, tb)
        want = oracle.matmul(mat(a, ta).reshape((-1, M, K)) if len(ba) == 2 else mat(a, ta),
                             mat(b, tb).reshape((-1, K, N)) if len(bb) == 2 else mat(b, tb), lut, m)
        got = ops.matmulam(dev(a), dev(b), transpose_a=ta, transpose_b=tb, mant_mul_lut=p7, deterministic=True)
        assert_bit_equal(got.cpu().numpy().reshape(want.shape), want, f"det ta={ta} tb={tb} {ba} {bb}")
        fast = ops.matmulam(dev(a), dev(b), transpose_a=ta, transpose_b=tb, mant_mul_lut=p7)
        assert_close(fast.cpu().numpy().reshape(want.shape), want, f"fast ta={ta} tb={tb} {ba} {bb}")
        for det in (True, False):
            base = ops.matmulam(dev(a), dev(b), transpose_a=ta, transpose_b=tb, mant_mul_lut=p7, deterministic=det)
            al = float(np.float32(1.0) / np.float32(np.sqrt(float(K))))
            sc = ops.matmulam(dev(a), dev(b), transpose_a=ta, transpose_b=tb, mant_mul_lut=p7, deterministic=det, alpha=al)
            assert torch.equal(sc, base * al), "alpha is one FP32 multiply"


def test_empty_and_degenerate_inputs(ops):
    p = lut_path("MBM_7")
    y = ops.convam(torch.zeros(0, 5, 5, 4, device="cuda"), torch.zeros(3, 3, 4, 8, device="cuda"), [1, 1, 1, 1], "SAME", mant_mul_lut=p)
    assert tuple(y.shape) == (0, 5, 5, 8)
    dw = ops.convam_filter_grad((3, 3, 4, 8), torch.zeros(0, 5, 5, 4, device="cuda"), torch.zeros(0, 5, 5, 8, device="cuda"),
                                [1, 1, 1, 1], "SAME", mant_mul_lut=p)
    assert float(dw.abs().sum()) == 0.0
    c = ops.matmulam(torch.zeros(3, 0, device="cuda"), torch.zeros(0, 4, device="cuda"), mant_mul_lut=p)
    assert tuple(c.shape) == (3, 4) and float(c.abs().sum()) == 0.0
    assert tuple(ops.denseam(torch.zeros(0, 7, device="cuda"), torch.zeros(7, 3, device="cuda"), p).shape) == (0, 3)


def test_errors_through_the_abi(ops):
    from approxtrain_b200 import _lib
    with pytest.raises(_lib.AmsimError) as e:
        ops.denseam(torch.zeros(2, 2, device="cuda"), torch.zeros(2, 2, device="cuda"), "")
    assert e.value.code == _lib.ERR_LUT_NAME
    with pytest.raises(_lib.AmsimError) as e:
        ops.denseam(torch.zeros(2, 2, device="cuda"), torch.zeros(2, 2, device="cuda"), "/nonexistent/X_7.bin")
    assert e.value.code == _lib.ERR_LUT_IO
    # too-small workspace is refused, nothing is launched
    import ctypes as C
    lut = ops.get_lut(lut_path("MBM_7"), "cuda")
    x = torch.zeros(64, 8, 8, 16, device="cuda"); dy = torch.zeros(64, 8, 8, 16, device="cuda"); dw = torch.zeros(3, 3, 16, 16, device="cuda")
    need = _lib.lib.amsim_conv2d_bwd_filter_workspace(64, 8, 8, 16, 3, 3, 16, 8, 8, 0)
    assert need > 0
    rc = _lib.lib.amsim_conv2d_bwd_filter(None, lut.handle, C.c_void_p(x.data_ptr()), C.c_void_p(dy.data_ptr()), C.c_void_p(dw.data_ptr()),
                                          64, 8, 8, 16, 3, 3, 16, 8, 8, 1, 1, 1, 1, None, 0, 0)
    assert rc == _lib.ERR_WORKSPACE


def test_full_size_properties_config3_shapeB(ops):
    """Conv microbenchmark shape B (N64 14x14 256->256, 3x3 SAME) at full size,
    checked through properties that need no oracle run:
    linearity in the power-of-two scaling of an operand (exact for the AM
    multiplier: only exponents change) and <y,dy> = <dw,w>-style consistency is
    not available for a non-bilinear multiplier, so instead the three
    directions are compared with their deterministic-mode twins."""
    p = lut_path("MBM_7")
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(64, 14, 14, 256, device="cuda", generator=g)
    w = torch.randn(3, 3, 256, 256, device="cuda", generator=g)
    dy = torch.randn(64, 14, 14, 256, device="cuda", generator=g)
    kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=p)
    y = ops.convam(x, w, **kw_)
    y4 = ops.convam(x * 4.0, w, **kw_)
    assert torch.equal(y4, y * 4.0), "scaling an operand by 2^k scales every AM product by 2^k exactly"
    yd = ops.convam(x, w, deterministic=True, **kw_)
    assert rel_l2(y.cpu().numpy(), yd.cpu().numpy()) <= REL_L2_TOL
    dx = ops.convam_input_grad(x.shape, w, dy, **kw_)
    dxd = ops.convam_input_grad(x.shape, w, dy, deterministic=True, **kw_)
    assert rel_l2(dx.cpu().numpy(), dxd.cpu().numpy()) <= REL_L2_TOL
    dw = ops.convam_filter_grad(w.shape, x, dy, **kw_)
    dw2 = ops.convam_filter_grad(w.shape, x, dy, **kw_)
    assert torch.equal(dw, dw2), "split-K partials are summed in a fixed order: run-to-run identical"
    # exact-multiply sanity: the AM result tracks the exact convolution within the multiplier's error
    ref = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2), w.permute(3, 2, 0, 1), padding=1).permute(0, 2, 3, 1)
    assert rel_l2(y.cpu().numpy(), ref.cpu().numpy()) < 0.1


@pytest.mark.parametrize("force", [None, "2", "4", "8"])
def test_cluster_split_of_the_reduction(ops, oracle, luts, force, monkeypatch):
    """Few output tiles and a long reduction: the fast path lets a thread-block
    cluster share each tile's reduction and adds the partial tiles in rank order
    through distributed shared memory.  Deterministic mode never splits."""
    lut, m = luts["MBM_7"]
    rng = np.random.default_rng(31)
    x, wt = _conv_case(rng, 2, 7, 7, 64, 3, 3, 96)          # 98 pixels, 2 channel tiles, K = 576 (36 stages)
    g = oracle.geometry(2, 7, 7, 64, 3, 3, 96, 1, 1, "SAME")
    dy = rng.standard_normal((2, 7, 7, 96)).astype(np.float32)
    set_switch(monkeypatch, "AMSIM_BALANCED", "0")  # outside a graph capture the balanced launch would take this shape
    if force is not None:
        set_switch(monkeypatch, "AMSIM_FORCE_KSPLIT", force)
    kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=lut_path("MBM_7"))
    y = ops.convam(dev(x), dev(wt), **kw_).cpu().numpy()
    dx = ops.convam_input_grad(x.shape, dev(wt), dev(dy), **kw_).cpu().numpy()
    y2 = ops.convam(dev(x), dev(wt), **kw_).cpu().numpy()
    assert_close(y, oracle.conv2d_fwd(g, x, wt, lut, m), f"cluster split fwd ({force})")
    assert_close(dx, oracle.conv2d_bwd_input(g, wt, dy, lut, m), f"cluster split input-grad ({force})")
    assert np.array_equal(y, y2), "rank-ordered combine: run-to-run identical"
    yd = ops.convam(dev(x), dev(wt), deterministic=True, **kw_).cpu().numpy()
    assert_bit_equal(yd, oracle.conv2d_fwd(g, x, wt, lut, m), "deterministic mode ignores the split")


@pytest.mark.parametrize("balanced", [None, "1", "0"])
def test_balanced_launch_of_the_reduction(ops, oracle, luts, balanced, monkeypatch, tmp_path):
    """Fast mode deals the (tile, reduction block) pairs out in equal runs to as many
    CTAs as the device holds; tiles shared between CTAs are combined in CTA order by a
    second pass.  Forced on ("1"), off ("0") and chosen by the library (None): same
    parity bar, run-to-run identical, every epilogue (strided output rows of a
    stride-2 input gradient, bias + ReLU, batched matmul) and every table mode."""
    if balanced is not None:
        set_switch(monkeypatch, "AMSIM_BALANCED", balanced)
    lut, m = luts["MBM_7"]
    p7 = lut_path("MBM_7")
    rng = np.random.default_rng(77)
    cases = [(2, 7, 7, 64, 3, 3, 96, 1, "SAME"),      # 2 tiles, 36 reduction blocks
             (3, 20, 20, 32, 3, 3, 70, 1, "SAME"),    # 10 x 2 tiles, ragged in p and q
             (2, 15, 15, 16, 3, 3, 24, 2, "SAME"),    # stride 2: input gradient by stride phase
             (1, 12, 12, 3, 5, 5, 6, 2, "VALID")]     # scalar gather path
    for (n, h, w, c, kh, kw, k, s, pad) in cases:
        x, wt = _conv_case(rng, n, h, w, c, kh, kw, k)
        g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
        dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
        b = rng.standard_normal(k).astype(np.float32)
        kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=p7)
        y = ops.convam(dev(x), dev(wt), **kw_)
        assert_close(y.cpu().numpy(), oracle.conv2d_fwd(g, x, wt, lut, m), f"balanced fwd {balanced}")
        assert torch.equal(y, ops.convam(dev(x), dev(wt), **kw_)), "run-to-run identical"
        dx = ops.convam_input_grad(x.shape, dev(wt), dev(dy), **kw_).cpu().numpy()
        assert_close(dx, oracle.conv2d_bwd_input(g, wt, dy, lut, m), f"balanced input-grad {balanced}")
        fused = ops.convam_bias_act(dev(x), dev(wt), dev(b), activation="relu", **kw_)
        assert torch.equal(fused, torch.relu(y + dev(b))), "epilogue after the combine"
    a = rng.standard_normal((5, 40, 200)).astype(np.float32)
    bb = rng.standard_normal((5, 200, 70)).astype(np.float32)
    c_ = ops.matmulam(dev(a), dev(bb), mant_mul_lut=p7).cpu().numpy()
    assert_close(c_, oracle.matmul(a, bb, lut, m), f"balanced batched matmul {balanced}")
    # additive table (no lookup) and a table in global memory
    x, wt = _conv_case(rng, 2, 9, 9, 32, 3, 3, 40)
    g = oracle.geometry(2, 9, 9, 32, 3, 3, 40, 1, 1, "SAME")
    lutm, mm = luts["MIT_7"]
    ym = ops.convam(dev(x), dev(wt), strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=lut_path("MIT_7")).cpu().numpy()
    assert_close(ym, oracle.conv2d_fwd(g, x, wt, lutm, mm), f"balanced additive {balanced}")
    lut9 = rng.integers(0, 256, size=1 << 18, dtype=np.uint8)
    path9 = str(tmp_path / "RAND_9.bin")
    lut9.tofile(path9)
    y9 = ops.convam(dev(x), dev(wt), strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=path9).cpu().numpy()
    assert_close(y9, oracle.conv2d_fwd(g, x, wt, lut9, 9), f"balanced global table {balanced}")
    # deterministic mode never splits a reduction
    yd = ops.convam(dev(x), dev(wt), strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=p7, deterministic=True).cpu().numpy()
    assert_bit_equal(yd, oracle.conv2d_fwd(g, x, wt, lut, m), "deterministic mode ignores the balanced launch")


@pytest.mark.parametrize("chain", ["1", "0"])
def test_deterministic_filter_gradient_products_in_parallel_additions_in_order(ops, oracle, luts, chain, monkeypatch, tmp_path):
    """Few chains, long reduction: a stage's products are computed by all warps in parallel
    and each thread then adds its own chain's 16 products in ascending order.  Bit-identical
    to the oracle for every table mode, hazard data included; forced on and off."""
    set_switch(monkeypatch, "AMSIM_CHAIN_FGRAD", chain)
    set_switch(monkeypatch, "AMSIM_THIN_FGRAD", "1")
    rng = np.random.default_rng(404)
    lut9 = rng.integers(0, 256, size=1 << 18, dtype=np.uint8)
    path9 = str(tmp_path / "RAND_9.bin")
    lut9.tofile(path9)
    from oracle.oracle import DIRECT_MBM32, NO_LUT
    tables = [(lut_path("MBM_7"),) + luts["MBM_7"], (lut_path("MIT_7"),) + luts["MIT_7"], (path9, lut9, 9),
              ("direct:MBM32", NO_LUT, DIRECT_MBM32)]
    for (path, lut, m) in tables:
        for (n, h, w, c, kh, kw, k, s, pad) in [(3, 20, 20, 8, 3, 3, 20, 1, "SAME"), (2, 24, 24, 3, 5, 5, 6, 2, "VALID")]:
            x, _ = _conv_case(rng, n, h, w, c, kh, kw, k)
            x.reshape(-1)[rng.choice(x.size, x.size // 50, replace=False)] = rng.choice(
                np.array([2.5, -3.0, 1e-30, 1e25, 0.0, -0.0], np.float32), x.size // 50)
            g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
            dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
            dy.reshape(-1)[rng.choice(dy.size, dy.size // 50, replace=False)] = rng.choice(
                np.array([4.0, -2.0, 1e-28, -1e22, 0.0], np.float32), dy.size // 50)
            dw = ops.convam_filter_grad((kh, kw, c, k), dev(x), dev(dy), strides=[1, s, s, 1], padding=pad,
                                        mant_mul_lut=path, deterministic=True).cpu().numpy()
            with np.errstate(all="ignore"):
                want = oracle.conv2d_bwd_filter(g, x, dy, lut, m)
            nan = np.isnan(want)
            assert np.array_equal(np.isnan(dw), nan)
            assert_bit_equal(np.where(nan, 0, dw), np.where(nan, 0, want), f"chain={chain} {path[-9:]}")
    xd = rng.standard_normal((1100, 50)).astype(np.float32)
    gd = rng.standard_normal((1100, 70)).astype(np.float32)
    wd = rng.standard_normal((50, 70)).astype(np.float32)
    lut, m = luts["MBM_7"]
    _, dwd = ops.denseam_grad(dev(gd), dev(xd), dev(wd), lut_path("MBM_7"), deterministic=True)
    assert_bit_equal(dwd.cpu().numpy(), oracle.dense_bwd_weight(xd, gd, lut, m), f"dense weight-grad chain={chain}")


@pytest.mark.parametrize("thin", [None, "1", "0"])
def test_deterministic_filter_gradient_thin_and_tiled_kernels(ops, oracle, luts, thin, monkeypatch, tmp_path):
    """Deterministic filter / weight gradients keep one serial chain per output; small
    outputs run with few chains per thread (whole device busy), large ones with the
    64-chain register tile.  Both kernels, forced and as chosen by the library, are
    bit-identical to the oracle for every table mode."""
    if thin is not None:
        set_switch(monkeypatch, "AMSIM_THIN_FGRAD", thin)
    rng = np.random.default_rng(91)
    lut9 = rng.integers(0, 256, size=1 << 18, dtype=np.uint8)
    path9 = str(tmp_path / "RAND_9.bin")
    lut9.tofile(path9)
    tables = [(lut_path("MBM_7"),) + luts["MBM_7"], (lut_path("MIT_7"),) + luts["MIT_7"], (lut_path("MBM_3"),) + luts["MBM_3"],
              (path9, lut9, 9)]
    cases = [(2, 9, 9, 8, 3, 3, 20, 1, "SAME"), (3, 12, 12, 3, 5, 5, 6, 2, "VALID"), (2, 10, 10, 64, 1, 1, 130, 1, "VALID"),
             (1, 16, 16, 32, 3, 3, 40, 2, "SAME")]
    for (path, lut, m) in tables:
        for (n, h, w, c, kh, kw, k, s, pad) in cases:
            x, _ = _conv_case(rng, n, h, w, c, kh, kw, k)
            g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
            dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
            dw = ops.convam_filter_grad((kh, kw, c, k), dev(x), dev(dy), strides=[1, s, s, 1], padding=pad,
                                        mant_mul_lut=path, deterministic=True).cpu().numpy()
            assert_bit_equal(dw, oracle.conv2d_bwd_filter(g, x, dy, lut, m), f"det filter-grad thin={thin} {path[-9:]}")
        xd = rng.standard_normal((37, 50)).astype(np.float32)
        xd[xd < -0.5] = 0
        wd = rng.standard_normal((50, 70)).astype(np.float32)
        gd = rng.standard_normal((37, 70)).astype(np.float32)
        _, dwd = ops.denseam_grad(dev(gd), dev(xd), dev(wd), path, deterministic=True)
        assert_bit_equal(dwd.cpu().numpy(), oracle.dense_bwd_weight(xd, gd, lut, m), f"det dense weight-grad thin={thin}")


@pytest.mark.parametrize("m", [8, 9, 11])
def test_large_lut_global_memory_path(ops, oracle, m, tmp_path):
    """m = 8..11: the table (up to 4 MiB) does not fit in shared memory and is
    looked up in global memory (L2-resident).  Same parity bars.  m = 11 uses
    the LUT generated from the reference's 32-bit MBM model when it is built,
    other widths a seeded random table (any byte pattern is a valid LUT)."""
    rng = np.random.default_rng(40 + m)
    if m == 11 and os.path.exists(BIG_LUT):
        from oracle.oracle import load_lut
        path = BIG_LUT
        lutb, _ = load_lut(path)
    else:
        lutb = rng.integers(0, 256, size=1 << (2 * m), dtype=np.uint8)
        path = str(tmp_path / f"RAND_{m}.bin")
        lutb.tofile(path)
    x, wt = _conv_case(rng, 2, 9, 9, 8, 3, 3, 20)
    g = oracle.geometry(2, 9, 9, 8, 3, 3, 20, 1, 1, "SAME")
    dy = rng.standard_normal((2, 9, 9, 20)).astype(np.float32)
    kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=path)
    for det in (True, False):
        chk = assert_bit_equal if det else assert_close
        chk(ops.convam(dev(x), dev(wt), deterministic=det, **kw_).cpu().numpy(), oracle.conv2d_fwd(g, x, wt, lutb, m), f"m={m} fwd")
        chk(ops.convam_filter_grad(wt.shape, dev(x), dev(dy), deterministic=det, **kw_).cpu().numpy(),
            oracle.conv2d_bwd_filter(g, x, dy, lutb, m), f"m={m} fgrad")
        chk(ops.convam_input_grad(x.shape, dev(wt), dev(dy), deterministic=det, **kw_).cpu().numpy(),
            oracle.conv2d_bwd_input(g, wt, dy, lutb, m), f"m={m} igrad")
        a = rng.standard_normal((3, 10, 33)).astype(np.float32)
        b = rng.standard_normal((3, 33, 7)).astype(np.float32)
        chk(ops.matmulam(dev(a), dev(b), mant_mul_lut=path, deterministic=det).cpu().numpy(), oracle.matmul(a, b, lutb, m), f"m={m} matmul")
        xd = rng.standard_normal((9, 21)).astype(np.float32)
        wd = rng.standard_normal((21, 5)).astype(np.float32)
        gd = rng.standard_normal((9, 5)).astype(np.float32)
        dxx, dww = ops.denseam_grad(dev(gd), dev(xd), dev(wd), path, deterministic=det)
        chk(dxx.cpu().numpy(), oracle.dense_bwd_input(wd, gd, lutb, m), f"m={m} dense dx")
        chk(dww.cpu().numpy(), oracle.dense_bwd_weight(xd, gd, lutb, m), f"m={m} dense dw")


# The shape table of the reference's own convolution test (test/convam_final_test.py:167-196), including the
# four entries its dict literal overwrites: (N, H, W, C, KH, KW, C, K).
REFERENCE_TEST_SHAPES = [
    (1, 4, 4, 1, 4, 4, 1, 1), (1, 4, 4, 1, 3, 3, 1, 1), (1, 4, 4, 1, 2, 2, 1, 1), (1, 4, 4, 1, 1, 1, 1, 1),
    (1, 4, 8, 1, 4, 4, 1, 1), (1, 4, 8, 1, 3, 3, 1, 1), (1, 4, 8, 1, 2, 2, 1, 1), (1, 4, 8, 1, 1, 1, 1, 1),
    (1, 4, 8, 1, 4, 5, 1, 1), (1, 4, 8, 1, 3, 4, 1, 1), (1, 4, 8, 1, 2, 1, 1, 1),
    (1, 4, 8, 2, 4, 5, 2, 3), (1, 4, 8, 2, 3, 4, 2, 3), (1, 4, 8, 2, 2, 1, 2, 3), (1, 4, 8, 2, 1, 1, 2, 3),
    (1, 8, 4, 3, 5, 4, 3, 4), (1, 8, 4, 3, 3, 4, 3, 4), (1, 8, 4, 3, 2, 1, 3, 4), (1, 8, 4, 3, 1, 1, 3, 4),
    (1, 20, 20, 3, 5, 5, 3, 4), (1, 20, 20, 3, 5, 4, 3, 4), (1, 20, 20, 3, 2, 1, 3, 4), (1, 20, 20, 3, 1, 1, 3, 4),
    (128, 32, 32, 1, 5, 5, 1, 6), (128, 14, 14, 6, 5, 5, 6, 16), (4, 4, 4, 1, 2, 2, 1, 2), (4, 14, 14, 1, 5, 5, 1, 16),
]


@pytest.mark.parametrize("stride", [1, 2])
def test_reference_conv_test_matrix(ops, oracle, luts, stride):
    """Same inputs and acceptance as the reference's test: integers in [-2, 2)
    (:165-166), forward and both gradients for VALID and SAME compared with the
    exact convolution, pass if the mean error is <= 1e-7 (:16-17,64) — run with
    the bf16-exact LUT, the closest LUT to the exact-multiply build that test
    targets — and additionally bit for bit against the oracle in deterministic mode."""
    lut, m = luts["ACC_7"]
    rng = np.random.default_rng(1000 + stride)
    for shape in REFERENCE_TEST_SHAPES:
        n, h, w, c, kh, kw, _, k = shape
        for padding in ("VALID", "SAME"):
            if padding == "VALID" and (kh > h or kw > w):
                continue
            x = rng.integers(-2, 2, size=(n, h, w, c)).astype(np.float32)
            wt = rng.integers(-2, 2, size=(kh, kw, c, k)).astype(np.float32)
            g = oracle.geometry(n, h, w, c, kh, kw, k, stride, stride, padding)
            dy = rng.integers(-2, 2, size=(n, g.out_h, g.out_w, k)).astype(np.float32)
            kw_ = dict(strides=[1, stride, stride, 1], padding=padding, mant_mul_lut=lut_path("ACC_7"))
            exact = (oracle.cpu_conv2d_fwd(g, x, wt), oracle.cpu_conv2d_bwd_filter(g, x, dy), oracle.cpu_conv2d_bwd_input(g, wt, dy))
            for det in (False, True):
                got = (ops.convam(dev(x), dev(wt), deterministic=det, **kw_).cpu().numpy(),
                       ops.convam_filter_grad(wt.shape, dev(x), dev(dy), deterministic=det, **kw_).cpu().numpy(),
                       ops.convam_input_grad(x.shape, dev(wt), dev(dy), deterministic=det, **kw_).cpu().numpy())
                for a, b, what in zip(got, exact, ("fwd", "filter-grad", "input-grad")):
                    assert np.abs(a - b).mean() <= 1e-7, (shape, padding, what, det)
                if det:
                    assert_bit_equal(got[0], oracle.conv2d_fwd(g, x, wt, lut, m), f"{shape} {padding} fwd")
                    assert_bit_equal(got[1], oracle.conv2d_bwd_filter(g, x, dy, lut, m), f"{shape} {padding} fgrad")
                    assert_bit_equal(got[2], oracle.conv2d_bwd_input(g, wt, dy, lut, m), f"{shape} {padding} igrad")
                else:
                    for a, b in zip(got, exact):
                        assert np.array_equal(a, b)   # integer products and sums are exact in fast mode


def test_int32_ops(ops, oracle, luts):
    """T = int32 (the reference registers its conv and dense ops for float and
    int32): operands go through the multiplier as floats, the int32 accumulator
    is truncated at every step.  Bit-exact vs the oracle."""
    lut, m = luts["MBM_7"]
    rng = np.random.default_rng(77)
    for (n, h, w, c, kh, kw, k, s, pad) in [(2, 7, 6, 3, 3, 3, 5, 1, "SAME"), (1, 9, 9, 4, 3, 2, 6, 2, "VALID"), (2, 6, 6, 2, 5, 5, 3, 2, "SAME")]:
        g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
        x = rng.integers(-40, 40, size=(n, h, w, c)).astype(np.int32)
        x[rng.random(x.shape) < 0.3] = 0
        wt = rng.integers(-9, 9, size=(kh, kw, c, k)).astype(np.int32)
        dy = rng.integers(-20, 20, size=(n, g.out_h, g.out_w, k)).astype(np.int32)
        kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=lut_path("MBM_7"))
        y = ops.convam(dev(x), dev(wt), **kw_)
        assert y.dtype == torch.int32
        assert np.array_equal(y.cpu().numpy(), oracle.conv2d_i32("fwd", g, x, wt, lut, m))
        assert np.array_equal(ops.convam_filter_grad(wt.shape, dev(x), dev(dy), **kw_).cpu().numpy(),
                              oracle.conv2d_i32("bwd_filter", g, x, dy, lut, m))
        assert np.array_equal(ops.convam_input_grad(x.shape, dev(wt), dev(dy), **kw_).cpu().numpy(),
                              oracle.conv2d_i32("bwd_input", g, wt, dy, lut, m))
    xd = rng.integers(-30, 30, size=(6, 17)).astype(np.int32)
    wd = rng.integers(-30, 30, size=(17, 5)).astype(np.int32)
    gd = rng.integers(-30, 30, size=(6, 5)).astype(np.int32)
    p = lut_path("MBM_7")
    assert np.array_equal(ops.denseam(dev(xd), dev(wd), p).cpu().numpy(), oracle.gemm_i32(xd, wd, lut, m))
    dxx, dww = ops.denseam_grad(dev(gd), dev(xd), dev(wd), p)
    assert np.array_equal(dww.cpu().numpy(), oracle.gemm_i32(np.ascontiguousarray(xd.T), gd, lut, m))
    # dx[b,k] = sum_u AM(w[k,u], g[b,u]) with the weight as first operand
    assert np.array_equal(dxx.cpu().numpy(), np.ascontiguousarray(oracle.gemm_i32(wd, np.ascontiguousarray(gd.T), lut, m).T))
    with pytest.raises(TypeError):
        ops.matmulam(dev(xd), dev(wd), mant_mul_lut=p)
    with pytest.raises(TypeError):
        ops.denseam(dev(xd), dev(wd.astype(np.float32)), p)


def test_fused_bias_relu_epilogue_equals_unfused_sequence(ops, oracle, luts):
    """act(op(x, w) + bias) in the kernel epilogue vs op, then FP32 add, then
    ReLU as separate exact steps: bit-identical, both modes, including a shape
    that takes the cluster-split path."""
    lut, m = luts["MBM_7"]
    p = lut_path("MBM_7")
    rng = np.random.default_rng(55)
    for (n, h, w, c, kh, kw, k, s, pad) in [(2, 9, 9, 8, 3, 3, 20, 1, "SAME"), (2, 7, 7, 64, 3, 3, 96, 1, "SAME"), (1, 8, 8, 3, 5, 5, 6, 2, "VALID")]:
        x, wt = _conv_case(rng, n, h, w, c, kh, kw, k)
        b = rng.standard_normal(k).astype(np.float32)
        g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
        for det in (True, False):
            kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=p, deterministic=det)
            base = ops.convam(dev(x), dev(wt), **kw_)
            for act in (None, "relu"):
                want = base + dev(b)
                if act == "relu":
                    want = torch.relu(want)
                got = ops.convam_bias_act(dev(x), dev(wt), dev(b), activation=act, **kw_)
                assert torch.equal(got, want), (det, act)
            assert torch.equal(ops.convam_bias_act(dev(x), dev(wt), None, activation="relu", **kw_), torch.relu(base))
        ref = np.maximum(oracle.conv2d_fwd(g, x, wt, lut, m) + b, 0).astype(np.float32)
        got = ops.convam_bias_act(dev(x), dev(wt), dev(b), strides=[1, s, s, 1], padding=pad, activation="relu",
                                  mant_mul_lut=p, deterministic=True).cpu().numpy()
        assert np.array_equal(got, ref)
    # per-channel scale before the bias: an inference BatchNormalization folded behind the convolution
    x, wt = _conv_case(rng, 2, 9, 9, 8, 3, 3, 20)
    sc = (rng.standard_normal(20) * 0.5 + 1).astype(np.float32)
    b = rng.standard_normal(20).astype(np.float32)
    for det in (True, False):
        kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=p, deterministic=det)
        base = ops.convam(dev(x), dev(wt), **kw_)
        got = ops.convam_bias_act(dev(x), dev(wt), dev(b), activation="relu", scale=dev(sc), **kw_)
        assert torch.equal(got, torch.relu(base * dev(sc) + dev(b))), det
        assert torch.equal(ops.convam_bias_act(dev(x), dev(wt), None, scale=dev(sc), **kw_), base * dev(sc))
    xd = rng.standard_normal((33, 50)).astype(np.float32)
    wd = rng.standard_normal((50, 70)).astype(np.float32)
    bd = rng.standard_normal(70).astype(np.float32)
    for det in (True, False):
        want = torch.relu(ops.denseam(dev(xd), dev(wd), p, deterministic=det) + dev(bd))
        assert torch.equal(ops.denseam_bias_act(dev(xd), dev(wd), dev(bd), activation="relu", mant_mul_lut=p, deterministic=det), want)
    with pytest.raises(ValueError):
        ops.denseam_bias_act(dev(xd), dev(wd), dev(bd), activation="tanh", mant_mul_lut=p)


def test_lut_handle_cache_and_lifecycle(ops):
    """Handles are shared per (real path, device) and reference counted
    (the reference keeps one private copy per OpKernel: convam.cc:498-499,712,979)."""
    import ctypes as C
    from approxtrain_b200 import _lib
    p = lut_path("MIT_3").encode()
    h1, h2 = C.c_void_p(), C.c_void_p()
    assert _lib.lib.amsim_lut_open(p, 0, C.byref(h1)) == 0
    rel = os.path.relpath(lut_path("MIT_3")).encode()          # another spelling of the same file
    assert _lib.lib.amsim_lut_open(rel, 0, C.byref(h2)) == 0
    assert h1.value == h2.value
    m, mask, a_s, b_s, ptr = C.c_int(), C.c_uint32(), C.c_int(), C.c_int(), C.c_void_p()
    assert _lib.lib.amsim_lut_info(h1, C.byref(m), C.byref(mask), C.byref(a_s), C.byref(b_s), C.byref(ptr)) == 0
    assert (m.value, mask.value, a_s.value, b_s.value) == (3, 0x700000, 17, 20)   # approx_mul_lut.h:26-28
    assert _lib.lib.amsim_lut_close(h1) == 0
    # still usable through the second reference
    x = torch.randn(4, 8, device="cuda")
    w = torch.randn(8, 4, device="cuda")
    y = torch.empty(4, 4, device="cuda")
    assert _lib.lib.amsim_dense_fwd(None, h2, C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(y.data_ptr()), 4, 4, 8, 0) == 0
    torch.cuda.synchronize()
    assert _lib.lib.amsim_lut_close(h2) == 0
    assert _lib.lib.amsim_lut_close(None) == 0


def test_concurrent_streams_do_not_interfere(ops, oracle, luts):
    """Calls are stream-ordered and re-entrant: two streams running split-K filter
    gradients (each with its own workspace) and forward passes at the same time
    give the results of running them one after the other."""
    p = lut_path("MBM_7")
    g = torch.Generator(device="cuda").manual_seed(9)
    xs = [torch.randn(8, 20, 20, 16, device="cuda", generator=g) for _ in range(2)]
    ws = [torch.randn(3, 3, 16, 32, device="cuda", generator=g) for _ in range(2)]
    dys = [torch.randn(8, 20, 20, 32, device="cuda", generator=g) for _ in range(2)]
    kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=p)
    want = [(ops.convam(x, w, **kw_), ops.convam_filter_grad(w.shape, x, dy, **kw_)) for x, w, dy in zip(xs, ws, dys)]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = [None, None]
    for rep in range(5):
        for i, s in enumerate(streams):
            with torch.cuda.stream(s):
                got[i] = (ops.convam(xs[i], ws[i], **kw_), ops.convam_filter_grad(ws[i].shape, xs[i], dys[i], **kw_))
        torch.cuda.synchronize()
        for i in range(2):
            assert torch.equal(got[i][0], want[i][0]) and torch.equal(got[i][1], want[i][1])


def test_oversize_and_invalid_arguments_are_refused_before_any_launch(ops):
    """Index arithmetic is 32-bit for rows and the reduction: shapes beyond it are
    refused with a status, nothing is launched (the reference would overflow its
    int products silently)."""
    import ctypes as C
    from approxtrain_b200 import _lib
    lut = ops.get_lut(lut_path("MBM_7"), "cuda")
    t = torch.zeros(16, device="cuda")
    P = C.c_void_p(t.data_ptr())
    L = _lib.lib
    # 2^20 images of 64x64: more than 2^31 pixels
    assert L.amsim_conv2d_fwd(None, lut.handle, P, P, P, 1 << 20, 64, 64, 4, 3, 3, 4, 64, 64, 1, 1, 1, 1, 0) == _lib.ERR_UNSUPPORTED
    # reduction length beyond 2^30
    assert L.amsim_conv2d_fwd(None, lut.handle, P, P, P, 1, 4096, 4096, 1 << 16, 128, 128, 4, 3969, 3969, 1, 1, 0, 0, 0) == _lib.ERR_UNSUPPORTED
    # non-positive stride, negative padding, unknown flag bits, NULL tensors
    assert L.amsim_conv2d_fwd(None, lut.handle, P, P, P, 1, 4, 4, 1, 3, 3, 1, 2, 2, 0, 1, 0, 0, 0) == _lib.ERR_INVALID
    assert L.amsim_conv2d_fwd(None, lut.handle, P, P, P, 1, 4, 4, 1, 3, 3, 1, 2, 2, 1, 1, -1, 0, 0) == _lib.ERR_INVALID
    assert L.amsim_conv2d_fwd(None, lut.handle, P, P, P, 1, 4, 4, 1, 3, 3, 1, 2, 2, 1, 1, 0, 0, 64) == _lib.ERR_INVALID
    assert L.amsim_conv2d_fwd(None, lut.handle, None, P, P, 1, 4, 4, 1, 3, 3, 1, 2, 2, 1, 1, 0, 0, 0) == _lib.ERR_INVALID
    assert L.amsim_dense_fwd(None, None, P, P, P, 2, 2, 2, 0) == _lib.ERR_INVALID
    assert L.amsim_matmul(None, lut.handle, P, P, P, 0, 0, 2, 3, 4, 2, 0) == _lib.ERR_INVALID
    assert b"cols of mat a" in L.amsim_last_error()
    assert L.amsim_conv2d_fwd_bias_act(None, lut.handle, P, P, None, P, 1, 4, 4, 1, 3, 3, 1, 2, 2, 1, 1, 0, 0, 7, 0) == _lib.ERR_INVALID
    torch.cuda.synchronize()


def test_additive_table_shortcut_is_bit_identical_to_the_table_path(ops, oracle, luts, tmp_path, monkeypatch):
    """A LUT whose encoded entries satisfy entry(i, j) == i + j (Mitchell's
    multiplier: MIT_1/3/5/7) is served without table lookups (integer add of the
    mantissa fields).  Same bits as the shared-memory table path and the oracle,
    in both modes, for all three directions."""
    import shutil
    lut, m = luts["MIT_7"]
    rng = np.random.default_rng(123)
    x, wt = _conv_case(rng, 3, 11, 10, 12, 3, 3, 40)
    g = oracle.geometry(3, 11, 10, 12, 3, 3, 40, 1, 1, "SAME")
    dy = rng.standard_normal((3, g.out_h, g.out_w, 40)).astype(np.float32)
    dy[dy < -0.8] = 0
    # a second copy of the file, opened with the shortcut disabled -> table path
    table_copy = str(tmp_path / "MITCOPY_7.bin")
    shutil.copyfile(lut_path("MIT_7"), table_copy)
    set_switch(monkeypatch, "AMSIM_NO_ADDITIVE", "1")
    ops.get_lut(table_copy, "cuda")
    set_switch(monkeypatch, "AMSIM_NO_ADDITIVE", None)
    for det in (True, False):
        outs = {}
        for tag, path in (("add", lut_path("MIT_7")), ("table", table_copy)):
            kw_ = dict(strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=path, deterministic=det)
            outs[tag] = (ops.convam(dev(x), dev(wt), **kw_), ops.convam_filter_grad(wt.shape, dev(x), dev(dy), **kw_),
                         ops.convam_input_grad(x.shape, dev(wt), dev(dy), **kw_))
        for a, b in zip(outs["add"], outs["table"]):
            assert torch.equal(a, b), det
        if det:
            assert_bit_equal(outs["add"][0].cpu().numpy(), oracle.conv2d_fwd(g, x, wt, lut, m), "additive fwd")
            assert_bit_equal(outs["add"][1].cpu().numpy(), oracle.conv2d_bwd_filter(g, x, dy, lut, m), "additive fgrad")
            assert_bit_equal(outs["add"][2].cpu().numpy(), oracle.conv2d_bwd_input(g, wt, dy, lut, m), "additive igrad")


@pytest.mark.parametrize("name", ["MBM32", "MIT32"])
def test_direct_32bit_models(ops, oracle, name):
    """mant_mul_lut = "direct:MBM32" / "direct:MIT32": the reference's direct C simulation
    of its 32-bit multipliers (cuda/FPmultMBM_fast32.inl, cuda/Mitchell_32.inl) computed
    per product inside the same kernels.  The primitive reproduces the committed outputs
    of the reference's code bit for bit; conv / dense / matmul in every direction equal
    the oracle bit for bit with either mode flag (one ordered kernel flavour)."""
    from oracle.oracle import DIRECT_MBM32, DIRECT_MIT32, NO_LUT
    m = DIRECT_MBM32 if name == "MBM32" else DIRECT_MIT32
    path = "direct:" + name
    kat = np.load(os.path.join(GOLDEN, "direct_kat.npz"))
    at, bt = kat["at"], kat["bt"]
    got = ops.am_multiply(dev(at.view(np.float32)), dev(bt.view(np.float32)), path).cpu().numpy().view(np.uint32)
    want = kat["out_" + name]
    nan = np.isnan(want.view(np.float32))   # a NaN's payload is the host's or the GPU's, not the model's
    assert np.array_equal(np.isnan(got.view(np.float32)), nan)
    assert_bit_equal(np.where(nan, 0, got).view(np.float32), np.where(nan, 0, want).view(np.float32),
                     f"{name} primitive vs reference outputs")
    rng = np.random.default_rng(123)
    for (n, h, w, c, kh, kw, k, s, pad) in [(2, 9, 9, 8, 3, 3, 20, 1, "SAME"), (2, 11, 10, 3, 5, 3, 6, 2, "VALID"),
                                            (1, 12, 12, 16, 3, 3, 70, 2, "SAME")]:
        x, wt = _conv_case(rng, n, h, w, c, kh, kw, k)
        g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
        dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
        for det in (True, False):
            kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=path, deterministic=det)
            assert_bit_equal(ops.convam(dev(x), dev(wt), **kw_).cpu().numpy(), oracle.conv2d_fwd(g, x, wt, NO_LUT, m), f"{name} fwd")
            assert_bit_equal(ops.convam_input_grad(x.shape, dev(wt), dev(dy), **kw_).cpu().numpy(),
                             oracle.conv2d_bwd_input(g, wt, dy, NO_LUT, m), f"{name} input-grad")
            assert_bit_equal(ops.convam_filter_grad(wt.shape, dev(x), dev(dy), **kw_).cpu().numpy(),
                             oracle.conv2d_bwd_filter(g, x, dy, NO_LUT, m), f"{name} filter-grad")
    xd = rng.standard_normal((37, 50)).astype(np.float32)
    wd = rng.standard_normal((50, 70)).astype(np.float32)
    gd = rng.standard_normal((37, 70)).astype(np.float32)
    assert_bit_equal(ops.denseam(dev(xd), dev(wd), path).cpu().numpy(), oracle.dense_fwd(xd, wd, NO_LUT, m), f"{name} dense")
    dxd, dwd = ops.denseam_grad(dev(gd), dev(xd), dev(wd), path)
    assert_bit_equal(dxd.cpu().numpy(), oracle.dense_bwd_input(wd, gd, NO_LUT, m), f"{name} dense dx")
    assert_bit_equal(dwd.cpu().numpy(), oracle.dense_bwd_weight(xd, gd, NO_LUT, m), f"{name} dense dw")
    a = rng.standard_normal((3, 10, 21)).astype(np.float32)
    b = rng.standard_normal((3, 21, 14)).astype(np.float32)
    assert_bit_equal(ops.matmulam(dev(a), dev(b), mant_mul_lut=path).cpu().numpy(), oracle.matmul(a, b, NO_LUT, m), f"{name} matmul")
    # inf / NaN pass through, a zero product is +0
    sp = np.array([np.inf, -np.inf, np.nan, 0.0, -0.0, 1e-45, 3.0], np.float32)
    A, B = np.meshgrid(sp, sp)
    got = ops.am_multiply(dev(A.copy()), dev(B.copy()), path).cpu().numpy()
    want = oracle.mul(A.copy(), B.copy(), NO_LUT, m)
    assert np.array_equal(got.view(np.uint32) & 0x7F800000, want.view(np.uint32) & 0x7F800000) and \
        np.array_equal(np.isnan(got), np.isnan(want))
    with pytest.raises(Exception):
        ops.am_multiply(dev(A.copy()), dev(B.copy()), "direct:FOO")
    with pytest.raises(Exception):
        ops.denseam(dev(xd.astype(np.int32)), dev(wd.astype(np.int32)), path)


@pytest.mark.parametrize("noswap", [None, "1"])
def test_weight_gradient_with_swapped_operand_roles(ops, oracle, luts, noswap, monkeypatch):
    """GEMM-shaped weight gradients (dense; 1x1 stride-1 convolutions) with few inputs and
    many outputs run with the gradient as the lane operand and the input as the uniform
    one, the table indexed the other way round and the output written transposed: same
    products, same chains.  Deterministic bit-exact, fast within the bar, asymmetric LUT."""
    if noswap:
        set_switch(monkeypatch, "AMSIM_NO_WGRAD_SWAP", noswap)
    rng = np.random.default_rng(64)
    lut = rng.integers(0, 256, size=1 << 10, dtype=np.uint8)   # m = 5, not symmetric
    from approxtrain_b200 import _lib
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "ASYM_5.bin")
        lut.tofile(path)
        for name, (lt, m, pth) in {"asym": (lut, 5, path), "MBM_7": luts["MBM_7"] + (lut_path("MBM_7"),)}.items():
            x, _ = _conv_case(rng, 3, 10, 10, 64, 1, 1, 256)
            g = oracle.geometry(3, 10, 10, 64, 1, 1, 256, 1, 1, "VALID")
            dy = rng.standard_normal((3, 10, 10, 256)).astype(np.float32)
            want = oracle.conv2d_bwd_filter(g, x, dy, lt, m)
            kw_ = dict(strides=[1, 1, 1, 1], padding="VALID", mant_mul_lut=pth)
            got = ops.convam_filter_grad((1, 1, 64, 256), dev(x), dev(dy), deterministic=True, **kw_).cpu().numpy()
            assert_bit_equal(got, want, f"1x1 filter-grad det {name} noswap={noswap}")
            got = ops.convam_filter_grad((1, 1, 64, 256), dev(x), dev(dy), **kw_).cpu().numpy()
            assert_close(got, want, f"1x1 filter-grad fast {name} noswap={noswap}")
            xd = rng.standard_normal((300, 40)).astype(np.float32)
            wd = rng.standard_normal((40, 200)).astype(np.float32)
            gd = rng.standard_normal((300, 200)).astype(np.float32)
            wantd = oracle.dense_bwd_weight(xd, gd, lt, m)
            _, dwd = ops.denseam_grad(dev(gd), dev(xd), dev(wd), pth, deterministic=True)
            assert_bit_equal(dwd.cpu().numpy(), wantd, f"dense weight-grad det {name} noswap={noswap}")
            _, dwd = ops.denseam_grad(dev(gd), dev(xd), dev(wd), pth)
            assert_close(dwd.cpu().numpy(), wantd, f"dense weight-grad fast {name} noswap={noswap}")


@pytest.mark.parametrize("exact_only", [None, "1"])
def test_deterministic_mode_hazard_stages(ops, oracle, luts, exact_only, monkeypatch):
    """Deterministic kernels run a stage on the fast arithmetic when none of its operands can
    reach one of the reference's special behaviours, and bit by bit otherwise.  Data that
    mixes ordinary values with every hazard (zeros next to operands >= 2, magnitudes below
    2^-63 and above 2^63, denormals, exponent sums <= 127, overflow into the sign bit) stays
    bit-identical to the oracle in all three directions, with the fast arithmetic allowed
    and with it switched off."""
    if exact_only:
        set_switch(monkeypatch, "AMSIM_EXACT_ONLY", exact_only)
    set_switch(monkeypatch, "AMSIM_THIN_FGRAD", "0")   # the tiled filter-gradient kernel is the one with the two loops
    rng = np.random.default_rng(2718)

    def spice(a, frac=0.08):
        a = a.copy().reshape(-1)
        n = a.size
        specials = np.array([0.0, -0.0, 2.5, -3.0, 1e-30, -1e-25, 1e25, -3e30, 1e-40, 6e-39, 1e38, -2e38,
                             2.0 ** -63, 2.0 ** 63, 2.0 ** -64, 2.0 ** 64], np.float32)
        idx = rng.choice(n, size=max(1, int(n * frac)), replace=False)
        a[idx] = rng.choice(specials, size=idx.size)
        return a

    for name in ("MBM_7", "MIT_7", "MBM_3"):
        lut, m = luts[name]
        path = lut_path(name)
        for (n, h, w, c, kh, kw, k, s, pad) in [(2, 9, 9, 8, 3, 3, 20, 1, "SAME"), (1, 12, 12, 16, 3, 3, 70, 2, "SAME")]:
            x, wt = _conv_case(rng, n, h, w, c, kh, kw, k)
            g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
            dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
            for variant in range(3):
                # 0: hazards everywhere; 1: only in a corner of x (most stages hazard-free); 2: none
                xs, ws, ds = x, wt, dy
                if variant == 0:
                    xs, ws, ds = spice(x).reshape(x.shape), spice(wt).reshape(wt.shape), spice(dy).reshape(dy.shape)
                elif variant == 1:
                    xs = x.copy()
                    xs[0, :2, :2, :] = spice(xs[0, :2, :2, :], 0.5).reshape(xs[0, :2, :2, :].shape)
                kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=path, deterministic=True)
                with np.errstate(all="ignore"):
                    want_y = oracle.conv2d_fwd(g, xs, ws, lut, m)
                    want_dx = oracle.conv2d_bwd_input(g, ws, ds, lut, m)
                    want_dw = oracle.conv2d_bwd_filter(g, xs, ds, lut, m)
                def same(got, want, what):
                    got = got.cpu().numpy()
                    nan = np.isnan(want)
                    assert np.array_equal(np.isnan(got), nan), what
                    assert_bit_equal(np.where(nan, 0, got), np.where(nan, 0, want), what)
                same(ops.convam(dev(xs), dev(ws), **kw_), want_y, f"{name} fwd v{variant}")
                same(ops.convam_input_grad(xs.shape, dev(ws), dev(ds), **kw_), want_dx, f"{name} input-grad v{variant}")
                same(ops.convam_filter_grad(ws.shape, dev(xs), dev(ds), **kw_), want_dw, f"{name} filter-grad v{variant}")


@pytest.mark.parametrize("m", [5, 9])
def test_tables_with_16_bit_entries(ops, oracle, m, tmp_path):
    """A LUT file of twice the usual size holds 16-bit entries (carry << 15 | 15 mantissa
    bits), a format extension that makes m = 8..11 numerically meaningful.  The table is
    looked up in global memory; primitive bit-exact for every exponent class, GEMM ops
    bit-exact in deterministic mode and within the bar in fast mode."""
    from approxtrain_b200 import lutgen
    from oracle.oracle import DIRECT_MBM32, NO_LUT, load_lut
    path = str(tmp_path / f"MBMW_{m}.bin")
    lutgen.write(path, lambda a, b: oracle.mul(a, b, NO_LUT, DIRECT_MBM32), m, entry_bits=16)
    lut, mw = load_lut(path)
    kat = np.load(os.path.join(GOLDEN, "prim_kat.npz"))      # operand grid over all exponent classes
    at, bt = kat["at"], kat["bt"]
    got = ops.am_multiply(dev(at.view(np.float32)), dev(bt.view(np.float32)), path).cpu().numpy().view(np.uint32)
    want = oracle.mul(at.view(np.float32), bt.view(np.float32), lut, mw).view(np.uint32)
    assert np.array_equal(got, want)
    rng = np.random.default_rng(160 + m)
    for (n, h, w, c, kh, kw, k, s, pad) in [(2, 9, 9, 8, 3, 3, 20, 1, "SAME"), (1, 12, 12, 3, 5, 5, 6, 2, "VALID")]:
        x, wt = _conv_case(rng, n, h, w, c, kh, kw, k)
        g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
        dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
        kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=path)
        want_y, want_dx = oracle.conv2d_fwd(g, x, wt, lut, mw), oracle.conv2d_bwd_input(g, wt, dy, lut, mw)
        want_dw = oracle.conv2d_bwd_filter(g, x, dy, lut, mw)
        assert_bit_equal(ops.convam(dev(x), dev(wt), deterministic=True, **kw_).cpu().numpy(), want_y, "wide fwd det")
        assert_bit_equal(ops.convam_input_grad(x.shape, dev(wt), dev(dy), deterministic=True, **kw_).cpu().numpy(), want_dx, "wide dx det")
        assert_bit_equal(ops.convam_filter_grad(wt.shape, dev(x), dev(dy), deterministic=True, **kw_).cpu().numpy(), want_dw, "wide dw det")
        assert_close(ops.convam(dev(x), dev(wt), **kw_).cpu().numpy(), want_y, "wide fwd fast")
        assert_close(ops.convam_input_grad(x.shape, dev(wt), dev(dy), **kw_).cpu().numpy(), want_dx, "wide dx fast")
        assert_close(ops.convam_filter_grad(wt.shape, dev(x), dev(dy), **kw_).cpu().numpy(), want_dw, "wide dw fast")
    a = rng.standard_normal((3, 10, 21)).astype(np.float32)
    b = rng.standard_normal((3, 21, 14)).astype(np.float32)
    assert_bit_equal(ops.matmulam(dev(a), dev(b), mant_mul_lut=path, deterministic=True).cpu().numpy(),
                     oracle.matmul(a, b, lut, mw), "wide matmul")
    with pytest.raises(Exception):   # int32 ops take byte tables only
        ops.denseam(dev(np.ones((2, 3), np.int32)), dev(np.ones((3, 2), np.int32)), path)
    bad = str(tmp_path / "BAD_5.bin")
    np.zeros(3 << 10, np.uint8).tofile(bad)     # neither 2^(2m) nor twice that
    with pytest.raises(Exception):
        ops.am_multiply(dev(a), dev(a), bad)


@pytest.mark.parametrize("off", [None, "1"])
def test_narrow_outputs_share_column_groups_between_warps(ops, oracle, luts, off, monkeypatch):
    """Outputs of at most 32 columns (a 3-channel image gradient, LeNet-5's 6 and 16 filters, a
    10-class head): 2 or 4 warps take the same columns and every 2nd / 4th reduction step, and
    their register tiles are added in warp order.  Fast mode only; same bar, run-to-run identical,
    fused epilogue and strided (stride-phase) outputs included."""
    if off:
        set_switch(monkeypatch, "AMSIM_NO_QSPLIT", off)
    rng = np.random.default_rng(321)
    for name in ("MBM_7", "MIT_7"):
        lut, m = luts[name]
        path = lut_path(name)
        for (n, h, w, c, kh, kw, k, s, pad) in [(2, 20, 20, 3, 7, 7, 16, 2, "VALID"),   # input gradient has 3 columns
                                                (4, 28, 28, 1, 5, 5, 6, 1, "SAME"),     # LeNet-5 conv1
                                                (4, 14, 14, 6, 5, 5, 16, 1, "VALID"),   # LeNet-5 conv2
                                                (2, 9, 9, 32, 3, 3, 20, 1, "SAME")]:    # 20 columns: two warps per group
            x, wt = _conv_case(rng, n, h, w, c, kh, kw, k)
            g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
            dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
            b = rng.standard_normal(k).astype(np.float32)
            kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=path)
            y = ops.convam(dev(x), dev(wt), **kw_)
            assert_close(y.cpu().numpy(), oracle.conv2d_fwd(g, x, wt, lut, m), f"narrow fwd {name}")
            assert torch.equal(y, ops.convam(dev(x), dev(wt), **kw_))
            dx = ops.convam_input_grad(x.shape, dev(wt), dev(dy), **kw_).cpu().numpy()
            assert_close(dx, oracle.conv2d_bwd_input(g, wt, dy, lut, m), f"narrow input-grad {name}")
            fused = ops.convam_bias_act(dev(x), dev(wt), dev(b), activation="relu", **kw_)
            assert torch.equal(fused, torch.relu(y + dev(b)))
        xd = rng.standard_normal((256, 84)).astype(np.float32)
        wd = rng.standard_normal((84, 10)).astype(np.float32)
        assert_close(ops.denseam(dev(xd), dev(wd), path).cpu().numpy(), oracle.dense_fwd(xd, wd, lut, m), f"narrow dense {name}")


def test_plain_c_program_over_the_abi():
    """approxtrain_b200/csrc/abi_driver.c — C99, no Python, no torch — opens a LUT, checks a
    deterministic convolution output against the ascending chain of primitive products, runs
    both gradients in both modes and the error path; exit code 0 means all of it passed."""
    import subprocess
    from approxtrain_b200 import _build
    exe = _build.DRIVER_PATH
    if not os.path.exists(exe):
        _build.build_driver()
    for name in ("MBM_7", "MIT_5"):
        out = subprocess.run([exe, lut_path(name)], capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, out.stderr[-2000:]
        assert "abi_driver ok" in out.stdout


@pytest.mark.parametrize("name", ["MBM_7", "MIT_7"])
def test_reference_gemm_known_inputs(ops, oracle, luts, name):
    """The reference's own GEMM test case (test/test_gemm.cu:10-15,45-67): A is 800 x 1600 with
    A[i][j] = i + j, B is 1600 x 800 with B[i][j] = i - j.  Its stored outputs are missing from
    the reference checkout, so the oracle's chain stands in for them: deterministic mode equals
    it bit for bit, fast mode within the bar (max-abs reported on failure)."""
    lut, m = luts[name]
    i, j = np.meshgrid(np.arange(800, dtype=np.float32), np.arange(1600, dtype=np.float32), indexing="ij")
    a = (i + j).astype(np.float32)
    i, j = np.meshgrid(np.arange(1600, dtype=np.float32), np.arange(800, dtype=np.float32), indexing="ij")
    b = (i - j).astype(np.float32)
    want = oracle.matmul(a, b, lut, m)
    got = ops.matmulam(dev(a), dev(b), mant_mul_lut=lut_path(name), deterministic=True).cpu().numpy()
    assert_bit_equal(got, want, f"reference GEMM case, deterministic, {name}")
    fast = ops.matmulam(dev(a), dev(b), mant_mul_lut=lut_path(name)).cpu().numpy()
    assert_close(fast, want, f"reference GEMM case, fast, {name}")
    # the dense entry points compute the same product
    y = ops.denseam(dev(a), dev(b), lut_path(name), deterministic=True).cpu().numpy()
    assert_bit_equal(y, want, f"reference GEMM case through Denseam, {name}")


@pytest.mark.parametrize("shape", [(32, 55, 55, 64), (8, 14, 14, 1024), (16, 28, 28, 6), (128, 10), (3, 7, 5, 2048), (1, 1000), (5, 0 + 1, 1, 3)])
def test_bias_gradient_is_the_exact_column_sum(ops, shape):
    """dbias[c] = sum of the output gradient over every other axis: exact FP32 adds in a fixed order.
    Compared with a float64 sum (the FP32 result is within a few ulp of accumulated rounding) and
    with itself (same bits on a second run, and on a copy at another address)."""
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    dy = torch.randn(*shape, device="cuda", generator=g)
    got = ops.bias_grad(dy)
    want = dy.double().reshape(-1, shape[-1]).sum(0)
    scale = dy.double().abs().reshape(-1, shape[-1]).sum(0).clamp_min(1e-30)
    assert got.shape == (shape[-1],)
    assert float(((got.double() - want).abs() / scale).max()) <= 1e-6
    assert torch.equal(got, ops.bias_grad(dy.clone()))
    ints = torch.randint(-3, 4, shape, device="cuda", generator=g).float()   # small integers: every partial sum is exact
    assert torch.equal(ops.bias_grad(ints), ints.reshape(-1, shape[-1]).sum(0))
