"""CPU tests that pin the oracle: LUT bytes against the reference's shipped
files (md5), the primitive against the reference's own cuda/AMsimulator.inl
(committed known answers, and exhaustively when oracle/_ref is built), and the
op restatements against an independent numpy formulation."""
import hashlib
import os

import numpy as np
import pytest

from conftest import GOLDEN, SMALL_LUTS, lut_path

# md5 of the LUT files the reference ships under lut/
REF_LUT_MD5 = {
    "ACC_7": "cf67922a5640c55b6a7abf0c4b927c47",
    "MBM_1": "bb82fc6713b0896b01e9f0fa476d50c1",
    "MBM_3": "29e18c81689699c7179d508bcd0dfe56",
    "MBM_5": "ca0ddff95daf9da6c5508136e946c88f",
    "MBM_7": "6bc995143860e1b32c681203c3b97e60",
    "MIT_1": "10aa0419ffedddf2b3fd08f5ee55ff7c",
    "MIT_3": "e383916434999b10672b6c6b5f0d91a9",
    "MIT_5": "219bd3e55a3641190adeacd167aceb84",
    "MIT_7": "444faa87fc98ce7326cc3fe3aa8b4b47",
}


@pytest.mark.parametrize("name", SMALL_LUTS)
def test_lut_bytes_match_reference_md5(name):
    with open(lut_path(name), "rb") as f:
        assert hashlib.md5(f.read()).hexdigest() == REF_LUT_MD5[name]


def test_tiny_luts_in_full():
    assert open(lut_path("MBM_1"), "rb").read() == bytes([0x80, 0x80, 0x80, 0x80])
    assert open(lut_path("MIT_1"), "rb").read() == bytes([0x00, 0x01, 0x01, 0x80])


def test_lut_name_parsing(oracle):
    p = oracle.lib.am_parse_mant_width
    assert p(b"lut/MBM_7.bin") == 7
    assert p(b"/a_b/c_d/MIT_11.bin") == 11
    assert p(b"nounderscore.bin") == -1
    assert p(b"X_12.bin") == -1      # a_shift = 23 - 2m would go negative
    assert p(b"X_0.bin") == -1
    assert p(b"X_.bin") == -1
    assert p(b"X_7") == -1


@pytest.mark.parametrize("name", SMALL_LUTS)
def test_primitive_matches_reference_known_answers(oracle, luts, name):
    kat = np.load(os.path.join(GOLDEN, "prim_kat.npz"))
    lut, m = luts[name]
    at, bt, want = kat["at"], kat["bt"], kat["out_" + name]
    got = oracle.mul(at.view(np.float32), bt.view(np.float32), lut, m).view(np.uint32)
    assert np.array_equal(got, want)


def test_primitive_documented_quirks(oracle, luts):
    lut, m = luts["MBM_7"]
    f = lambda a, b: oracle.mul(np.float32([a]), np.float32([b]), lut, m)
    assert f(0.0, 1.0).view(np.uint32)[0] == 0
    assert f(0.0, 4.0).view(np.uint32)[0] == 0x010C0000      # zero times |x| >= 2 is not zero
    assert f(1.0, 1.0)[0] == np.float32(1.09375)
    assert f(1e30, 1e30).view(np.uint32)[0] == 0xA3170000     # exponent overflow wraps into the sign
    assert f(np.inf, 2.0).view(np.uint32)[0] == 0x800C0000


@pytest.mark.parametrize("name", SMALL_LUTS)
def test_primitive_exhaustive_vs_reference_source(oracle, luts, name):
    """All 2^(2m) mantissa-index pairs x exponent classes x signs, compared
    bit for bit with the reference's cuda/AMsimulator.inl built as host code."""
    from oracle.oracle import RefPrimitive
    if not RefPrimitive.available():
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    ref = RefPrimitive()
    lut, m = luts[name]
    n = 1 << m
    ia, ib = np.meshgrid(np.arange(n, dtype=np.uint32), np.arange(n, dtype=np.uint32), indexing="ij")
    rng = np.random.default_rng(7)
    low = rng.integers(0, 1 << (23 - m), size=ia.shape, dtype=np.uint32)  # ignored low mantissa bits
    classes = [0, 1, 64, 126, 127, 128, 129, 200, 254, 255]
    for ea in classes:
        for eb in classes:
            for sa, sb in ((0, 0), (1, 0), (1, 1)):
                at = (np.uint32(sa) << 31) | (np.uint32(ea) << 23) | (ia << (23 - m)) | low
                bt = (np.uint32(sb) << 31) | (np.uint32(eb) << 23) | (ib << (23 - m)) | (low ^ 1)
                got = oracle.mul(at.view(np.float32), bt.view(np.float32), lut, m).view(np.uint32)
                want = ref.mul_bits_array(at, bt, lut, m).reshape(at.shape)
                assert np.array_equal(got, want), (name, ea, eb, sa, sb)


def _np_am(a, b, lut, m):
    """Independent vectorised numpy statement of the primitive."""
    at = np.ascontiguousarray(a, np.float32).view(np.uint32)
    bt = np.ascontiguousarray(b, np.float32).view(np.uint32)
    mask = np.uint32(((1 << m) - 1) << (23 - m))
    idx = ((at & mask) >> np.uint32(23 - 2 * m)) | ((bt & mask) >> np.uint32(23 - m))
    v = lut[idx].astype(np.uint32)
    e = ((at >> np.uint32(23)) & np.uint32(0xFF)) + ((bt >> np.uint32(23)) & np.uint32(0xFF))
    bits = ((at ^ bt) & np.uint32(0x80000000)) + ((e - np.uint32(127) + (v >> np.uint32(7))) << np.uint32(23)) \
        + ((v & np.uint32(0x7F)) << np.uint32(23 - m))
    bits = np.where(e <= 127, np.uint32(0), bits).astype(np.uint32)
    return bits.view(np.float32)


def _np_gemm(A, B, lut, m):
    M, K = A.shape
    N = B.shape[1]
    acc = np.zeros((M, N), np.float32)
    for k in range(K):
        acc = (acc + _np_am(np.broadcast_to(A[:, k:k + 1], (M, N)), np.broadcast_to(B[k:k + 1, :], (M, N)), lut, m)).astype(np.float32)
    return acc


def test_gemm_vs_numpy(oracle, luts):
    rng = np.random.default_rng(0)
    for name in ("MBM_7", "MIT_3", "ACC_7"):
        lut, m = luts[name]
        A = rng.standard_normal((13, 29)).astype(np.float32)
        B = rng.standard_normal((29, 11)).astype(np.float32)
        A[A < -1] = 0
        assert np.array_equal(oracle.gemm(A, B, lut, m).view(np.uint32), _np_gemm(A, B, lut, m).view(np.uint32))


def _np_im2col_fwd(g, x):
    cols = np.zeros((g.batch * g.out_h * g.out_w, g.f_h * g.f_w * g.in_c), np.float32)
    r = 0
    for n in range(g.batch):
        for oh in range(g.out_h):
            for ow in range(g.out_w):
                patch = np.zeros((g.f_h, g.f_w, g.in_c), np.float32)
                for kh in range(g.f_h):
                    for kw in range(g.f_w):
                        ih, iw = oh * g.stride_h - g.pad_top + kh, ow * g.stride_w - g.pad_left + kw
                        if 0 <= ih < g.in_h and 0 <= iw < g.in_w:
                            patch[kh, kw] = x[n, ih, iw]
                cols[r] = patch.reshape(-1)
                r += 1
    return cols


@pytest.mark.parametrize("pad,stride", [("SAME", 1), ("VALID", 1), ("SAME", 2), ("VALID", 2)])
def test_conv_ops_vs_numpy_im2col(oracle, luts, pad, stride):
    """Forward = im2col + GEMM (cuda_kernel.cu:34-60,161-172); gradients are
    checked through the same GEMM on explicitly built patch matrices."""
    lut, m = luts["MBM_7"]
    rng = np.random.default_rng(3)
    g = oracle.geometry(2, 6, 7, 3, 3, 2, 4, stride, stride, pad)
    x = rng.standard_normal((2, 6, 7, 3)).astype(np.float32)
    x[x < -0.3] = 0
    w = rng.standard_normal((3, 2, 3, 4)).astype(np.float32)
    dy = rng.standard_normal((2, g.out_h, g.out_w, 4)).astype(np.float32)
    cols = _np_im2col_fwd(g, x)
    y = _np_gemm(cols, w.reshape(-1, 4), lut, m).reshape(2, g.out_h, g.out_w, 4)
    assert np.array_equal(oracle.conv2d_fwd(g, x, w, lut, m).view(np.uint32), y.view(np.uint32))
    # filter grad: A = cols^T (rows (kh,kw,c), columns (n,oh,ow)), B = dy
    dw = _np_gemm(np.ascontiguousarray(cols.T), dy.reshape(-1, 4), lut, m).reshape(w.shape)
    assert np.array_equal(oracle.conv2d_bwd_filter(g, x, dy, lut, m).view(np.uint32), dw.view(np.uint32))
    # input grad: dilate + pad dy, gather (kh,kw,ko), B = flipped filter with C and K swapped
    hh, hw = (g.out_h - 1) * stride + 1, (g.out_w - 1) * stride + 1
    hole = np.zeros((2, hh, hw, 4), np.float32)
    hole[:, ::stride, ::stride] = dy
    bpt, bpl = g.f_h - 1 - g.pad_top, g.f_w - 1 - g.pad_left
    colsg = np.zeros((2 * 6 * 7, g.f_h * g.f_w * 4), np.float32)
    r = 0
    for n in range(2):
        for yy in range(6):
            for xx in range(7):
                patch = np.zeros((g.f_h, g.f_w, 4), np.float32)
                for kh in range(g.f_h):
                    for kw in range(g.f_w):
                        u, v = yy - bpt + kh, xx - bpl + kw
                        if 0 <= u < hh and 0 <= v < hw:
                            patch[kh, kw] = hole[n, u, v]
                colsg[r] = patch.reshape(-1)
                r += 1
    rs = np.ascontiguousarray(w[::-1, ::-1].transpose(0, 1, 3, 2)).reshape(-1, 3)
    dx = _np_gemm(colsg, rs, lut, m).reshape(x.shape)
    assert np.array_equal(oracle.conv2d_bwd_input(g, w, dy, lut, m).view(np.uint32), dx.view(np.uint32))


def test_dense_and_matmul_vs_numpy(oracle, luts):
    lut, m = luts["MIT_7"]
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 17)).astype(np.float32)
    w = rng.standard_normal((17, 9)).astype(np.float32)
    g = rng.standard_normal((6, 9)).astype(np.float32)
    eq = lambda a, b: np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert eq(oracle.dense_fwd(x, w, lut, m), _np_gemm(x, w, lut, m))
    assert eq(oracle.dense_bwd_weight(x, g, lut, m), _np_gemm(np.ascontiguousarray(x.T), g, lut, m))
    # dx[b,k] = sum_u AM(w[k,u], g[b,u]): the weight is the LUT-row operand
    assert eq(oracle.dense_bwd_input(w, g, lut, m), np.ascontiguousarray(_np_gemm(w, np.ascontiguousarray(g.T), lut, m).T))
    a = rng.standard_normal((3, 5, 8)).astype(np.float32)
    b = rng.standard_normal((8, 4)).astype(np.float32)
    c = oracle.matmul(a, b, lut, m)
    for i in range(3):
        assert eq(c[i], _np_gemm(a[i], b, lut, m))
    b3 = rng.standard_normal((3, 8, 4)).astype(np.float32)
    c = oracle.matmul(a[:1], b3, lut, m)
    for i in range(3):
        assert eq(c[i], _np_gemm(a[0], b3[i], lut, m))


def test_ops_regression_fixture(oracle, luts):
    kat = np.load(os.path.join(GOLDEN, "ops_kat.npz"))
    for tag, lname in (("convA", "MBM_7"), ("convB", "MIT_5"), ("convC", "MBM_7")):
        lut, m = luts[lname]
        n, h, w, c, kh, kw, k, s, same = [int(v) for v in kat[tag + "_geom"]]
        g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, "SAME" if same else "VALID")
        assert np.array_equal(oracle.conv2d_fwd(g, kat[tag + "_x"], kat[tag + "_w"], lut, m), kat[tag + "_y"])
        assert np.array_equal(oracle.conv2d_bwd_filter(g, kat[tag + "_x"], kat[tag + "_dy"], lut, m), kat[tag + "_dw"])
        assert np.array_equal(oracle.conv2d_bwd_input(g, kat[tag + "_w"], kat[tag + "_dy"], lut, m), kat[tag + "_dx"])


def test_acc7_small_integers_equal_exact_conv(oracle, luts):
    """The reference's own conv test feeds integers in [-2,2) and compares with
    the exact convolution (test/convam_final_test.py:165-166).  With the
    bf16-exact LUT the only deviation is the AM(0, +-2) quirk (~1e-38)."""
    lut, m = luts["ACC_7"]
    rng = np.random.default_rng(11)
    g = oracle.geometry(2, 8, 8, 3, 3, 3, 4, 1, 1, "SAME")
    x = rng.integers(-2, 2, size=(2, 8, 8, 3)).astype(np.float32)
    w = rng.integers(-2, 2, size=(3, 3, 3, 4)).astype(np.float32)
    y = oracle.conv2d_fwd(g, x, w, lut, m)
    assert np.abs(y - oracle.cpu_conv2d_fwd(g, x, w)).max() < 1e-30


def test_cpu_baseline_loops_agree_with_each_other(oracle):
    """The exact-multiply baseline restatements: gradients agree with
    finite-difference-free identities of the exact convolution."""
    rng = np.random.default_rng(13)
    g = oracle.geometry(2, 7, 6, 3, 3, 3, 5, 2, 2, "SAME")
    x = rng.standard_normal((2, 7, 6, 3)).astype(np.float32)
    w = rng.standard_normal((3, 3, 3, 5)).astype(np.float32)
    dy = rng.standard_normal((2, g.out_h, g.out_w, 5)).astype(np.float32)
    y = oracle.cpu_conv2d_fwd(g, x, w)
    dw = oracle.cpu_conv2d_bwd_filter(g, x, dy)
    dx = oracle.cpu_conv2d_bwd_input(g, w, dy)
    # <y, dy> = <w, dw> = <x, dx> for a bilinear map
    s = float((y.astype(np.float64) * dy).sum())
    assert abs(float((w.astype(np.float64) * dw).sum()) - s) < 1e-3 * abs(s)
    assert abs(float((x.astype(np.float64) * dx).sum()) - s) < 1e-3 * abs(s)


@pytest.mark.parametrize("name", SMALL_LUTS)
def test_lut_primitive_vs_functional_model_sweep(oracle, luts, name):
    """The reference's own LUT check (lut/test.cc:70-101): sweep operands whose
    mantissas carry only the top m bits, compare AMsimulator(LUT) with the
    functional C model the LUT was generated from, skipping pairs with a zero
    exponent field (:84) as that test does.  Where the product is a normal
    number the two must agree bit for bit; outside that range the model clamps
    (subnormal -> 0, overflow -> inf) while the simulator's exponent wraps."""
    from oracle.oracle import RefModel
    if not RefModel.available(name):
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    model = RefModel(name)
    lut, m = luts[name]
    rng = np.random.default_rng(99)
    n = 400_000
    ea = rng.integers(1, 255, size=n, dtype=np.uint32)
    eb = rng.integers(1, 255, size=n, dtype=np.uint32)
    ma = rng.integers(0, 1 << m, size=n, dtype=np.uint32) << np.uint32(23 - m)
    mb = rng.integers(0, 1 << m, size=n, dtype=np.uint32) << np.uint32(23 - m)
    sa = rng.integers(0, 2, size=n, dtype=np.uint32) << np.uint32(31)
    sb = rng.integers(0, 2, size=n, dtype=np.uint32) << np.uint32(31)
    at, bt = sa | (ea << np.uint32(23)) | ma, sb | (eb << np.uint32(23)) | mb
    got = oracle.mul(at.view(np.float32), bt.view(np.float32), lut, m).view(np.uint32)
    want = model.mul_bits_array(at, bt)
    # result exponent of the simulator: ea + eb - 127 + carry must be a normal exponent
    e_sum = ea.astype(np.int64) + eb.astype(np.int64) - 127
    normal = (e_sum >= 2) & (e_sum <= 252)
    assert normal.sum() > n // 4
    mism = (got != want) & normal
    assert not mism.any(), f"{name}: {mism.sum()} mismatches in the normal range, first at {np.argwhere(mism)[0]}"


@pytest.mark.parametrize("name", ["MBM32", "MIT32"])
def test_direct_32bit_models_match_reference(oracle, name):
    """The direct simulation of the 32-bit multipliers (no table) against the
    committed outputs of the reference's cuda/FPmultMBM_fast32.inl /
    cuda/Mitchell_32.inl, and, when oracle/_ref is built, against that code itself
    on four million fresh random operand pairs (all exponent classes, NaN/inf,
    subnormals)."""
    from oracle.oracle import DIRECT_MBM32, DIRECT_MIT32, NO_LUT, RefPrimitive
    m = DIRECT_MBM32 if name == "MBM32" else DIRECT_MIT32
    kat = np.load(os.path.join(GOLDEN, "direct_kat.npz"))
    got = oracle.mul(kat["at"].view(np.float32), kat["bt"].view(np.float32), NO_LUT, m).view(np.uint32)
    assert np.array_equal(got, kat["out_" + name])
    # the approximate product stays within the models' published error of the exact one
    a, b = kat["at"][:16000].view(np.float32), kat["bt"][:16000].view(np.float32)
    exact = a.astype(np.float64) * b.astype(np.float64)
    rel = np.abs(got[:16000].view(np.float32).astype(np.float64) - exact) / np.abs(exact)
    assert rel.max() < (0.09 if name == "MBM32" else 0.12)
    if not RefPrimitive.available():
        pytest.skip("oracle/_ref not built: golden vectors only")
    ref = RefPrimitive()
    rng = np.random.default_rng(5)
    at = rng.integers(0, 1 << 32, size=4_000_000, dtype=np.uint64).astype(np.uint32)
    bt = rng.integers(0, 1 << 32, size=4_000_000, dtype=np.uint64).astype(np.uint32)
    ex = np.array([0, 1, 2, 64, 126, 127, 128, 129, 200, 253, 254, 255], np.uint32)
    at[1::2] = (at[1::2] & np.uint32(0x807FFFFF)) | (rng.choice(ex, size=2_000_000) << np.uint32(23))
    bt[1::2] = (bt[1::2] & np.uint32(0x807FFFFF)) | (rng.choice(ex, size=2_000_000) << np.uint32(23))
    at[::7] |= np.uint32(0x7FFFF0)
    want = ref.direct_mul_bits_array(at, bt, m)
    got = oracle.mul(at.view(np.float32), bt.view(np.float32), NO_LUT, m).view(np.uint32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("name,digest,err", [("MBM_7", "e50d824f5fb99916", 0.02), ("MIT_7", "b29086e212f1ebda", 0.05),
                                             ("ACC_7", "943976896378e5ff", 0.01)])
def test_reference_gemm_known_inputs_checksum(oracle, luts, name, digest, err):
    """The reference's GEMM test case (test/test_gemm.cu:10-15,45-67: A[i][j] = i + j, 800 x 1600;
    B[i][j] = i - j, 1600 x 800).  Its stored outputs are missing from the reference checkout;
    the oracle's result is frozen here by checksum and bounded against the exact product."""
    lut, m = luts[name]
    i, j = np.meshgrid(np.arange(800, dtype=np.float32), np.arange(1600, dtype=np.float32), indexing="ij")
    a = (i + j).astype(np.float32)
    i, j = np.meshgrid(np.arange(1600, dtype=np.float32), np.arange(800, dtype=np.float32), indexing="ij")
    b = (i - j).astype(np.float32)
    c = oracle.matmul(a, b, lut, m)
    assert hashlib.sha256(c.tobytes()).hexdigest()[:16] == digest
    exact = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(c - exact).max() / np.abs(exact).max() < err
