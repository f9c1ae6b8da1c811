"""The product's deterministic mode against the reference's OWN GPU kernels.

oracle/build_ref_cuda.sh compiles the reference's cuda/gemm.cu, cuda/cuda_kernel.cu (im2col
kernels and launchers), cuda/reverseNswapdim23.cu, cuda/denseam_kernel.cu and
cuda/matmulam_kernel.cu unmodified (stand-in TensorFlow / Eigen names only) into
oracle/_ref/libref_cuda.so.  Here both run on the same device tensors: AMSIM_DETERMINISTIC must
be bit-identical to what the reference's kernels write, the CPU oracle must be too (which pins
the oracle to the reference's GPU path at op level), and AMSIM_FAST must be within rel-L2 1e-5.
Small shapes only (the reference materialises the im2col matrix)."""
import numpy as np
import pytest

from conftest import lut_path, rel_l2

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle.oracle import RefCuda
    if not RefCuda.available():
        pytest.skip("oracle/_ref/libref_cuda.so not built (needs a reference checkout at build time)")
    assert torch.cuda.is_available()
    made = {}

    def get(name):
        if name not in made:
            made[name] = RefCuda(lut_path(name))
        return made[name]
    yield get
    for r in made.values():
        r.close()


@pytest.fixture(scope="module")
def ops():
    from approxtrain_b200 import ops as o
    return o


def same_bits(a, b, what):
    a, b = a.detach().cpu().numpy(), (b.detach().cpu().numpy() if hasattr(b, "detach") else np.asarray(b))
    bad = a.view(np.uint32) != b.view(np.uint32)
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} words differ"


CASES = [
    # n, h, w, c, kh, kw, k, stride, padding, lut
    (2, 9, 8, 8, 3, 3, 16, 1, "SAME", "MBM_7"),
    (3, 12, 11, 3, 5, 5, 6, 2, "SAME", "MIT_7"),
    (2, 14, 14, 16, 3, 3, 48, 1, "VALID", "MBM_5"),
    (1, 10, 10, 12, 1, 1, 20, 1, "VALID", "MBM_7"),
    (2, 13, 13, 8, 3, 3, 8, 2, "VALID", "MBM_3"),
    (2, 6, 6, 4, 6, 6, 5, 1, "VALID", "MBM_7"),     # filter as large as the input: the reference's direct-GEMM branch
    (4, 16, 16, 32, 3, 3, 64, 1, "SAME", "MBM_7"),
]


@pytest.mark.parametrize("case", CASES)
def test_conv_deterministic_equals_reference_gpu_kernels(ops, ref, oracle, luts, case):
    n, h, w, c, kh, kw, k, s, pad, lname = case
    r = ref(lname)
    lut, m = luts[lname]
    rng = np.random.default_rng(sum(case[:8]) * 7919)
    x = rng.standard_normal((n, h, w, c)).astype(np.float32)
    x[x < -0.7] = 0.0                                  # zeros: the reference's 0 x (|v| >= 2) residue is exercised
    wt = (rng.standard_normal((kh, kw, c, k)) * 2).astype(np.float32)
    g = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
    dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
    dy[dy < -1.0] = 0.0
    X, W, DY = (torch.from_numpy(a).cuda() for a in (x, wt, dy))
    kw_ = dict(strides=[1, s, s, 1], padding=pad, mant_mul_lut=lut_path(lname))

    y_ref = r.conv2d_fwd(g, X, W, pad == "SAME")
    dw_ref = r.conv2d_bwd_filter(g, X, DY)
    dx_ref = r.conv2d_bwd_input(g, W, DY)
    same_bits(ops.convam(X, W, deterministic=True, **kw_), y_ref, "forward vs reference GPU")
    same_bits(ops.convam_filter_grad(wt.shape, X, DY, deterministic=True, **kw_), dw_ref, "filter gradient vs reference GPU")
    same_bits(ops.convam_input_grad(x.shape, W, DY, deterministic=True, **kw_), dx_ref, "input gradient vs reference GPU")
    # the CPU oracle is the same function
    same_bits(y_ref, oracle.conv2d_fwd(g, x, wt, lut, m), "oracle forward vs reference GPU")
    same_bits(dw_ref, oracle.conv2d_bwd_filter(g, x, dy, lut, m), "oracle filter gradient vs reference GPU")
    same_bits(dx_ref, oracle.conv2d_bwd_input(g, wt, dy, lut, m), "oracle input gradient vs reference GPU")
    # fast mode: within the bar of the reference's GPU result
    for got, want in ((ops.convam(X, W, **kw_), y_ref), (ops.convam_filter_grad(wt.shape, X, DY, **kw_), dw_ref),
                      (ops.convam_input_grad(x.shape, W, DY, **kw_), dx_ref)):
        assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("b,kin,u,lname", [(64, 100, 30, "MBM_7"), (256, 784, 300, "MBM_7"), (7, 33, 5, "MIT_7")])
def test_dense_deterministic_equals_reference_gpu_kernels(ops, ref, oracle, luts, b, kin, u, lname):
    r = ref(lname)
    lut, m = luts[lname]
    rng = np.random.default_rng(b + kin)
    x = rng.random((b, kin)).astype(np.float32)
    x[x < 0.3] = 0
    w = rng.standard_normal((kin, u)).astype(np.float32)
    gy = rng.standard_normal((b, u)).astype(np.float32)
    X, W, G = (torch.from_numpy(a).cuda() for a in (x, w, gy))
    lp = lut_path(lname)
    y_ref = r.dense("fwd", X, W, b, u, kin)
    dw_ref = r.dense("bwd_weight", X, G, b, u, kin)
    dx_ref = r.dense("bwd_input", W, G, b, u, kin)
    same_bits(ops.denseam(X, W, lp, deterministic=True), y_ref, "dense forward vs reference GPU")
    dx, dw = ops.denseam_grad(G, X, W, lp, deterministic=True)
    same_bits(dw, dw_ref, "dense weight gradient vs reference GPU")
    same_bits(dx, dx_ref, "dense input gradient vs reference GPU")
    same_bits(y_ref, oracle.dense_fwd(x, w, lut, m), "oracle dense forward vs reference GPU")
    same_bits(dw_ref, oracle.dense_bwd_weight(x, gy, lut, m), "oracle dense weight gradient vs reference GPU")
    same_bits(dx_ref, oracle.dense_bwd_input(w, gy, lut, m), "oracle dense input gradient vs reference GPU")


@pytest.mark.parametrize("sa,sb", [((16, 24), (24, 8)), ((4, 16, 24), (4, 24, 8)), ((16, 24), (3, 24, 8)), ((3, 16, 24), (24, 8)),
                                   ((5, 16, 24), (1, 24, 8))])
def test_matmul_deterministic_equals_reference_gpu_kernels(ops, ref, sa, sb):
    """Rank and broadcast combinations the reference's launcher serves.  (A first operand of batch 1
    against a larger second batch is left out: cuda/matmulam_kernel.cu:62-72 loops over batch_a
    there and so writes only the first product.)"""
    r = ref("MBM_7")
    rng = np.random.default_rng(len(sa) * 10 + len(sb))
    A = torch.from_numpy(rng.standard_normal(sa).astype(np.float32)).cuda()
    B = torch.from_numpy(rng.standard_normal(sb).astype(np.float32)).cuda()
    same_bits(ops.matmulam(A, B, mant_mul_lut=lut_path("MBM_7"), deterministic=True), r.matmul(A, B), f"matmul {sa} x {sb}")
