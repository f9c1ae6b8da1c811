"""The bounds-checking debug build of the library (libamsim_check.so, -DAMSIM_BOUNDS_CHECK) on the
tiny, ragged, strided and padded shapes: every access the kernels make to a tensor or to scratch
is compared with that buffer's extent and alignment before it is made (a device-side memory
checker is not available where these tests run).  A child process loads that build instead of the
normal one (AMSIM_LIBRARY), runs the cases in every mode against the CPU oracle and reads the
verdict after each: no access may have been out of bounds.  One more case shortens the recorded
extent of the output by 64 bytes on purpose and expects the checker to catch, and skip, the last
stores: the checker itself works, and the process stays healthy because a flagged access is never made.
"""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

CHILD = r'''
import ctypes as C, os, sys, zlib
import numpy as np, torch
sys.path.insert(0, os.environ["AMSIM_REPO"]); sys.path.insert(0, os.path.join(os.environ["AMSIM_REPO"], "tests"))
from approxtrain_b200 import ops, _lib
from oracle.oracle import Oracle, load_lut
from conftest import lut_path, rel_l2
assert _lib.lib._name.endswith("libamsim_check.so"), _lib.lib._name
o = Oracle.get()
def verdict():
    w = C.c_ulonglong(0)
    assert _lib.lib.amsim_debug_bounds_report(C.byref(w)) == 0, _lib.lib.amsim_last_error()
    return w.value
def dev(a): return torch.from_numpy(np.ascontiguousarray(a)).cuda()
assert verdict() == 0
SHAPES = [(2, 9, 8, 8, 3, 3, 16), (1, 12, 12, 4, 3, 3, 70), (2, 7, 7, 3, 3, 3, 5), (3, 10, 11, 1, 5, 5, 6), (2, 6, 6, 6, 5, 5, 16),
          (1, 8, 8, 16, 1, 1, 32), (2, 5, 5, 8, 5, 5, 8), (5, 17, 19, 12, 3, 2, 24), (4, 10, 10, 32, 3, 3, 40), (2, 11, 11, 64, 1, 1, 256)]
n_cases = 0
for wide in ("-1", "1"):
    os.environ["AMSIM_WIDE"] = wide
    _lib.lib.amsim_debug_reload_env()
    for shape in SHAPES:
        n, h, w, c, kh, kw, k = shape
        for stride in (1, 2):
            for pad in ("SAME", "VALID"):
                if pad == "VALID" and (kh > h or kw > w):
                    continue
                for lname in ("MBM_7", "MIT_7"):
                    lut, m = load_lut(lut_path(lname))
                    rng = np.random.default_rng(zlib.crc32(repr((shape, stride, pad, lname)).encode()))
                    x = rng.standard_normal((n, h, w, c)).astype(np.float32); x[x < -0.5] = 0
                    wt = rng.standard_normal((kh, kw, c, k)).astype(np.float32)
                    g = o.geometry(n, h, w, c, kh, kw, k, stride, stride, pad)
                    dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
                    kw_ = dict(strides=[1, stride, stride, 1], padding=pad, mant_mul_lut=lut_path(lname))
                    refs = (o.conv2d_fwd(g, x, wt, lut, m), o.conv2d_bwd_filter(g, x, dy, lut, m), o.conv2d_bwd_input(g, wt, dy, lut, m))
                    for det in (True, False):
                        outs = (ops.convam(dev(x), dev(wt), deterministic=det, **kw_),
                                ops.convam_filter_grad(wt.shape, dev(x), dev(dy), deterministic=det, **kw_),
                                ops.convam_input_grad(x.shape, dev(wt), dev(dy), deterministic=det, **kw_))
                        v = verdict()
                        assert v == 0, f"out-of-bounds access: line {v >> 44} buffer {((v >> 40) & 15) - 1} offset {v & ((1 << 40) - 1)} in {shape} s{stride} {pad} {lname} det={det} wide={wide}"
                        for got, want in zip(outs, refs):
                            got = got.cpu().numpy()
                            if det:
                                assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
                            else:
                                assert rel_l2(got, want) <= 1e-5
                        n_cases += 1
# dense layers and batched products
lut, m = load_lut(lut_path("MBM_7")); lp = lut_path("MBM_7")
rng = np.random.default_rng(1)
for b, kin, u in ((7, 33, 5), (130, 64, 129), (256, 100, 10), (1, 1, 1), (300, 64, 72)):
    x = rng.random((b, kin)).astype(np.float32); wm = rng.standard_normal((kin, u)).astype(np.float32)
    gy = rng.standard_normal((b, u)).astype(np.float32)
    for det in (True, False):
        ops.denseam(dev(x), dev(wm), lp, deterministic=det); ops.denseam_grad(dev(gy), dev(x), dev(wm), lp, deterministic=det)
        assert verdict() == 0
for sa, sb, ta, tb in (((4, 16, 24), (4, 24, 8), False, False), ((16, 24), (3, 24, 8), False, False), ((3, 24, 16), (3, 8, 24), True, True),
                       ((6, 130, 64), (6, 70, 64), False, True)):
    a = dev(rng.standard_normal(sa).astype(np.float32)); bb = dev(rng.standard_normal(sb).astype(np.float32))
    for det in (True, False):
        ops.matmulam(a, bb, transpose_a=ta, transpose_b=tb, mant_mul_lut=lp, deterministic=det)
        assert verdict() == 0
# the checker's own test: the output's recorded extent is 64 bytes short, so the last stores must be caught
os.environ["AMSIM_BOUNDS_SHRINK"] = "64"; os.environ["AMSIM_WIDE"] = "-1"
_lib.lib.amsim_debug_reload_env()
x = dev(rng.standard_normal((2, 9, 8, 8)).astype(np.float32)); wt = dev(rng.standard_normal((3, 3, 8, 16)).astype(np.float32))
ops.convam(x, wt, strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=lp)
v = verdict()
assert v != 0 and ((v >> 40) & 15) - 1 == 2, hex(v)      # buffer 2 = the output
del os.environ["AMSIM_BOUNDS_SHRINK"]
_lib.lib.amsim_debug_reload_env()
ops.convam(x, wt, strides=[1, 1, 1, 1], padding="SAME", mant_mul_lut=lp)
assert verdict() == 0
print(f"bounds-checked cases: {n_cases}, all accesses in bounds; checker self-test caught the shortened output")
'''


def test_bounds_checking_build_sees_no_out_of_range_access():
    assert torch.cuda.is_available()
    from approxtrain_b200 import _build
    if not os.path.exists(_build.CHECKED_LIB_PATH):
        pytest.skip("libamsim_check.so not built (approxtrain_b200._build.build_checked)")
    env = dict(os.environ, AMSIM_LIBRARY=_build.CHECKED_LIB_PATH, AMSIM_REPO=ROOT)
    out = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=1500, env=env, cwd=ROOT)
    assert out.returncode == 0, (out.stdout + out.stderr)[-4000:]
    assert "all accesses in bounds" in out.stdout
    print(out.stdout.strip().splitlines()[-1])
