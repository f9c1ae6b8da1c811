"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
header declares, and its host-only logic (LUT name/size validation, window
geometry, constant division) behaves.  No kernel is launched."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import ROOT, lut_path


@pytest.fixture(scope="module")
def L():
    from approxtrain_b200 import _build
    _build.build()
    from approxtrain_b200 import _lib
    return _lib


def test_every_declared_symbol_is_exported(L):
    header = open(os.path.join(ROOT, "include", "amsim.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(amsim_[a-z0-9_]+)\s*\(", header))
    assert declared == set(L.EXPORTS)
    for name in declared:
        assert hasattr(L.lib, name), name


def test_lut_open_rejects_bad_names_before_touching_cuda(L, tmp_path):
    h = C.c_void_p()
    for bad in ("MBM.bin", "MBM_.bin", "MBM_x7.bin", "MBM_12.bin", "MBM_0.bin", "MBM_7"):
        assert L.lib.amsim_lut_open(str(tmp_path / bad).encode(), 0, C.byref(h)) == L.ERR_LUT_NAME
    assert L.lib.amsim_lut_open(b"", 0, C.byref(h)) == L.ERR_LUT_NAME
    assert b"no mant lut file name given" in L.lib.amsim_last_error()
    assert L.lib.amsim_lut_open(str(tmp_path / "missing_7.bin").encode(), 0, C.byref(h)) == L.ERR_LUT_IO
    assert L.lib.amsim_lut_open(None, 0, C.byref(h)) == L.ERR_INVALID


def test_lut_open_rejects_wrong_size(L, tmp_path):
    h = C.c_void_p()
    short = tmp_path / "SHORT_3.bin"
    short.write_bytes(bytes(63))
    assert L.lib.amsim_lut_open(str(short).encode(), 0, C.byref(h)) == L.ERR_LUT_SIZE
    long = tmp_path / "LONG_3.bin"
    long.write_bytes(bytes(65))
    assert L.lib.amsim_lut_open(str(long).encode(), 0, C.byref(h)) == L.ERR_LUT_SIZE
    assert b"exactly 64" in L.lib.amsim_last_error()


def test_geometry_matches_oracle(L, oracle):
    rng = np.random.default_rng(0)
    for _ in range(300):
        h, w = int(rng.integers(1, 40)), int(rng.integers(1, 40))
        kh, kw = int(rng.integers(1, 8)), int(rng.integers(1, 8))
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        for same in (0, 1):
            if not same and (kh > h or kw > w):
                continue
            oh, ow, pt, pl = C.c_int(), C.c_int(), C.c_int(), C.c_int()
            assert L.lib.amsim_conv2d_geometry(h, w, kh, kw, sh, sw, same, C.byref(oh), C.byref(ow), C.byref(pt), C.byref(pl)) == 0
            g = oracle.geometry(1, h, w, 1, kh, kw, 1, sh, sw, "SAME" if same else "VALID")
            assert (oh.value, ow.value, pt.value, pl.value) == (g.out_h, g.out_w, g.pad_top, g.pad_left)
    assert L.lib.amsim_conv2d_geometry(3, 3, 5, 5, 1, 1, 0, None, None, None, None) == L.ERR_INVALID


def test_geometry_same_padding_equals_reference_offset_formula():
    """filter_top_offset of convam.cc:565-571: ((out-1)*s + k - in) / 2, floored at 0."""
    from approxtrain_b200.ops import conv2d_geometry
    for (i, k, s) in [(56, 3, 1), (224, 7, 2), (28, 5, 1), (55, 3, 2), (7, 3, 2), (8, 3, 2)]:
        oh, _, pt, _ = conv2d_geometry(i, i, k, k, s, s, "SAME")
        assert oh == -(-i // s)
        assert pt == max(((oh - 1) * s + k - i) // 2, 0)


def test_fastdiv_matches_integer_division(L):
    rng = np.random.default_rng(1)
    ds = [1, 2, 3, 5, 7, 9, 49, 64, 196, 576, 3136, 12544, 200704, 2**20 + 1, 2**30]
    ns = list(rng.integers(0, 2**31 - 1, size=400)) + [0, 1, 2**31 - 1, 2**31 - 2]
    for d in ds:
        for n in ns + [d - 1, d, d + 1, 2 * d - 1, 2 * d]:
            n = int(n) % (2**31)
            assert L.lib.amsim_debug_fastdiv(n, d) == n // d, (n, d)


def test_ops_reject_cpu_tensors_and_bad_arguments(L):
    import torch
    from approxtrain_b200 import ops
    x = torch.zeros(1, 4, 4, 2)
    w = torch.zeros(3, 3, 2, 2)
    with pytest.raises(ValueError, match="CUDA"):
        ops.convam(x, w, [1, 1, 1, 1], "SAME", mant_mul_lut=lut_path("MBM_7"))
    with pytest.raises(ValueError, match="Matmulam unsupported args"):
        ops.matmulam(x, w, adjoint_a=True, mant_mul_lut=lut_path("MBM_7"))
    with pytest.raises(ValueError, match="Dilation is not supported"):
        ops._check_format("NHWC", [1, 2, 2, 1])
    assert ops._hw([1, 2, 3, 1], "strides") == (2, 3)
    with pytest.raises(ValueError):
        ops._hw([2, 1, 1, 1], "strides")


def test_header_is_valid_c99_and_cxx11():
    """include/amsim.h is the whole boundary: it has to compile as C and as C++ on its own."""
    import subprocess
    hdr = os.path.join(ROOT, "include", "amsim.h")
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-x", "c", hdr])
    subprocess.check_call(["g++", "-std=c++11", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", hdr])
