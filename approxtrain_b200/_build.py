"""Compiles the CUDA library for sm_100a into the package directory.

The shared object is built in-tree (``approxtrain_b200/libamsim.so``) with nvcc;
there is no other backend and no fallback.
"""
from __future__ import annotations

import os
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB_PATH = os.path.join(_PKG, "libamsim.so")
# AMSIM_LIBRARY: load another build of the same library instead, e.g. the bounds-checking debug
# build libamsim_check.so (build_checked below); it is never rebuilt automatically.
LIB_PATH = os.environ.get("AMSIM_LIBRARY") or DEFAULT_LIB_PATH
CHECKED_LIB_PATH = os.path.join(_PKG, "libamsim_check.so")
SOURCES = [os.path.join(_PKG, "csrc", "amsim.cu")]
HEADERS = [os.path.join(_PKG, "csrc", "amsim_kernels.cuh"), os.path.join(_PKG, "csrc", "amsim_wide.cuh"),
           os.path.join(os.path.dirname(_PKG), "include", "amsim.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def needs_build() -> bool:
    if LIB_PATH != DEFAULT_LIB_PATH:
        return False
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.exists(f) and os.path.getmtime(f) > t for f in SOURCES + HEADERS)


DRIVER_SRC = os.path.join(_PKG, "csrc", "abi_driver.c")
DRIVER_PATH = os.path.join(_PKG, "abi_driver")


def build_driver() -> str:
    """The plain-C program over the C ABI (csrc/abi_driver.c): gcc, the header, libamsim.so
    and the CUDA runtime for its device buffers.  Proves the header is C and the library
    usable without Python or C++."""
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.check_call([
        os.environ.get("CC", "gcc"), "-std=c99", "-O1", "-Wall", "-o", DRIVER_PATH, DRIVER_SRC,
        "-I", os.path.join(os.path.dirname(_PKG), "include"), "-I", os.path.join(cuda, "include"),
        "-L", _PKG, "-lamsim", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lm",
        "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda, "lib64")])
    return DRIVER_PATH


def build_checked(force: bool = False) -> str:
    """The bounds-checking debug build (libamsim_check.so, -DAMSIM_BOUNDS_CHECK): every kernel access
    to a tensor or to scratch is checked against the buffer's extent before it is made.  Loaded with
    AMSIM_LIBRARY=<path>; read the verdict with amsim_debug_bounds_report()."""
    if force or not os.path.exists(CHECKED_LIB_PATH) or any(
            os.path.getmtime(f) > os.path.getmtime(CHECKED_LIB_PATH) for f in SOURCES + HEADERS if os.path.exists(f)):
        nvcc = os.environ.get("NVCC", "nvcc")
        subprocess.check_call([nvcc] + NVCC_FLAGS + ["-DAMSIM_BOUNDS_CHECK", "-o", CHECKED_LIB_PATH] + SOURCES)
    return CHECKED_LIB_PATH


def build(force: bool = False, verbose: bool = False) -> str:
    """Build libamsim.so (and the C driver) if missing or older than the sources."""
    if force or needs_build():
        nvcc = os.environ.get("NVCC", "nvcc")
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", DEFAULT_LIB_PATH] + SOURCES
        subprocess.check_call(cmd)
    if force or not os.path.exists(DRIVER_PATH) or os.path.getmtime(DRIVER_PATH) < max(
            os.path.getmtime(DRIVER_SRC), os.path.getmtime(DEFAULT_LIB_PATH)):
        build_driver()
    return LIB_PATH


if __name__ == "__main__":
    build(force=True, verbose=True)
    print(LIB_PATH)
