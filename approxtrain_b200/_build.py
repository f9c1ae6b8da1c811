"""Compiles the CUDA library for sm_100a into the package directory.

The shared object is built in-tree (``approxtrain_b200/libamsim.so``) with nvcc;
there is no other backend and no fallback.
"""
from __future__ import annotations

import os
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libamsim.so")
SOURCES = [os.path.join(_PKG, "csrc", "amsim.cu")]
HEADERS = [os.path.join(_PKG, "csrc", "amsim_kernels.cuh"),
           os.path.join(os.path.dirname(_PKG), "include", "amsim.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.exists(f) and os.path.getmtime(f) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Build libamsim.so if it is missing or older than its sources."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + SOURCES
    subprocess.check_call(cmd)
    return LIB_PATH


if __name__ == "__main__":
    build(force=True, verbose=True)
    print(LIB_PATH)
