"""Mantissa-LUT generator: turns a functional model of an approximate FP32
multiplier into the ``<MODEL>_<m>.bin`` file the ops load.

Same procedure and file format as the reference's ``lut/lut_gen.cc:86-127``:
for every pair (i, j) of m-bit mantissa prefixes the model multiplies
``1.i x 1.j`` (both at biased exponent 127); the entry is one byte,
``carry | mantissa`` with ``mantissa`` = the top m mantissa bits of the product
(truncated to 8 bits, as the reference's ``uint8_t`` does) and ``carry = 0x80``
when the product's exponent exceeds 127.  Entry order: ``i * 2^m + j``.

The model is any callable on float32 arrays, or a C function
``float f(float, float)`` in a shared library (the flow developer.md:38-87 of
the reference describes for adding a multiplier: write the C model, generate
the LUT, name it ``<MODEL>_<m>.bin``).

    python -m approxtrain_b200.lutgen libmymul.so my_mul 7 MYMUL_7.bin
"""
from __future__ import annotations

import ctypes as C
import sys
from typing import Callable

import numpy as np


def generate(model: Callable[[np.ndarray, np.ndarray], np.ndarray], m: int, entry_bits: int = 8) -> np.ndarray:
    """Return the 2^(2m) LUT entries for ``model`` (vectorised: float32 arrays in, float32 array out).

    ``entry_bits=8`` is the reference's format (uint8 array).  ``entry_bits=16`` is a format
    extension of this library (little-endian uint16 array, written to a file of twice the
    size under the same ``<MODEL>_<m>.bin`` name): ``carry << 15 | top 15 mantissa bits`` of
    the product.  A byte keeps 7 mantissa bits, so tables for m = 8..11 in the reference's
    format drop the product's leading mantissa bits; 16-bit entries keep them."""
    if not 1 <= m <= 11:
        raise ValueError("mantissa width must be in 1..11 (the ops derive a_shift = 23 - 2m)")
    if entry_bits not in (8, 16):
        raise ValueError("entry_bits must be 8 or 16")
    n = 1 << m
    i, j = np.meshgrid(np.arange(n, dtype=np.uint32), np.arange(n, dtype=np.uint32), indexing="ij")
    one = np.uint32(0x3F800000)
    a = (one | (i << np.uint32(23 - m))).view(np.float32)
    b = (one | (j << np.uint32(23 - m))).view(np.float32)
    c = np.ascontiguousarray(model(a.reshape(-1), b.reshape(-1)), dtype=np.float32).view(np.uint32)
    if entry_bits == 16:
        mant = ((c >> np.uint32(8)) & np.uint32(0x7FFF)).astype(np.uint16)
        carry = np.where((c & np.uint32(0x7F800000)) > one, 0x8000, 0).astype(np.uint16)
        return (carry | mant).astype("<u2")
    mask = np.uint32(((1 << m) - 1) << (23 - m))
    mant = ((c & mask) >> np.uint32(23 - m)).astype(np.uint8)          # truncation to uint8 as in lut_gen.cc:114
    carry = np.where((c & np.uint32(0x7F800000)) > one, 0x80, 0).astype(np.uint8)
    return (carry | mant).astype(np.uint8)


def c_model(library: str, symbol: str) -> Callable[[np.ndarray, np.ndarray], np.ndarray]:
    """Wrap ``float symbol(float, float)`` from a shared library as a vectorised model."""
    fn = getattr(C.CDLL(library), symbol)
    fn.argtypes = [C.c_float, C.c_float]
    fn.restype = C.c_float

    def model(a: np.ndarray, b: np.ndarray) -> np.ndarray:
        out = np.empty(a.shape, np.float32)
        for k in range(a.size):
            out[k] = fn(float(a[k]), float(b[k]))
        return out
    return model


def write(path: str, model: Callable, m: int, entry_bits: int = 8) -> None:
    import os
    import re
    mm = re.search(r"_(\d+)\.[^._/]*$", os.path.basename(path))
    if not mm or int(mm.group(1)) != m:
        raise ValueError(f"{path!r}: the ops read the mantissa width from the file name, it must end in _{m}.<ext>")
    generate(model, m, entry_bits).tofile(path)


if __name__ == "__main__":
    if len(sys.argv) != 5:
        sys.exit(__doc__)
    lib, sym, width, out = sys.argv[1], sys.argv[2], int(sys.argv[3]), sys.argv[4]
    write(out, c_model(lib, sym), width)
    print(f"wrote {out}: {1 << (2 * width)} bytes")
