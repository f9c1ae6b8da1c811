"""ctypes binding of the CPU oracle (``oracle/libamsim_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, the smoke check and the
benchmark's CPU-baseline leg.  The product package never imports this module.

``Oracle`` wraps the C restatement (amsim_oracle.c); ``RefPrimitive`` wraps the
reference's own ``cuda/AMsimulator.inl`` compiled as host C++ by
``oracle/build.sh`` (``oracle/_ref/libref_amsim.so``), when that file exists.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libamsim_oracle.so")
_REF_LIB = os.path.join(_HERE, "_ref", "libref_amsim.so")

# Pseudo mantissa widths selecting the direct 32-bit models (amsim_oracle.h); pass NO_LUT as the table.
DIRECT_MBM32 = 132
DIRECT_MIT32 = 123
NO_LUT = np.zeros(1, dtype=np.uint8)
WIDE_ENTRIES = 0x100   # m | WIDE_ENTRIES: the table holds 16-bit little-endian entries (pass the bytes)

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")


class _Geom(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "batch", "in_h", "in_w", "in_c", "f_h", "f_w", "out_c", "out_h", "out_w",
        "stride_h", "stride_w", "pad_top", "pad_left")]


@dataclass
class ConvGeom:
    batch: int
    in_h: int
    in_w: int
    in_c: int
    f_h: int
    f_w: int
    out_c: int
    out_h: int
    out_w: int
    stride_h: int
    stride_w: int
    pad_top: int
    pad_left: int

    def _c(self) -> _Geom:
        return _Geom(*[getattr(self, n) for n, _ in _Geom._fields_])


def build(force: bool = False) -> None:
    """Compile the oracle (and oracle/_ref when a reference checkout exists)."""
    if force or not os.path.exists(_LIB):
        subprocess.check_call(["bash", os.path.join(_HERE, "build.sh")])


def load_lut(path: str):
    """Return (bytes as uint8 array, m) — approx_mul_lut.h:15-45."""
    o = Oracle.get()
    m = o.lib.am_parse_mant_width(path.encode())
    if m < 0:
        raise ValueError(f"cannot parse mantissa width from {path!r}")
    data = np.fromfile(path, dtype=np.uint8)
    if data.size == 2 << (2 * m):      # 16-bit entries (format extension)
        return data, m | WIDE_ENTRIES
    if data.size != 1 << (2 * m):
        raise ValueError(f"{path}: {data.size} bytes, expected {1 << (2 * m)}")
    return data, m


class Oracle:
    _inst = None

    @classmethod
    def get(cls) -> "Oracle":
        if cls._inst is None:
            cls._inst = cls()
        return cls._inst

    def __init__(self):
        build()
        L = self.lib = C.CDLL(_LIB)
        L.am_parse_mant_width.argtypes = [C.c_char_p]
        L.am_parse_mant_width.restype = C.c_int
        L.am_mul_bits.argtypes = [C.c_uint32, C.c_uint32, _u8p, C.c_int]
        L.am_mul_bits.restype = C.c_uint32
        L.am_mul_array.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, _u8p, C.c_int]
        L.am_gemm.argtypes = [C.c_int] * 3 + [_f32p, C.c_int, _f32p, C.c_int, _f32p, C.c_int, _u8p, C.c_int]
        L.am_conv_geometry.argtypes = [C.c_int] * 10 + [C.POINTER(_Geom)]
        for name in ("am_conv2d_fwd", "am_conv2d_bwd_filter", "am_conv2d_bwd_input"):
            getattr(L, name).argtypes = [C.POINTER(_Geom), _f32p, _f32p, _f32p, _u8p, C.c_int]
        for name in ("cpu_conv2d_fwd", "cpu_conv2d_bwd_filter", "cpu_conv2d_bwd_input"):
            getattr(L, name).argtypes = [C.POINTER(_Geom), _f32p, _f32p, _f32p]
        for name in ("am_dense_fwd", "am_dense_bwd_weight", "am_dense_bwd_input"):
            getattr(L, name).argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, _u8p, C.c_int]
        for name in ("cpu_dense_fwd", "cpu_dense_bwd_weight", "cpu_dense_bwd_input"):
            getattr(L, name).argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.am_matmul.argtypes = [_f32p, _f32p, _f32p] + [C.c_int] * 5 + [_u8p, C.c_int]
        L.cpu_gemm.argtypes = [C.c_int] * 3 + [_f32p, C.c_int, _f32p, C.c_int, _f32p, C.c_int]
        L.am_oracle_set_threads.argtypes = [C.c_int]
        i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
        L.am_gemm_i32.argtypes = [C.c_int] * 3 + [i32p, C.c_int, i32p, C.c_int, i32p, C.c_int, _u8p, C.c_int]
        for name in ("am_conv2d_fwd_i32", "am_conv2d_bwd_filter_i32", "am_conv2d_bwd_input_i32"):
            getattr(L, name).argtypes = [C.POINTER(_Geom), i32p, i32p, i32p, _u8p, C.c_int]

    # -- primitive ---------------------------------------------------------
    def mul_bits(self, at: int, bt: int, lut: np.ndarray, m: int) -> int:
        return int(self.lib.am_mul_bits(at, bt, lut, m))

    def mul(self, a: np.ndarray, b: np.ndarray, lut: np.ndarray, m: int) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        out = np.empty_like(a)
        self.lib.am_mul_array(a.reshape(-1), b.reshape(-1), out.reshape(-1), a.size, lut, m)
        return out

    # -- geometry ----------------------------------------------------------
    def geometry(self, batch, in_h, in_w, in_c, f_h, f_w, out_c, stride_h, stride_w, padding) -> ConvGeom:
        g = _Geom()
        same = 1 if str(padding).upper() == "SAME" else 0
        self.lib.am_conv_geometry(batch, in_h, in_w, in_c, f_h, f_w, out_c, stride_h, stride_w, same, C.byref(g))
        return ConvGeom(*[getattr(g, n) for n, _ in _Geom._fields_])

    # -- ops (reference GPU semantics: AM multiply, reference order) --------
    def gemm(self, A, B, lut, m):
        A = np.ascontiguousarray(A, np.float32)
        B = np.ascontiguousarray(B, np.float32)
        out = np.empty((A.shape[0], B.shape[1]), np.float32)
        self.lib.am_gemm(A.shape[0], B.shape[1], A.shape[1], A.reshape(-1), A.shape[1],
                         B.reshape(-1), B.shape[1], out.reshape(-1), B.shape[1], lut, m)
        return out

    def conv2d_fwd(self, g: ConvGeom, x, w, lut, m):
        y = np.empty((g.batch, g.out_h, g.out_w, g.out_c), np.float32)
        gc = g._c()
        self.lib.am_conv2d_fwd(C.byref(gc), _flat(x), _flat(w), y.reshape(-1), lut, m)
        return y

    def conv2d_bwd_filter(self, g: ConvGeom, x, dy, lut, m):
        dw = np.empty((g.f_h, g.f_w, g.in_c, g.out_c), np.float32)
        gc = g._c()
        self.lib.am_conv2d_bwd_filter(C.byref(gc), _flat(x), _flat(dy), dw.reshape(-1), lut, m)
        return dw

    def conv2d_bwd_input(self, g: ConvGeom, w, dy, lut, m):
        dx = np.empty((g.batch, g.in_h, g.in_w, g.in_c), np.float32)
        gc = g._c()
        self.lib.am_conv2d_bwd_input(C.byref(gc), _flat(w), _flat(dy), dx.reshape(-1), lut, m)
        return dx

    def dense_fwd(self, x, w, lut, m):
        b, k = x.shape
        u = w.shape[1]
        y = np.empty((b, u), np.float32)
        self.lib.am_dense_fwd(_flat(x), _flat(w), y.reshape(-1), b, u, k, lut, m)
        return y

    def dense_bwd_weight(self, x, g, lut, m):
        b, k = x.shape
        u = g.shape[1]
        dw = np.empty((k, u), np.float32)
        self.lib.am_dense_bwd_weight(_flat(x), _flat(g), dw.reshape(-1), b, u, k, lut, m)
        return dw

    def dense_bwd_input(self, w, g, lut, m):
        k, u = w.shape
        b = g.shape[0]
        dx = np.empty((b, k), np.float32)
        self.lib.am_dense_bwd_input(_flat(w), _flat(g), dx.reshape(-1), b, u, k, lut, m)
        return dx

    def matmul(self, a, b, lut, m):
        """a: [M,K] or [Ba,M,K]; b: [K,N] or [Bb,K,N] (matmulam.cc:86-147)."""
        ba = a.shape[0] if a.ndim == 3 else 0
        bb = b.shape[0] if b.ndim == 3 else 0
        M, K = a.shape[-2:]
        N = b.shape[-1]
        nb = max(ba, bb)
        out = np.empty((nb, M, N) if nb else (M, N), np.float32)
        self.lib.am_matmul(_flat(a), _flat(b), out.reshape(-1), ba, bb, M, K, N, lut, m)
        return out

    # -- T = int32 ----------------------------------------------------------
    def gemm_i32(self, A, B, lut, m):
        A = np.ascontiguousarray(A, np.int32)
        B = np.ascontiguousarray(B, np.int32)
        out = np.empty((A.shape[0], B.shape[1]), np.int32)
        self.lib.am_gemm_i32(A.shape[0], B.shape[1], A.shape[1], A.reshape(-1), A.shape[1],
                             B.reshape(-1), B.shape[1], out.reshape(-1), B.shape[1], lut, m)
        return out

    def conv2d_i32(self, which, g: ConvGeom, p, q, lut, m):
        shape = {"fwd": (g.batch, g.out_h, g.out_w, g.out_c), "bwd_filter": (g.f_h, g.f_w, g.in_c, g.out_c),
                 "bwd_input": (g.batch, g.in_h, g.in_w, g.in_c)}[which]
        out = np.empty(shape, np.int32)
        gc = g._c()
        getattr(self.lib, f"am_conv2d_{which}_i32")(C.byref(gc), np.ascontiguousarray(p, np.int32).reshape(-1),
                                                    np.ascontiguousarray(q, np.int32).reshape(-1), out.reshape(-1), lut, m)
        return out

    # -- reference CPU op path (exact multiply; timing baseline) ------------
    def cpu_conv2d_fwd(self, g: ConvGeom, x, w):
        y = np.empty((g.batch, g.out_h, g.out_w, g.out_c), np.float32)
        gc = g._c()
        self.lib.cpu_conv2d_fwd(C.byref(gc), _flat(x), _flat(w), y.reshape(-1))
        return y

    def cpu_conv2d_bwd_filter(self, g: ConvGeom, x, dy):
        dw = np.empty((g.f_h, g.f_w, g.in_c, g.out_c), np.float32)
        gc = g._c()
        self.lib.cpu_conv2d_bwd_filter(C.byref(gc), _flat(x), _flat(dy), dw.reshape(-1))
        return dw

    def cpu_conv2d_bwd_input(self, g: ConvGeom, w, dy):
        dx = np.empty((g.batch, g.in_h, g.in_w, g.in_c), np.float32)
        gc = g._c()
        self.lib.cpu_conv2d_bwd_input(C.byref(gc), _flat(w), _flat(dy), dx.reshape(-1))
        return dx

    def cpu_dense(self, which, p, q, batch, units, in_w):
        shape = {"fwd": (batch, units), "bwd_weight": (in_w, units), "bwd_input": (batch, in_w)}[which]
        out = np.empty(shape, np.float32)
        getattr(self.lib, f"cpu_dense_{which}")(_flat(p), _flat(q), out.reshape(-1), batch, units, in_w)
        return out

    def cpu_gemm(self, A, B):
        A = np.ascontiguousarray(A, np.float32)
        B = np.ascontiguousarray(B, np.float32)
        out = np.empty((A.shape[0], B.shape[1]), np.float32)
        self.lib.cpu_gemm(A.shape[0], B.shape[1], A.shape[1], A.reshape(-1), A.shape[1],
                          B.reshape(-1), B.shape[1], out.reshape(-1), B.shape[1])
        return out

    def set_threads(self, n: int) -> None:
        self.lib.am_oracle_set_threads(n)


def _flat(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


class RefPrimitive:
    """The reference's own cuda/AMsimulator.inl, built as host code."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(_REF_LIB)

    def __init__(self):
        if not self.available():
            raise FileNotFoundError(_REF_LIB)
        L = self.lib = C.CDLL(_REF_LIB)
        L.ref_am_mul_bits.argtypes = [C.c_uint32, C.c_uint32, _u8p, C.c_int]
        L.ref_am_mul_bits.restype = C.c_uint32
        L.ref_am_mul_bits_array.argtypes = [_u32p, _u32p, _u32p, C.c_uint64, _u8p, C.c_int]

    def mul_bits_array(self, at: np.ndarray, bt: np.ndarray, lut: np.ndarray, m: int) -> np.ndarray:
        at = np.ascontiguousarray(at, np.uint32).reshape(-1)
        bt = np.ascontiguousarray(bt, np.uint32).reshape(-1)
        out = np.empty_like(at)
        self.lib.ref_am_mul_bits_array(at, bt, out, at.size, lut, m)
        return out

    def direct_mul_bits_array(self, at: np.ndarray, bt: np.ndarray, m: int) -> np.ndarray:
        """The reference's cuda/FPmultMBM_fast32.inl (m = DIRECT_MBM32) or
        cuda/Mitchell_32.inl (m = DIRECT_MIT32) on raw bit patterns."""
        at = np.ascontiguousarray(at, np.uint32).reshape(-1)
        bt = np.ascontiguousarray(bt, np.uint32).reshape(-1)
        out = np.empty_like(at)
        self.lib.ref_direct_mul_bits_array.argtypes = [_u32p, _u32p, _u32p, C.c_uint64, C.c_int]
        self.lib.ref_direct_mul_bits_array(at, bt, out, at.size, 1 if m == DIRECT_MBM32 else 0)
        return out


class RefModel:
    """One of the reference's functional multiplier models (the C code a shipped
    LUT was generated from), built as host code by oracle/build.sh."""

    def __init__(self, lut_name: str):
        path = os.path.join(_HERE, "_ref", f"libref_model_{lut_name}.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        self.lib.ref_model_mul_array.argtypes = [_u32p, _u32p, _u32p, C.c_uint64]

    @staticmethod
    def available(lut_name: str) -> bool:
        return os.path.exists(os.path.join(_HERE, "_ref", f"libref_model_{lut_name}.so"))

    def mul_bits_array(self, at: np.ndarray, bt: np.ndarray) -> np.ndarray:
        at = np.ascontiguousarray(at, np.uint32).reshape(-1)
        bt = np.ascontiguousarray(bt, np.uint32).reshape(-1)
        out = np.empty_like(at)
        self.lib.ref_model_mul_array(at, bt, out, at.size)
        return out


class RefCuda:
    """The reference's own GPU functors, compiled unmodified from a reference checkout by
    oracle/build_ref_cuda.sh (oracle/_ref/libref_cuda.so).  Takes and returns torch CUDA
    tensors; every call synchronises the device, as the reference does.  Checker only."""

    _LIB = os.path.join(_HERE, "_ref", "libref_cuda.so")

    @staticmethod
    def available() -> bool:
        return os.path.exists(RefCuda._LIB)

    def __init__(self, lut_path: str):
        L = self.lib = C.CDLL(self._LIB)
        vp, ip = C.c_void_p, C.c_int
        L.ref_cuda_lut_open.argtypes = [C.c_char_p]
        L.ref_cuda_lut_open.restype = vp
        L.ref_cuda_lut_close.argtypes = [vp]
        L.ref_cuda_conv2d_fwd.argtypes = [vp] * 5 + [ip] * 14
        L.ref_cuda_conv2d_bwd_filter.argtypes = [vp] * 5 + [ip] * 13
        L.ref_cuda_conv2d_bwd_input.argtypes = [vp] * 6 + [ip] * 13
        for n in ("ref_cuda_dense_fwd", "ref_cuda_dense_bwd_weight", "ref_cuda_dense_bwd_input"):
            getattr(L, n).argtypes = [vp] * 4 + [ip] * 3
        L.ref_cuda_matmul.argtypes = [vp] * 4 + [ip] * 6
        self.h = L.ref_cuda_lut_open(lut_path.encode())

    def close(self):
        if self.h:
            self.lib.ref_cuda_lut_close(self.h)
            self.h = None

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    def conv2d_fwd(self, g: ConvGeom, x, w, same: bool):
        import torch
        y = torch.empty((g.batch, g.out_h, g.out_w, g.out_c), dtype=torch.float32, device=x.device)
        col = torch.empty(g.batch * g.out_h * g.out_w * g.f_h * g.f_w * g.in_c, dtype=torch.float32, device=x.device)
        self.lib.ref_cuda_conv2d_fwd(self.h, self._p(x), self._p(w), self._p(y), self._p(col), g.batch, g.in_h, g.in_w, g.in_c,
                                     g.f_h, g.f_w, g.out_c, g.out_h, g.out_w, g.stride_h, g.stride_w, g.pad_top, g.pad_left,
                                     2 if same else 1)   # tensorflow::Padding: VALID = 1, SAME = 2 (convam.cc:557)
        return y

    def conv2d_bwd_filter(self, g: ConvGeom, x, dy):
        import torch
        dw = torch.empty((g.f_h, g.f_w, g.in_c, g.out_c), dtype=torch.float32, device=x.device)
        col = torch.empty(g.batch * g.out_h * g.out_w * g.f_h * g.f_w * g.in_c, dtype=torch.float32, device=x.device)
        self.lib.ref_cuda_conv2d_bwd_filter(self.h, self._p(x), self._p(dy), self._p(dw), self._p(col), g.batch, g.in_h, g.in_w,
                                            g.in_c, g.f_h, g.f_w, g.out_c, g.out_h, g.out_w, g.stride_h, g.stride_w,
                                            g.pad_top, g.pad_left)
        return dw

    def conv2d_bwd_input(self, g: ConvGeom, w, dy):
        import torch
        dx = torch.empty((g.batch, g.in_h, g.in_w, g.in_c), dtype=torch.float32, device=w.device)
        col = torch.empty(g.batch * g.in_h * g.in_w * g.f_h * g.f_w * g.out_c, dtype=torch.float32, device=w.device)
        rs = torch.empty(g.f_h * g.f_w * g.in_c * g.out_c, dtype=torch.float32, device=w.device)
        self.lib.ref_cuda_conv2d_bwd_input(self.h, self._p(w), self._p(dy), self._p(dx), self._p(col), self._p(rs), g.batch,
                                           g.in_h, g.in_w, g.in_c, g.f_h, g.f_w, g.out_c, g.out_h, g.out_w, g.stride_h,
                                           g.stride_w, g.pad_top, g.pad_left)
        return dx

    def dense(self, which, p, q, batch, units, in_w):
        import torch
        shape = {"fwd": (batch, units), "bwd_weight": (in_w, units), "bwd_input": (batch, in_w)}[which]
        out = torch.empty(shape, dtype=torch.float32, device=p.device)
        getattr(self.lib, "ref_cuda_dense_" + which)(self.h, self._p(p), self._p(q), self._p(out), batch, units, in_w)
        return out

    def matmul(self, a, b):
        """Ranks (2,2), (3,3), (2,3), (3,2); a batch of 0 marks a rank-2 operand (matmulam.cc:86-147)."""
        import torch
        ba = a.shape[0] if a.dim() == 3 else 0
        bb = b.shape[0] if b.dim() == 3 else 0
        nb = max(ba, bb)
        m, n = a.shape[-2], b.shape[-1]
        out = torch.empty((nb, m, n) if nb else (m, n), dtype=torch.float32, device=a.device)
        self.lib.ref_cuda_matmul(self.h, self._p(a), self._p(b), self._p(out), ba, bb, a.shape[-2], a.shape[-1], b.shape[-2],
                                 b.shape[-1])
        return out
