"""Host-side mirror of ApproxTrain's custom-op interface on top of the C ABI.

One function per TensorFlow op the reference registers, same names, argument
meaning and error behaviour:

=====================  =======================================================
``convam``             ``Convam``            (convam.cc:427-437, :502-595)
``convam_input_grad``  ``ConvamInputGrad``   (convam.cc:958-975, :1018-1136)
``convam_filter_grad`` ``ConvamFilterGrad``  (convam.cc:690-707, :751-866)
``denseam``            ``Denseam``           (denseam.cc:36-57, :81-118)
``denseam_grad``       ``DenseamGrad``       (denseam.cc:177-235)
``matmulam``           ``MatMulAM``          (matmulam.cc:48-172,
                                              python/ops/math_ops.py:12-95)
=====================  =======================================================

Tensors are ``torch`` CUDA tensors (torch supplies device memory and the
current stream, nothing else); every op is a single call into
``libamsim.so``.  ``mant_mul_lut`` is the path of a ``<MODEL>_<m>.bin`` file as
in the reference.  ``deterministic=True`` selects the bit-exact
reference-order mode (``AMSIM_DETERMINISTIC``).
"""
from __future__ import annotations

import contextlib

import ctypes as C
import threading
from typing import Sequence

import torch

from . import _lib
from ._lib import AmsimError, lib, check

__all__ = [
    "AMLut", "get_lut", "am_multiply", "conv2d_geometry", "convam", "convam_input_grad", "convam_filter_grad",
    "denseam", "denseam_grad", "matmulam", "convam_bias_act", "denseam_bias_act", "bias_grad", "AmsimError",
]


class AMLut:
    """Device-resident mantissa LUT (approx_mul_lut<GpuDevice>,
    cuda/approx_mul_lut.cu:24-53).  Handles are shared per (path, device)."""

    def __init__(self, path: str, device: int):
        if not path:
            # approx_mul_lut.h:18-21 prints this and exits; here it is an error
            raise AmsimError(_lib.ERR_LUT_NAME, "no mant lut file name given")
        h = C.c_void_p()
        check(lib.amsim_lut_open(path.encode(), int(device), C.byref(h)))
        self._h = h
        self.path = path
        self.device = int(device)
        m, mask, a_s, b_s, ptr = C.c_int(), C.c_uint32(), C.c_int(), C.c_int(), C.c_void_p()
        check(lib.amsim_lut_info(h, C.byref(m), C.byref(mask), C.byref(a_s), C.byref(b_s), C.byref(ptr)))
        self.mant_width, self.mant_mask, self.a_shift, self.b_shift = m.value, mask.value, a_s.value, b_s.value
        self.device_ptr = ptr.value

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    def close(self) -> None:
        if self._h:
            lib.amsim_lut_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_lut_cache: dict = {}
_lut_mu = threading.Lock()


def get_lut(path: str, device) -> AMLut:
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    key = (path, idx)
    with _lut_mu:
        lut = _lut_cache.get(key)
        if lut is None:
            lut = _lut_cache[key] = AMLut(path, idx)
        return lut


def _prep(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must live on a CUDA device: the AM ops have no CPU implementation")
    if t.dtype not in (torch.float32, torch.int32):
        raise TypeError(f"{name} must be float32 or int32 (attr T of the reference ops), got {t.dtype}")
    return t.contiguous()


def _dtype_flag(*tensors) -> int:
    """T: {float, int32} — all tensors of a call share the type."""
    dts = {t.dtype for t in tensors}
    if len(dts) != 1:
        raise TypeError(f"all tensors of an op must have the same dtype, got {sorted(str(d) for d in dts)}")
    return _lib.INT32 if dts.pop() == torch.int32 else 0


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(t.data_ptr())


def _flags(deterministic: bool) -> int:
    return _lib.DETERMINISTIC if deterministic else _lib.FAST


def _hw(value, name: str):
    """strides / dilations as TF passes them: int, [h, w] or [1, h, w, 1] (NHWC)."""
    if value is None:
        return 1, 1
    if isinstance(value, int):
        return value, value
    v = list(value)
    if len(v) == 1:
        return v[0], v[0]
    if len(v) == 2:
        return v[0], v[1]
    if len(v) == 4:
        if v[0] != 1 or v[3] != 1:
            raise ValueError(f"Current implementation does not yet support {name} in the batch and depth dimensions.")
        return v[1], v[2]
    raise ValueError(f"{name} should be of length 1, 2 or 4 but was {len(v)}")


def _check_format(data_format, dilations):
    if data_format not in (None, "NHWC"):
        raise ValueError("only data_format NHWC is supported")
    dh, dw = _hw(dilations, "dilations")
    if dh != 1 or dw != 1:
        # python/ops/amnn_ops.py:196-197
        raise ValueError("Dilation is not supported in current implementation")


def _same(padding) -> int:
    p = padding.upper() if isinstance(padding, str) else padding
    if p == "SAME":
        return 1
    if p == "VALID":
        return 0
    raise ValueError(f"padding must be 'SAME' or 'VALID', got {padding!r}")


def conv2d_geometry(in_h, in_w, f_h, f_w, stride_h, stride_w, padding):
    """(out_h, out_w, pad_top, pad_left) — convam.cc:315-407, :557-572."""
    oh, ow, pt, pl = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    check(lib.amsim_conv2d_geometry(in_h, in_w, f_h, f_w, stride_h, stride_w, _same(padding),
                                    C.byref(oh), C.byref(ow), C.byref(pt), C.byref(pl)))
    return oh.value, ow.value, pt.value, pl.value


def am_multiply(a: torch.Tensor, b: torch.Tensor, mant_mul_lut: str) -> torch.Tensor:
    """Elementwise AMsimulator(a, b) (cuda/AMsimulator.inl:13-36), bit-exact."""
    a, b = _prep(a, "a"), _prep(b, "b")
    if a.shape != b.shape:
        raise ValueError("a and b must have the same shape")
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise TypeError("am_multiply takes float32 tensors")
    lut = get_lut(mant_mul_lut, a.device)
    out = torch.empty_like(a)
    with torch.cuda.device(a.device):
        check(lib.amsim_mul(_stream(), lut.handle, _ptr(a), _ptr(b), _ptr(out), a.numel()))
    return out


def convam(input: torch.Tensor, filter: torch.Tensor, strides=None, padding="VALID", data_format="NHWC",
           dilations=None, mant_mul_lut: str = "", deterministic: bool = False) -> torch.Tensor:
    """AMConv2D forward.  input NHWC, filter HWIO."""
    _check_format(data_format, dilations)
    x, w = _prep(input, "input"), _prep(filter, "filter")
    if x.dim() != 4:
        raise ValueError(f"input must be 4-dimensional{list(x.shape)}")
    if w.dim() != 4:
        raise ValueError(f"filter must be 4-dimensional: {list(w.shape)}")
    n, h, wd, c = x.shape
    kh, kw, ci, k = w.shape
    if c != ci:
        # the reference checks divisibility (convam.cc:343-346) but its kernels have no groups
        raise ValueError(f"input depth must be evenly divisible by filter depth: {c} vs {ci}")
    sh, sw = _hw(strides, "strides")
    oh, ow, pt, pl = conv2d_geometry(h, wd, kh, kw, sh, sw, padding)
    lut = get_lut(mant_mul_lut, x.device)
    y = torch.empty((n, oh, ow, k), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.amsim_conv2d_fwd(_stream(), lut.handle, _ptr(x), _ptr(w), _ptr(y), n, h, wd, c, kh, kw, k, oh, ow,
                                   sh, sw, pt, pl, _flags(deterministic) | _dtype_flag(x, w)))
    return y


def _act_code(activation) -> int:
    if activation in (None, "linear"):
        return _lib.ACT_NONE
    if activation == "relu":
        return _lib.ACT_RELU
    raise ValueError(f"only None / 'relu' can be fused into the op, got {activation!r}")


def convam_bias_act(input: torch.Tensor, filter: torch.Tensor, bias, strides=None, padding="VALID",
                    activation=None, mant_mul_lut: str = "", deterministic: bool = False, scale=None) -> torch.Tensor:
    """``act(convam(input, filter) * scale + bias)`` in one launch: the exact bias add and
    ReLU that follow the op in the reference's Keras layer
    (am_convolutional.py:267-292) run in the kernel's epilogue, bit-identical to
    the unfused sequence.  ``bias`` may be None.  ``scale`` (per output channel,
    optional) folds an inference-time BatchNormalization behind the convolution:
    scale = gamma / sqrt(var + eps), bias = beta - mean * scale."""
    x, w = _prep(input, "input"), _prep(filter, "filter")
    if x.dtype != torch.float32 or w.dtype != torch.float32:
        raise TypeError("the fused epilogue is float32 only")
    n, h, wd, c = x.shape
    kh, kw, ci, k = w.shape
    if c != ci:
        raise ValueError(f"input depth must be evenly divisible by filter depth: {c} vs {ci}")
    b = None
    if bias is not None:
        b = _prep(bias, "bias")
        if b.dtype != torch.float32 or tuple(b.shape) != (k,):
            raise ValueError("bias must be float32 of shape [filters]")
    sc = None
    if scale is not None:
        sc = _prep(scale, "scale")
        if sc.dtype != torch.float32 or tuple(sc.shape) != (k,):
            raise ValueError("scale must be float32 of shape [filters]")
    sh, sw = _hw(strides, "strides")
    oh, ow, pt, pl = conv2d_geometry(h, wd, kh, kw, sh, sw, padding)
    lut = get_lut(mant_mul_lut, x.device)
    y = torch.empty((n, oh, ow, k), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        if sc is None:
            check(lib.amsim_conv2d_fwd_bias_act(_stream(), lut.handle, _ptr(x), _ptr(w), _ptr(b) if b is not None else None,
                                                _ptr(y), n, h, wd, c, kh, kw, k, oh, ow, sh, sw, pt, pl,
                                                _act_code(activation), _flags(deterministic)))
        else:
            check(lib.amsim_conv2d_fwd_scale_bias_act(_stream(), lut.handle, _ptr(x), _ptr(w), _ptr(sc),
                                                      _ptr(b) if b is not None else None, _ptr(y), n, h, wd, c, kh, kw, k,
                                                      oh, ow, sh, sw, pt, pl, _act_code(activation), _flags(deterministic)))
    return y


def denseam_bias_act(input: torch.Tensor, weights: torch.Tensor, bias, activation=None, mant_mul_lut: str = "",
                     deterministic: bool = False) -> torch.Tensor:
    """``act(denseam(input, weights) + bias)`` in one launch (amdenselayer.py:222-226 fused)."""
    x, w = _prep(input, "input"), _prep(weights, "weights")
    if x.dtype != torch.float32 or w.dtype != torch.float32:
        raise TypeError("the fused epilogue is float32 only")
    if x.dim() != 2 or w.dim() != 2 or w.shape[0] != x.shape[1]:
        raise ValueError("Denseam takes input [batch, width] and weights [width, units]")
    bsz, kin = x.shape
    u = w.shape[1]
    b = None
    if bias is not None:
        b = _prep(bias, "bias")
        if b.dtype != torch.float32 or tuple(b.shape) != (u,):
            raise ValueError("bias must be float32 of shape [units]")
    lut = get_lut(mant_mul_lut, x.device)
    y = torch.empty((bsz, u), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.amsim_dense_fwd_bias_act(_stream(), lut.handle, _ptr(x), _ptr(w), _ptr(b) if b is not None else None,
                                           _ptr(y), bsz, u, kin, _act_code(activation), _flags(deterministic)))
    return y


def convam_input_grad(input_sizes: Sequence[int], filter: torch.Tensor, out_backprop: torch.Tensor, strides=None,
                      padding="VALID", data_format="NHWC", dilations=None, mant_mul_lut: str = "",
                      deterministic: bool = False) -> torch.Tensor:
    _check_format(data_format, dilations)
    w, dy = _prep(filter, "filter"), _prep(out_backprop, "out_backprop")
    sizes = [int(v) for v in input_sizes]
    if len(sizes) != 4:
        raise ValueError(f"Conv2DBackpropInput: input_sizes input must be 1-dim, not {len(sizes)}")
    n, h, wd, c = sizes
    kh, kw, ci, k = w.shape
    sh, sw = _hw(strides, "strides")
    oh, ow, pt, pl = conv2d_geometry(h, wd, kh, kw, sh, sw, padding)
    if tuple(dy.shape) != (n, oh, ow, k) or ci != c:
        raise ValueError(f"out_backprop shape {list(dy.shape)} does not match the forward output {[n, oh, ow, k]}")
    lut = get_lut(mant_mul_lut, dy.device)
    dx = torch.empty((n, h, wd, c), dtype=dy.dtype, device=dy.device)
    if dx.numel() == 0:
        return dx
    with torch.cuda.device(dy.device):
        check(lib.amsim_conv2d_bwd_input(_stream(), lut.handle, _ptr(w), _ptr(dy), _ptr(dx), n, h, wd, c, kh, kw, k,
                                         oh, ow, sh, sw, pt, pl, _flags(deterministic) | _dtype_flag(w, dy)))
    return dx


def _out_tensor(out, shape, dtype, device, name):
    """``out=``: a caller-owned result buffer (e.g. a view into a gradient bucket); must match exactly."""
    if out is None:
        return torch.empty(shape, dtype=dtype, device=device)
    if tuple(out.shape) != tuple(shape) or out.dtype != dtype or out.device != device or not out.is_contiguous():
        raise ValueError(f"{name}: out must be a contiguous {dtype} tensor of shape {list(shape)} on {device}")
    return out


def convam_filter_grad(filter_sizes: Sequence[int], input: torch.Tensor, out_backprop: torch.Tensor, strides=None,
                       padding="VALID", data_format="NHWC", dilations=None, mant_mul_lut: str = "",
                       deterministic: bool = False, out: torch.Tensor = None) -> torch.Tensor:
    """``out`` (optional): write the gradient into this tensor instead of a new one."""
    _check_format(data_format, dilations)
    x, dy = _prep(input, "input"), _prep(out_backprop, "out_backprop")
    sizes = [int(v) for v in filter_sizes]
    if len(sizes) != 4:
        raise ValueError(f"Conv2DBackpropFilter: filter_sizes input must be 1-dim, not {len(sizes)}")
    kh, kw, ci, k = sizes
    n, h, wd, c = x.shape
    sh, sw = _hw(strides, "strides")
    oh, ow, pt, pl = conv2d_geometry(h, wd, kh, kw, sh, sw, padding)
    if tuple(dy.shape) != (n, oh, ow, k) or ci != c:
        raise ValueError(f"out_backprop shape {list(dy.shape)} does not match the forward output {[n, oh, ow, k]}")
    lut = get_lut(mant_mul_lut, x.device)
    dw = _out_tensor(out, (kh, kw, c, k), x.dtype, x.device, "convam_filter_grad")
    if dw.numel() == 0:
        return dw
    fl = _flags(deterministic) | _dtype_flag(x, dy)
    ws_bytes = lib.amsim_conv2d_bwd_filter_workspace(n, h, wd, c, kh, kw, k, oh, ow, fl)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
    with torch.cuda.device(x.device):
        check(lib.amsim_conv2d_bwd_filter(_stream(), lut.handle, _ptr(x), _ptr(dy), _ptr(dw), n, h, wd, c, kh, kw, k,
                                          oh, ow, sh, sw, pt, pl, _ptr(ws) if ws is not None else None, ws_bytes, fl))
    return dw


def denseam(input: torch.Tensor, weights: torch.Tensor, mant_mul_lut: str = "",
            deterministic: bool = False) -> torch.Tensor:
    x, w = _prep(input, "input"), _prep(weights, "weights")
    if x.dim() != 2 or w.dim() != 2:
        raise ValueError("Denseam takes rank-2 input and weights")
    b, kin = x.shape
    if w.shape[0] != kin:
        raise ValueError(f"input width {kin} does not match weights rows {w.shape[0]}")
    u = w.shape[1]
    lut = get_lut(mant_mul_lut, x.device)
    y = torch.empty((b, u), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.amsim_dense_fwd(_stream(), lut.handle, _ptr(x), _ptr(w), _ptr(y), b, u, kin,
                                  _flags(deterministic) | _dtype_flag(x, w)))
    return y


def denseam_grad(grad: torch.Tensor, input: torch.Tensor, weights: torch.Tensor, mant_mul_lut: str = "",
                 deterministic: bool = False, out_weights: torch.Tensor = None, weights_stream=None):
    """Returns (grad_input, grad_weights) like DenseamGrad (denseam.cc:177-235).  ``out_weights``
    (optional): write grad_weights into this tensor instead of a new one.  ``weights_stream`` (optional
    ``torch.cuda.Stream`` that already waits for the operands): the weight gradient and its scratch are
    launched there, the input gradient on the current stream; the caller joins the two."""
    g, x, w = _prep(grad, "grad"), _prep(input, "input"), _prep(weights, "weights")
    b, kin = x.shape
    u = w.shape[1]
    if tuple(g.shape) != (b, u) or w.shape[0] != kin:
        raise ValueError("grad / input / weights shapes are inconsistent")
    lut = get_lut(mant_mul_lut, x.device)
    fl = _flags(deterministic) | _dtype_flag(g, x, w)
    dx = torch.empty_like(x)
    ws_bytes = lib.amsim_dense_bwd_weight_workspace(b, u, kin, fl)
    with torch.cuda.device(x.device):
        if weights_stream is not None:   # input gradient first: it is the one the rest of backward waits for
            check(lib.amsim_dense_bwd_input(_stream(), lut.handle, _ptr(w), _ptr(g), _ptr(dx), b, u, kin, fl))
        with (torch.cuda.stream(weights_stream) if weights_stream is not None else contextlib.nullcontext()):
            dw = _out_tensor(out_weights, tuple(w.shape), w.dtype, w.device, "denseam_grad")
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
            check(lib.amsim_dense_bwd_weight(_stream(), lut.handle, _ptr(x), _ptr(g), _ptr(dw), b, u, kin,
                                             _ptr(ws) if ws is not None else None, ws_bytes, fl))
        if weights_stream is None:
            check(lib.amsim_dense_bwd_input(_stream(), lut.handle, _ptr(w), _ptr(g), _ptr(dx), b, u, kin, fl))
    return dx, dw


def matmulam(a: torch.Tensor, b: torch.Tensor, transpose_a: bool = False, transpose_b: bool = False,
             adjoint_a: bool = False, adjoint_b: bool = False, a_is_sparse: bool = False, b_is_sparse: bool = False,
             mant_mul_lut: str = "", deterministic: bool = False, alpha=None) -> torch.Tensor:
    """``alpha * op(a) @ op(b)`` with the approximate multiplier.  Same arguments as
    python/ops/math_ops.py:60-93; there the transposes are materialised before the
    op because its kernel ignores the attrs, here the kernel reads the operands
    transposed in place.  Operands of rank > 3 (ammha/multihead_attention.py:18
    passes [batch, heads, seq, d]) have their leading axes folded into the batch;
    a rank-2 operand or a batch of 1 broadcasts.  ``alpha`` (optional Python float)
    multiplies every finished sum once in FP32."""
    if adjoint_a or adjoint_b or a_is_sparse or b_is_sparse:
        raise ValueError("Matmulam unsupported args: adjoint_a, adjoint_b, a_is_sparse, b_is_sparse.")
    a, b = _prep(a, "a"), _prep(b, "b")
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise TypeError("MatMulAM is registered for float only")
    if a.dim() < 2 or b.dim() < 2:
        raise ValueError("Input a and b should be 2 dimensional or 3 dimensional and compitable batch size")
    lead = None
    if a.dim() > 3 or b.dim() > 3:
        if a.dim() != b.dim() or a.shape[:-2] != b.shape[:-2]:
            raise ValueError("operands of rank > 3 need equal leading axes")
        lead = tuple(a.shape[:-2])
        a = a.reshape(-1, *a.shape[-2:])
        b = b.reshape(-1, *b.shape[-2:])
    ba = a.shape[0] if a.dim() == 3 else 0
    bb = b.shape[0] if b.dim() == 3 else 0
    ra, ca = a.shape[-2:]
    rb, cb = b.shape[-2:]
    m, k = (ca, ra) if transpose_a else (ra, ca)
    kb, n = (cb, rb) if transpose_b else (rb, cb)
    if ba and bb and not (ba == bb or ba == 1 or bb == 1):
        raise ValueError("Does not meet batch of mat a is equal batch of matb")
    if k != kb:
        raise ValueError("Does not meet cols of mat a is equal rows of mat b")
    nb = max(ba, bb)
    lut = get_lut(mant_mul_lut, a.device)
    out = torch.empty((nb, m, n) if nb else (m, n), dtype=torch.float32, device=a.device)
    al = C.byref(C.c_float(float(alpha))) if alpha is not None else None
    with torch.cuda.device(a.device):
        check(lib.amsim_matmul_ex(_stream(), lut.handle, _ptr(a), _ptr(b), _ptr(out), ba, bb, ra, ca, rb, cb,
                                  int(bool(transpose_a)), int(bool(transpose_b)), al, _flags(deterministic)))
    if lead is not None:
        out = out.reshape(*lead, m, n)
    return out


def bias_grad(out_backprop: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Gradient of a bias that was added along the last axis: the sum of ``out_backprop`` over all
    other axes (TensorFlow's BiasAddGrad behind the reference's Keras layers,
    am_convolutional.py:267-292, amdenselayer.py:222-226).  Exact FP32 adds in a fixed order, one
    read of the gradient.  ``out`` (optional): write the result into this tensor."""
    g = _prep(out_backprop, "out_backprop")
    if g.dtype != torch.float32 or g.dim() < 1:
        raise TypeError("bias_grad takes a float32 tensor of rank >= 1")
    cols = g.shape[-1]
    rows = g.numel() // cols if cols else 0
    db = _out_tensor(out, (cols,), torch.float32, g.device, "bias_grad")
    if cols == 0:
        return db
    ws_bytes = lib.amsim_bias_grad_workspace(rows, cols)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=g.device) if ws_bytes else None
    with torch.cuda.device(g.device):
        check(lib.amsim_bias_grad(_stream(), _ptr(g), _ptr(db), rows, cols, _ptr(ws) if ws is not None else None, ws_bytes))
    return db


def _install_nvtx_ranges() -> None:
    """With AMSIM_NVTX set in the environment every op call is bracketed by an NVTX range
    named after the op and its output shape, so a timeline profiler shows the ops by name
    (the reference has no tracing beyond per-batch wall-clock prints, profile/profile_lut.py:81-106)."""
    import functools
    import os
    if not os.environ.get("AMSIM_NVTX"):
        return
    g = globals()
    for name in ("am_multiply", "convam", "convam_bias_act", "denseam_bias_act", "convam_input_grad",
                 "convam_filter_grad", "denseam", "denseam_grad", "matmulam", "bias_grad"):
        fn = g[name]

        def wrapped(*a, __fn=fn, __name=name, **k):
            torch.cuda.nvtx.range_push("amsim." + __name)
            try:
                return __fn(*a, **k)
            finally:
                torch.cuda.nvtx.range_pop()
        g[name] = functools.wraps(fn)(wrapped)


_install_nvtx_ranges()
