"""Layers over the AM ops, with the reference's gradient wiring.

``AMConv2D`` and ``denseam`` mirror the Keras layers of the reference
(python/keras/layers/am_convolutional.py:259-292, amdenselayer.py:180-227):
the approximate op computes the linear part, bias add and activation are
ordinary exact ops outside it.  Gradients are registered the way the reference
does it in Python:

* ``Convam``  -> ``ConvamInputGrad`` + ``ConvamFilterGrad``
  (python/ops/amnn_ops.py:220-244),
* ``Denseam`` -> ``DenseamGrad`` (amdenselayer.py:258-260),
* ``MatMulAM`` -> ``dA = MatMulAM(g, B^T)``, ``dB = MatMulAM(A^T, g)`` with the
  same LUT (the intent of python/ops/math_ops.py:127-157, whose code does not
  forward the LUT).

Activations are NHWC, filters HWIO, dense weights [in, out] — the reference's
layouts, so weights are interchangeable with its Keras checkpoints.
"""
from __future__ import annotations

import math
import os

import torch
from torch import nn

from . import ops


class GradSink:
    """Where a parameter's gradient may be written directly.  A trainer that keeps gradients in its
    own buffers (``dp.DataParallelSGD``: views into flat all-reduce buckets) attaches one to each
    parameter as ``param.amsim_grad_sink``; the backward of an AM layer then lets the gradient kernel
    write straight into ``view`` (autograd's accumulate kernel is skipped) and calls ``ready(param)``
    in place of the post-accumulate hook autograd would have fired.  Only a parameter that one
    layer call used since the trainer's last ``reset()`` is written directly; a parameter used by
    several calls (shared weights) has its contributions summed by autograd as usual."""

    def __init__(self, view: torch.Tensor, ready=None):
        self.view = view
        self.ready = ready
        self.uses = 0          # layer calls that took this parameter since reset()

    def reset(self):
        self.uses = 0

    def take(self):
        """The buffer for a direct write, or None if autograd has to sum several contributions."""
        return self.view if self.uses == 1 else None


def _sink_of(param):
    s = getattr(param, "amsim_grad_sink", None)
    if not isinstance(s, GradSink) or not param.requires_grad:
        return None
    s.uses += 1
    return s


def _deliver(sink, param):
    if sink.ready is not None:
        sink.ready(param)


# The input gradient of a layer and its filter / weight / bias gradients read the same output gradient and
# do not depend on each other.  The backward functions below launch the input gradient on the current
# stream and the parameter gradients on a second stream forked from it, and join before they return: the
# kernels of the one fill the multiprocessors that the other leaves idle while it ramps up and drains
# (measured inside a replayed graph: 0.4-2.6 % of a layer's backward time, most on the short 1x1 layers).
# Only kernels that take no library-owned scratch run on the second stream (filter / weight / bias
# gradients get theirs from the caller), so the one persistent scratch buffer of captured launches is
# never used by two launches at once.  TWO_STREAM_BACKWARD = False launches everything in order on the
# current stream (the benchmark's instrumented step does, so that its per-op event pairs do not overlap).
TWO_STREAM_BACKWARD = os.environ.get("AMSIM_TWO_STREAM_BACKWARD", "1") != "0"
_side_streams = {}


class _Fork:
    """``with fork: ...`` runs the body on the device's second stream, ordered after everything launched on
    the current stream before ``_Fork()`` was created; ``join()`` makes the current stream wait for it."""

    def __init__(self, tensor):
        self.side = None
        if TWO_STREAM_BACKWARD and tensor.is_cuda:
            idx = tensor.device.index
            if idx not in _side_streams:
                _side_streams[idx] = torch.cuda.Stream(tensor.device)
            self.side = _side_streams[idx]
            self.cur = torch.cuda.current_stream(tensor.device)
            self.side.wait_stream(self.cur)

    def __enter__(self):
        if self.side is not None:
            self._ctx = torch.cuda.stream(self.side)
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self.side is not None:
            self._ctx.__exit__(*exc)

    def join(self):
        if self.side is not None:
            self.cur.wait_stream(self.side)


def _filter_grad(ctx, w, x, g, strides, padding, lut, det):
    """ConvamFilterGrad into the parameter's sink if it has a fresh one (returns the sink to report once
    the streams have joined: autograd has nothing left to accumulate), else as a new tensor."""
    buf = ctx.w_sink.take() if ctx.w_sink is not None else None
    dw = ops.convam_filter_grad(w.shape, x, g, strides=strides, padding=padding, mant_mul_lut=lut, deterministic=det, out=buf)
    return (dw, None) if buf is None else (None, (ctx.w_sink, ctx.w_param))


def _bias_grad(ctx, g):
    buf = ctx.b_sink.take() if ctx.b_sink is not None else None
    db = ops.bias_grad(g, out=buf)
    return (db, None) if buf is None else (None, (ctx.b_sink, ctx.b_param))


def _conv_backward(ctx, g, x, w, strides, padding, lut, det, want_dx, want_dw, want_db):
    """(dx, dw, db) of a convolution layer from its (already masked) output gradient ``g``."""
    dx = dw = db = None
    done = []
    fork = _Fork(g)
    if want_dx:
        dx = ops.convam_input_grad(x.shape, w, g, strides=strides, padding=padding, mant_mul_lut=lut, deterministic=det)
    with fork:
        if want_dw:
            dw, d = _filter_grad(ctx, w, x, g, strides, padding, lut, det)
            done.append(d)
        if want_db:
            db, d = _bias_grad(ctx, g)
            done.append(d)
    fork.join()
    for d in done:
        if d is not None:
            _deliver(*d)
    return dx, dw, db


def _dense_backward(ctx, g, x, w, lut, det, want_dw, want_db):
    """(dx, dw, db) of a dense layer: DenseamGrad (input gradient on the current stream, weight gradient
    on the second one; into the parameter's sink if it has a fresh one) and the bias gradient."""
    buf = ctx.w_sink.take() if (ctx.w_sink is not None and want_dw) else None
    fork = _Fork(g)
    dx, dw = ops.denseam_grad(g, x, w, lut, deterministic=det, out_weights=buf, weights_stream=fork.side)
    db, d = None, None
    with fork:
        if want_db:
            db, d = _bias_grad(ctx, g)
    fork.join()
    if buf is not None:
        _deliver(ctx.w_sink, ctx.w_param)
        dw = None
    if d is not None:
        _deliver(*d)
    return dx, dw, db


class _ConvamFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, strides, padding, lut, deterministic):
        ctx.save_for_backward(x, w)
        ctx.cfg = (strides, padding, lut, deterministic)
        ctx.w_param, ctx.w_sink = w, _sink_of(w)
        return ops.convam(x, w, strides=strides, padding=padding, mant_mul_lut=lut, deterministic=deterministic)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        strides, padding, lut, det = ctx.cfg
        dx, dw, _ = _conv_backward(ctx, dy.contiguous(), x, w, strides, padding, lut, det, ctx.needs_input_grad[0],
                                   ctx.needs_input_grad[1], False)
        return dx, dw, None, None, None, None


class _DenseamFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, lut, deterministic):
        ctx.save_for_backward(x, w)
        ctx.cfg = (lut, deterministic)
        ctx.w_param, ctx.w_sink = w, _sink_of(w)
        return ops.denseam(x, w, lut, deterministic=deterministic)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        lut, det = ctx.cfg
        dx, dw, _ = _dense_backward(ctx, g.contiguous(), x, w, lut, det, ctx.needs_input_grad[1], False)
        return dx, dw, None, None


class _ConvamBiasActFn(torch.autograd.Function):
    """act(Convam(x, w) + b) with the bias add and ReLU fused into the forward
    kernel; backward masks the gradient with the saved output (ReLU), reduces the
    bias gradient and then follows the Convam gradient wiring."""

    @staticmethod
    def forward(ctx, x, w, b, strides, padding, activation, lut, deterministic):
        y = ops.convam_bias_act(x, w, b, strides=strides, padding=padding, activation=activation, mant_mul_lut=lut,
                                deterministic=deterministic)
        ctx.save_for_backward(x, w, y if activation == "relu" else None)
        ctx.cfg = (strides, padding, lut, deterministic, b is not None)
        ctx.w_param, ctx.w_sink = w, _sink_of(w)
        ctx.b_param, ctx.b_sink = b, (_sink_of(b) if b is not None else None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, y = ctx.saved_tensors
        strides, padding, lut, det, has_bias = ctx.cfg
        # ReLU gradient as one kernel: dy where the output was positive, +0 elsewhere (TF's ReluGrad)
        g = torch.ops.aten.threshold_backward(dy, y, 0.0) if y is not None else dy
        dx, dw, db = _conv_backward(ctx, g.contiguous(), x, w, strides, padding, lut, det, ctx.needs_input_grad[0],
                                    ctx.needs_input_grad[1], has_bias and ctx.needs_input_grad[2])
        return dx, dw, db, None, None, None, None, None


class _DenseamBiasActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, activation, lut, deterministic):
        y = ops.denseam_bias_act(x, w, b, activation=activation, mant_mul_lut=lut, deterministic=deterministic)
        ctx.save_for_backward(x, w, y if activation == "relu" else None)
        ctx.cfg = (lut, deterministic, b is not None)
        ctx.w_param, ctx.w_sink = w, _sink_of(w)
        ctx.b_param, ctx.b_sink = b, (_sink_of(b) if b is not None else None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, y = ctx.saved_tensors
        lut, det, has_bias = ctx.cfg
        g = (torch.ops.aten.threshold_backward(dy, y, 0.0) if y is not None else dy).contiguous()
        dx, dw, db = _dense_backward(ctx, g, x, w, lut, det, ctx.needs_input_grad[1], has_bias and ctx.needs_input_grad[2])
        return dx, dw, db, None, None, None


def _unbroadcast(grad, operand):
    """Gradient of an operand that MatMulAM broadcast over the batch: a rank-2 operand, or a
    rank-3 operand whose batch is 1 against a larger batch (matmulam.cc:86-147).  The per-batch
    gradients are summed (exact FP32 adds) back to the operand's shape."""
    if operand.dim() == 2 and grad.dim() == 3:
        return grad.sum(0)
    if operand.dim() == 3 and grad.dim() == 3 and operand.shape[0] == 1 and grad.shape[0] > 1:
        return grad.sum(0, keepdim=True)
    return grad


class _MatMulAMFn(torch.autograd.Function):
    """C = alpha * op(A) @ op(B).  Gradients follow the four transpose cases of the
    reference's registered gradient (python/ops/math_ops.py:127-157), every product
    through MatMulAM with the same LUT; the transposes are index maps in the kernel."""

    @staticmethod
    def forward(ctx, a, b, lut, deterministic, ta, tb, alpha):
        ctx.save_for_backward(a, b)
        ctx.cfg = (lut, deterministic, ta, tb, alpha)
        return ops.matmulam(a, b, transpose_a=ta, transpose_b=tb, mant_mul_lut=lut, deterministic=deterministic,
                            alpha=alpha)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        lut, det, ta, tb, alpha = ctx.cfg
        g = g.contiguous()
        kw = dict(mant_mul_lut=lut, deterministic=det, alpha=alpha)
        da = db = None
        if ctx.needs_input_grad[0]:
            if not ta:
                da = ops.matmulam(g, b, transpose_b=not tb, **kw)
            else:
                da = ops.matmulam(b, g, transpose_a=tb, transpose_b=True, **kw)
            da = _unbroadcast(da, a)
        if ctx.needs_input_grad[1]:
            if not tb:
                db = ops.matmulam(a, g, transpose_a=not ta, **kw)
            else:
                db = ops.matmulam(g, a, transpose_a=True, transpose_b=ta, **kw)
            db = _unbroadcast(db, b)
        return da, db, None, None, None, None, None


def amconv2d(x, w, strides=1, padding="VALID", mant_mul_lut="", deterministic=False):
    return _ConvamFn.apply(x, w, strides, padding, mant_mul_lut, deterministic)


def amdense(x, w, mant_mul_lut="", deterministic=False):
    """AM dense on the last axis.  The reference's layer falls back to an exact
    ``tensordot`` for rank > 2 inputs (amdenselayer.py:214-215); here the leading
    axes are flattened so the approximate multiplier is used for every rank."""
    lead = x.shape[:-1]
    y = _DenseamFn.apply(x.reshape(-1, x.shape[-1]).contiguous(), w, mant_mul_lut, deterministic)
    return y.reshape(*lead, w.shape[1])


def ammatmul(a, b, mant_mul_lut="", deterministic=False, transpose_a=False, transpose_b=False, alpha=None):
    """Batched AM matmul ``alpha * op(a) @ op(b)`` for rank >= 2 operands with equal
    leading axes (the reference op takes rank 2/3: matmulam.cc:86-120; extra leading axes
    are folded into the batch, which is what ammha/multihead_attention.py:18,30 needs)."""
    return _MatMulAMFn.apply(a.contiguous(), b.contiguous(), mant_mul_lut, deterministic, bool(transpose_a),
                             bool(transpose_b), alpha)


_ACT = {None: lambda t: t, "linear": lambda t: t, "relu": torch.relu, "tanh": torch.tanh,
        "softmax": lambda t: torch.softmax(t, -1)}


class AMConv2D(nn.Module):
    """2-D convolution with the approximate multiplier (am_convolutional.py AMConv2D).
    NHWC in/out; kernel HWIO; ``padding`` 'valid' | 'same'."""

    def __init__(self, in_channels, filters, kernel_size, strides=1, padding="valid", activation=None, use_bias=True,
                 mant_mul_lut="", kernel_initializer="glorot_uniform", deterministic=False):
        super().__init__()
        kh, kw = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        self.strides = (strides, strides) if isinstance(strides, int) else tuple(strides)
        self.padding = padding.upper()
        self.activation = activation
        self.mant_mul_lut = mant_mul_lut
        self.deterministic = deterministic
        self.kernel = nn.Parameter(torch.empty(kh, kw, in_channels, filters))
        self.bias = nn.Parameter(torch.zeros(filters)) if use_bias else None
        fan_in, fan_out = kh * kw * in_channels, kh * kw * filters
        with torch.no_grad():
            if kernel_initializer == "he_normal":
                nn.init.trunc_normal_(self.kernel, std=math.sqrt(2.0 / fan_in) / 0.87962566103423978, a=-2 * math.sqrt(2.0 / fan_in) / 0.8796, b=2 * math.sqrt(2.0 / fan_in) / 0.8796)
            else:
                lim = math.sqrt(6.0 / (fan_in + fan_out))
                self.kernel.uniform_(-lim, lim)

    def forward(self, x):
        st = [1, self.strides[0], self.strides[1], 1]
        if self.activation in (None, "linear", "relu") and (self.bias is not None or self.activation == "relu"):
            return _ConvamBiasActFn.apply(x, self.kernel, self.bias, st, self.padding, self.activation,
                                          self.mant_mul_lut, self.deterministic)
        y = amconv2d(x, self.kernel, st, self.padding, self.mant_mul_lut, self.deterministic)
        if self.bias is not None:
            y = y + self.bias
        return _ACT[self.activation](y)


class denseam(nn.Module):
    """Dense layer with the approximate multiplier (amdenselayer.py denseam)."""

    def __init__(self, in_features, units, activation=None, use_bias=True, mant_mul_lut="",
                 kernel_initializer="glorot_uniform", deterministic=False):
        super().__init__()
        self.activation = activation
        self.mant_mul_lut = mant_mul_lut
        self.deterministic = deterministic
        self.kernel = nn.Parameter(torch.empty(in_features, units))
        self.bias = nn.Parameter(torch.zeros(units)) if use_bias else None
        with torch.no_grad():
            if kernel_initializer == "he_normal":
                s = math.sqrt(2.0 / in_features)
                nn.init.trunc_normal_(self.kernel, std=s / 0.8796, a=-2 * s / 0.8796, b=2 * s / 0.8796)
            else:
                lim = math.sqrt(6.0 / (in_features + units))
                self.kernel.uniform_(-lim, lim)

    def forward(self, x):
        if self.activation in (None, "linear", "relu") and (self.bias is not None or self.activation == "relu"):
            lead = x.shape[:-1]
            y = _DenseamBiasActFn.apply(x.reshape(-1, x.shape[-1]).contiguous(), self.kernel, self.bias,
                                        self.activation, self.mant_mul_lut, self.deterministic)
            return y.reshape(*lead, self.kernel.shape[1])
        y = amdense(x, self.kernel, self.mant_mul_lut, self.deterministic)
        if self.bias is not None:
            y = y + self.bias
        return _ACT[self.activation](y)


# ---- exact helpers that keep activations physically NHWC --------------------------------------
def nhwc_max_pool(x, k, s, padding=0):
    return torch.nn.functional.max_pool2d(x.permute(0, 3, 1, 2), k, s, padding).permute(0, 2, 3, 1)


def nhwc_avg_pool(x, k, s):
    return torch.nn.functional.avg_pool2d(x.permute(0, 3, 1, 2), k, s).permute(0, 2, 3, 1)


class BatchNormNHWC(nn.BatchNorm2d):
    """Exact batch normalisation on an NHWC tensor (viewed as channels-last NCHW)."""

    def forward(self, x):
        return super().forward(x.permute(0, 3, 1, 2)).permute(0, 2, 3, 1)
