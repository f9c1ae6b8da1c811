"""The five benchmark networks (LeNet-300-100, LeNet-5, the conv microbenchmark's layers, ResNet-50, Transformer), built from the AM layers.

Every convolution is ``AMConv2D``, every dense layer ``denseam``, every attention
product ``MatMulAM``; pooling, normalisation, activations, softmax and the loss
are exact FP32 ops (as in the reference, where they are stock TensorFlow ops
around the custom ops).  Inputs are NHWC.

* ``LeNet300100``   lenet300100.py of the reference (784-300-100-10).
* ``LeNet5``        mnist_example.py:31-57 shapes: conv5x5x6 SAME, pool, conv5x5x16 VALID, pool, 120-84-10.
* ``ResNet50AM``    profile/resnet50_lut.py:568-718 (bottleneck v1; the 3x3/2 max pool is unpadded, so
                    stage 2 runs at 55x55 for a 224x224 input); the final FC is an AM dense.
* ``TransformerAM`` ammha/encoder.py, decoder.py, multihead_attention.py, positional_encoding.py:
                    post-norm encoder/decoder, sinusoidal positions, token id 0 is padding.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from .layers import AMConv2D, BatchNormNHWC, ammatmul, denseam, nhwc_avg_pool, nhwc_max_pool


class LeNet300100(nn.Module):
    def __init__(self, lut, deterministic=False, init="glorot_uniform"):
        super().__init__()
        kw = dict(mant_mul_lut=lut, deterministic=deterministic, kernel_initializer=init)
        self.fc1 = denseam(784, 300, activation="relu", **kw)
        self.fc2 = denseam(300, 100, activation="relu", **kw)
        self.fc3 = denseam(100, 10, **kw)

    def forward(self, x):
        return self.fc3(self.fc2(self.fc1(x.reshape(x.shape[0], -1))))


class LeNet5(nn.Module):
    def __init__(self, lut, deterministic=False, init="he_normal"):
        super().__init__()
        kw = dict(mant_mul_lut=lut, deterministic=deterministic, kernel_initializer=init)
        self.c1 = AMConv2D(1, 6, 5, padding="same", activation="relu", **kw)
        self.c2 = AMConv2D(6, 16, 5, padding="valid", activation="relu", **kw)
        self.f1 = denseam(400, 120, activation="relu", **kw)
        self.f2 = denseam(120, 84, activation="relu", **kw)
        self.f3 = denseam(84, 10, **kw)

    def forward(self, x):
        x = nhwc_max_pool(self.c1(x), 2, 2)
        x = nhwc_max_pool(self.c2(x), 2, 2)
        return self.f3(self.f2(self.f1(x.reshape(x.shape[0], -1))))


class _Bottleneck(nn.Module):
    def __init__(self, cin, filters, stride, project, kw):
        super().__init__()
        f1, f2, f3 = filters
        self.c1 = AMConv2D(cin, f1, 1, strides=stride, **kw)
        self.b1 = BatchNormNHWC(f1)
        self.c2 = AMConv2D(f1, f2, 3, padding="same", **kw)
        self.b2 = BatchNormNHWC(f2)
        self.c3 = AMConv2D(f2, f3, 1, **kw)
        self.b3 = BatchNormNHWC(f3)
        self.project = project
        if project:
            self.cs = AMConv2D(cin, f3, 1, strides=stride, **kw)
            self.bs = BatchNormNHWC(f3)

    def forward(self, x):
        y = torch.relu(self.b1(self.c1(x)))
        y = torch.relu(self.b2(self.c2(y)))
        y = self.b3(self.c3(y))
        s = self.bs(self.cs(x)) if self.project else x
        return torch.relu(y + s)


class ResNet50AM(nn.Module):
    def __init__(self, lut, classes=1000, deterministic=False):
        super().__init__()
        kw = dict(mant_mul_lut=lut, deterministic=deterministic, kernel_initializer="he_normal")
        self.conv1 = AMConv2D(3, 64, 7, strides=2, padding="valid", **kw)
        self.bn1 = BatchNormNHWC(64)
        blocks = []
        cin = 64
        for stage, (filters, n, stride) in enumerate([([64, 64, 256], 3, 1), ([128, 128, 512], 4, 2),
                                                      ([256, 256, 1024], 6, 2), ([512, 512, 2048], 3, 2)]):
            for i in range(n):
                blocks.append(_Bottleneck(cin, filters, stride if i == 0 else 1, i == 0, kw))
                cin = filters[2]
        self.blocks = nn.Sequential(*blocks)
        self.fc = denseam(2048, classes, **kw)

    def forward(self, x):
        x = torch.nn.functional.pad(x, (0, 0, 3, 3, 3, 3))  # ZeroPadding2D((3, 3)) on H and W of an NHWC tensor
        x = torch.relu(self.bn1(self.conv1(x)))
        x = nhwc_max_pool(x, 3, 2)
        x = self.blocks(x)
        x = nhwc_avg_pool(x, 7, 7)
        return self.fc(x.reshape(x.shape[0], -1))


def _sinusoid(length, depth):
    half = depth // 2
    pos = torch.arange(length, dtype=torch.float32)[:, None]
    rates = 1.0 / (10000 ** (torch.arange(half, dtype=torch.float32)[None, :] / half))
    ang = pos * rates
    return torch.cat([torch.sin(ang), torch.cos(ang)], dim=-1)


class _MHA(nn.Module):
    def __init__(self, lut, h, d_k, d_v, d_model, det):
        super().__init__()
        kw = dict(mant_mul_lut=lut, deterministic=det)
        self.h, self.d_k, self.lut, self.det = h, d_k, lut, det
        self.inv_scale = float(torch.tensor(1.0) / torch.tensor(math.sqrt(d_k), dtype=torch.float32))
        self.wq = denseam(d_model, d_k, **kw)
        self.wk = denseam(d_model, d_k, **kw)
        self.wv = denseam(d_model, d_v, **kw)
        self.wo = denseam(d_v, d_model, **kw)

    def _split(self, x):
        b, s, _ = x.shape
        return x.reshape(b, s, self.h, -1).permute(0, 2, 1, 3).contiguous()

    def forward(self, q, k, v, mask=None):
        q, k, v = self._split(self.wq(q)), self._split(self.wk(k)), self._split(self.wv(v))
        # scores are scaled by sqrt(d_k) with d_k as passed to the layer (multihead_attention.py:16-18)
        # (1 / sqrt(d_k) as one FP32 factor in the product's epilogue, K read transposed in place)
        scores = ammatmul(q, k, self.lut, self.det, transpose_b=True, alpha=self.inv_scale)
        if mask is not None:
            scores = scores + (-1e9) * mask
        o = ammatmul(torch.softmax(scores, -1), v, self.lut, self.det)
        b, h, s, d = o.shape
        return self.wo(o.permute(0, 2, 1, 3).reshape(b, s, h * d))


class _FFN(nn.Module):
    def __init__(self, lut, d_ff, d_model, det):
        super().__init__()
        self.f1 = denseam(d_model, d_ff, activation="relu", mant_mul_lut=lut, deterministic=det)
        self.f2 = denseam(d_ff, d_model, mant_mul_lut=lut, deterministic=det)

    def forward(self, x):
        return self.f2(self.f1(x))


class _EncLayer(nn.Module):
    def __init__(self, lut, h, d_k, d_v, d_model, d_ff, det):
        super().__init__()
        self.mha = _MHA(lut, h, d_k, d_v, d_model, det)
        self.n1 = nn.LayerNorm(d_model, eps=1e-3)
        self.ffn = _FFN(lut, d_ff, d_model, det)
        self.n2 = nn.LayerNorm(d_model, eps=1e-3)

    def forward(self, x, pad_mask):
        x = self.n1(x + self.mha(x, x, x, pad_mask))
        return self.n2(x + self.ffn(x))


class _DecLayer(nn.Module):
    def __init__(self, lut, h, d_k, d_v, d_model, d_ff, det):
        super().__init__()
        self.mha1 = _MHA(lut, h, d_k, d_v, d_model, det)
        self.n1 = nn.LayerNorm(d_model, eps=1e-3)
        self.mha2 = _MHA(lut, h, d_k, d_v, d_model, det)
        self.ffn = _FFN(lut, d_ff, d_model, det)
        self.n3 = nn.LayerNorm(d_model, eps=1e-3)

    def forward(self, x, enc, look_mask, pad_mask):
        a1 = self.n1(x + self.mha1(x, x, x, look_mask))
        # the reference reuses add_norm1 for the second residual (ammha/decoder.py:41)
        a2 = self.n1(a1 + self.mha2(a1, enc, enc, pad_mask))
        return self.n3(a2 + self.ffn(a2))


class TransformerAM(nn.Module):
    def __init__(self, lut, vocab=8000, layers=6, d_model=512, heads=8, d_ff=2048, d_k=512, d_v=512,
                 deterministic=False):
        super().__init__()
        self.d_model = d_model
        self.src_emb = nn.Embedding(vocab, d_model, padding_idx=0)
        self.tgt_emb = nn.Embedding(vocab, d_model, padding_idx=0)
        self.register_buffer("pos", _sinusoid(2048, d_model), persistent=False)
        self.enc = nn.ModuleList([_EncLayer(lut, heads, d_k, d_v, d_model, d_ff, deterministic) for _ in range(layers)])
        self.dec = nn.ModuleList([_DecLayer(lut, heads, d_k, d_v, d_model, d_ff, deterministic) for _ in range(layers)])
        self.out = denseam(d_model, vocab, mant_mul_lut=lut, deterministic=deterministic)

    def _embed(self, emb, ids):
        return emb(ids) * math.sqrt(self.d_model) + self.pos[None, : ids.shape[1]]

    def forward(self, src, tgt):
        pad_src = (src == 0).float()[:, None, None, :]
        pad_tgt = (tgt == 0).float()[:, None, None, :]
        s = tgt.shape[1]
        look = torch.maximum(torch.triu(torch.ones(s, s, device=tgt.device), 1)[None, None], pad_tgt)
        x = self._embed(self.src_emb, src)
        for layer in self.enc:
            x = layer(x, pad_src)
        y = self._embed(self.tgt_emb, tgt)
        for layer in self.dec:
            y = layer(y, x, look, pad_src)
        return self.out(y)
