"""approxtrain_b200 — B200 (sm_100a) kernels for ApproxTrain's AM-Simulator
hot path: the LUT-based approximate FP32 multiply inside the AMConv2D,
denseam and MatMulAM GEMMs, behind the reference's operator interface.

``approxtrain_b200.ops`` mirrors the reference's TensorFlow custom ops on
torch CUDA tensors; the compute is in ``libamsim.so`` (C ABI in
``include/amsim.h``), which has to be built first
(``python -m approxtrain_b200._build``).  There is no CPU fallback.
"""
from ._build import build, LIB_PATH  # noqa: F401

__version__ = "0.1.0"
