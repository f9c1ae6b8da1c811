"""ctypes binding of the C ABI in ``include/amsim.h``.

The library is the only implementation of these ops: if ``libamsim.so`` is
missing the import of this module raises, there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

from ._build import LIB_PATH

OK = 0
ERR_INVALID, ERR_LUT_NAME, ERR_LUT_IO, ERR_LUT_SIZE, ERR_CUDA, ERR_WORKSPACE, ERR_UNSUPPORTED = range(1, 8)
FAST = 0
DETERMINISTIC = 1
INT32 = 2
ACT_NONE, ACT_RELU = 0, 1
STATIC_SCRATCH_BYTES = 8 << 20

# every symbol include/amsim.h declares
EXPORTS = [
    "amsim_last_error", "amsim_version", "amsim_lut_open", "amsim_lut_open_bytes", "amsim_lut_close",
    "amsim_lut_info", "amsim_mul", "amsim_conv2d_geometry", "amsim_conv2d_fwd", "amsim_conv2d_fwd_bias_act",
    "amsim_dense_fwd_bias_act", "amsim_conv2d_fwd_scale_bias_act", "amsim_conv2d_bwd_input",
    "amsim_conv2d_bwd_filter_workspace", "amsim_conv2d_bwd_filter", "amsim_conv2d_bwd_filter_static",
    "amsim_dense_fwd",
    "amsim_dense_bwd_weight_workspace", "amsim_dense_bwd_weight", "amsim_dense_bwd_input", "amsim_matmul",
    "amsim_matmul_ex", "amsim_bias_grad_workspace", "amsim_bias_grad",
    "amsim_debug_fastdiv", "amsim_debug_launch_count", "amsim_debug_reload_env", "amsim_debug_bounds_report",
]


class AmsimError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"amsim error {code}: {message}")
        self.code = code
        self.message = message


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m approxtrain_b200._build` "
            "(nvcc, sm_100a).  There is no fallback implementation.")
    L = C.CDLL(LIB_PATH)
    vp, ip, fp, sz, u = C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_uint
    L.amsim_last_error.restype = C.c_char_p
    L.amsim_version.restype = C.c_char_p
    L.amsim_lut_open.argtypes = [C.c_char_p, ip, C.POINTER(vp)]
    L.amsim_lut_open_bytes.argtypes = [C.c_char_p, ip, ip, C.POINTER(vp)]
    L.amsim_lut_close.argtypes = [vp]
    L.amsim_lut_info.argtypes = [vp, C.POINTER(ip), C.POINTER(C.c_uint32), C.POINTER(ip), C.POINTER(ip), C.POINTER(vp)]
    L.amsim_mul.argtypes = [vp, vp, fp, fp, fp, sz]
    L.amsim_conv2d_geometry.argtypes = [ip] * 7 + [C.POINTER(ip)] * 4
    conv_dims = [ip] * 13
    L.amsim_conv2d_fwd.argtypes = [vp, vp, fp, fp, fp] + conv_dims + [u]
    L.amsim_conv2d_fwd_bias_act.argtypes = [vp, vp, fp, fp, fp, fp] + conv_dims + [ip, u]
    L.amsim_dense_fwd_bias_act.argtypes = [vp, vp, fp, fp, fp, fp, ip, ip, ip, ip, u]
    L.amsim_conv2d_fwd_scale_bias_act.argtypes = [vp, vp, fp, fp, fp, fp, fp] + conv_dims + [ip, u]
    L.amsim_conv2d_bwd_input.argtypes = [vp, vp, fp, fp, fp] + conv_dims + [u]
    L.amsim_conv2d_bwd_filter_workspace.argtypes = [ip] * 9 + [u]
    L.amsim_conv2d_bwd_filter_workspace.restype = sz
    L.amsim_conv2d_bwd_filter.argtypes = [vp, vp, fp, fp, fp] + conv_dims + [vp, sz, u]
    L.amsim_conv2d_bwd_filter_static.argtypes = [vp, vp, fp, fp, fp] + conv_dims + [u]
    L.amsim_dense_fwd.argtypes = [vp, vp, fp, fp, fp, ip, ip, ip, u]
    L.amsim_dense_bwd_weight_workspace.argtypes = [ip, ip, ip, u]
    L.amsim_dense_bwd_weight_workspace.restype = sz
    L.amsim_dense_bwd_weight.argtypes = [vp, vp, fp, fp, fp, ip, ip, ip, vp, sz, u]
    L.amsim_dense_bwd_input.argtypes = [vp, vp, fp, fp, fp, ip, ip, ip, u]
    L.amsim_matmul.argtypes = [vp, vp, fp, fp, fp] + [ip] * 6 + [u]
    L.amsim_matmul_ex.argtypes = [vp, vp, fp, fp, fp] + [ip] * 8 + [C.POINTER(C.c_float), u]
    L.amsim_bias_grad_workspace.argtypes = [C.c_longlong, ip]
    L.amsim_bias_grad_workspace.restype = sz
    L.amsim_bias_grad.argtypes = [vp, fp, fp, C.c_longlong, ip, vp, sz]
    L.amsim_debug_fastdiv.argtypes = [C.c_uint32, C.c_uint32]
    L.amsim_debug_fastdiv.restype = C.c_uint32
    L.amsim_debug_launch_count.argtypes = []
    L.amsim_debug_launch_count.restype = C.c_ulonglong
    L.amsim_debug_bounds_report.argtypes = [C.POINTER(C.c_ulonglong)]
    L.amsim_debug_reload_env.argtypes = []
    L.amsim_debug_reload_env.restype = None
    return L


lib = _load()


def check(code: int) -> None:
    if code != OK:
        raise AmsimError(code, lib.amsim_last_error().decode("utf-8", "replace"))
