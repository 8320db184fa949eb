"""ctypes binding of the C ABI in ``include/inferno_b200_attn.h``.

The library is required: importing this module where the shared object has not been
built raises, and no operation falls back to another implementation.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

OK = 0
ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_MISALIGNED, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_NO_DEVICE, ERR_TOO_LARGE = range(1, 9)
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024
DTYPE_F32, DTYPE_BF16 = 0, 1
MATH_SPLIT_BF16 = 0
PASS_FWD, PASS_BWD = 0, 1

EXPORTS = (
    "ib200_attn_workspace_bytes", "ib200_attn_fwd", "ib200_attn_bwd", "ib200_attn_check",
    "ib200_status_string", "ib200_last_cuda_error", "ib200_version", "ib200_attn_set_timing_events", "ib200_attn_bwd_static", "ib200_attn_fwd_strided", "ib200_attn_bwd_strided", "ib200_gemm_bf16", "ib200_linear_fwd", "ib200_linear_bwd",
    "ib200_cast_f32_to_bf16", "ib200_cast_bf16_to_f32", "ib200_attn_item_order", "ib200_attn_check_static",
    "ib200_selftest_wait_expiry",
)



class Layout(ctypes.Structure):
    """``ib200_layout``: element strides of the batch, head and token axes of a [B, H, T, D] operand."""
    _fields_ = [("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64), ("stride_t", ctypes.c_int64)]


_lib = None


class Ib200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        detail = f", cudaError {lib().ib200_last_cuda_error()}" if status == ERR_CUDA else ""
        super().__init__(f"{where}: {status_string(status)} (status {status}{detail})")


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = os.environ.get("IB200_LIB") or _build.LIB_PATH      # IB200_LIB: another build of the same library (e.g. the bounds-checked one)
        if not os.path.isfile(path):
            raise ImportError(
                f"{path} is missing: build it with `python -m inferno_b200.build` (there is no fallback path)")
        L = ctypes.CDLL(path)
        vp, i, f, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
        L.ib200_attn_workspace_bytes.argtypes = [i, i, i, i, i, i, ctypes.POINTER(sz)]
        L.ib200_attn_workspace_bytes.restype = i
        L.ib200_attn_fwd.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, f, i, i, i, vp, sz, vp]
        L.ib200_attn_fwd.restype = i
        L.ib200_attn_bwd.argtypes = [vp] * 9 + [i, i, i, i, f, i, i, i, vp, sz, vp]
        L.ib200_attn_bwd.restype = i
        lp = ctypes.POINTER(Layout)
        L.ib200_attn_fwd_strided.argtypes = [vp, vp, vp, vp, vp, lp, lp, lp, lp, i, i, i, i, f, i, i, i, vp, sz, vp]
        L.ib200_attn_fwd_strided.restype = i
        L.ib200_attn_bwd_strided.argtypes = [vp] * 9 + [lp] * 8 + [i, i, i, i, f, i, i, i, vp, sz, vp]
        L.ib200_attn_bwd_strided.restype = i
        L.ib200_attn_bwd_static.argtypes = [vp] * 9 + [i, i, i, i, f, i, i, i, vp]
        L.ib200_attn_bwd_static.restype = i
        L.ib200_gemm_bf16.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp]
        L.ib200_gemm_bf16.restype = i
        L.ib200_linear_fwd.argtypes = [vp, vp, vp, vp, i, i, i, vp]
        L.ib200_linear_fwd.restype = i
        L.ib200_linear_bwd.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, vp]
        L.ib200_linear_bwd.restype = i
        L.ib200_cast_f32_to_bf16.argtypes = [vp, vp, sz, vp]
        L.ib200_cast_f32_to_bf16.restype = i
        L.ib200_cast_bf16_to_f32.argtypes = [vp, vp, sz, vp]
        L.ib200_cast_bf16_to_f32.restype = i
        ip = ctypes.POINTER(ctypes.c_int)
        L.ib200_attn_item_order.argtypes = [i, i, i, i, i, i, ip, ip, i, ip]
        L.ib200_attn_item_order.restype = i
        L.ib200_attn_check.argtypes = [vp, vp, ctypes.POINTER(i)]
        L.ib200_attn_check.restype = i
        L.ib200_attn_check_static.argtypes = [vp, ctypes.POINTER(i)]
        L.ib200_attn_check_static.restype = i
        L.ib200_selftest_wait_expiry.argtypes = [vp, sz, ctypes.c_uint, vp]
        L.ib200_selftest_wait_expiry.restype = i
        L.ib200_attn_set_timing_events.argtypes = [vp, vp, vp, vp]
        L.ib200_attn_set_timing_events.restype = i
        L.ib200_status_string.argtypes = [i]
        L.ib200_status_string.restype = ctypes.c_char_p
        L.ib200_last_cuda_error.restype = i
        L.ib200_version.restype = i
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().ib200_status_string(int(status)).decode()


def workspace_bytes(B: int, H: int, T: int, D: int, dtype: int, pass_: int) -> int:
    out = ctypes.c_size_t(0)
    rc = lib().ib200_attn_workspace_bytes(B, H, T, D, dtype, pass_, ctypes.byref(out))
    if rc != OK:
        raise Ib200Error(rc, "ib200_attn_workspace_bytes")
    return int(out.value)
