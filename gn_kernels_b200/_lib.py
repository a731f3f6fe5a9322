"""ctypes binding of libgnk.so (the C ABI declared in include/gnk.h).

There is no fallback: if the library cannot be loaded (and cannot be built because nvcc
is missing) importing an op raises.  Status codes become Python exceptions here.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

from . import build as _build

_lib = None

# enums of include/gnk.h
BF16, F16, F32 = 0, 1, 2
Q_INT8, Q_E4M3, Q_E5M2, Q_E2M1, Q_BF16, Q_F16 = 0, 1, 2, 3, 4, 5
MX_OCP, MX_NV = 0, 1
OUT_BF16, OUT_I32 = 0, 1

ERR_BAD_ARG, ERR_BAD_SHAPE, ERR_BAD_ALIGN, ERR_ARCH, ERR_CUDA, ERR_TIMEOUT, ERR_TOO_LARGE, ERR_UNSUPPORTED = range(-1, -9, -1)

_P = c_void_p
_SIGNATURES = {
    "gnk_version": (c_int, []),
    "gnk_strerror": (c_char_p, [c_int]),
    "gnk_last_cuda_error": (c_char_p, []),
    "gnk_device_status": (c_int, [POINTER(c_int), POINTER(c_uint32), c_int]),
    "gnk_absmax_scratch_bytes": (c_size_t, [c_int64]),
    "gnk_absmax": (c_int, [_P, c_int, c_int64, c_float, _P, _P, _P]),
    "gnk_absmax_static_max_elems": (c_int64, []),
    "gnk_absmax_static": (c_int, [_P, c_int, c_int64, c_float, _P, _P]),
    "gnk_quant_rowwise": (c_int, [_P, c_int, c_int64, c_int64, c_int64, c_int, _P, _P, c_int64, c_int64, _P]),
    "gnk_quant_mx": (c_int, [_P, c_int, c_int64, c_int64, c_int64, c_int, c_int, _P, _P, c_int, _P]),
    "gnk_quant_nvfp4": (c_int, [_P, c_int, c_int64, c_int64, c_int64, _P, c_float, _P, _P, c_int, _P]),
    "gnk_sf_swizzle": (c_int, [_P, _P, c_int64, c_int64, c_int, _P]),
    "gnk_dequant_block": (c_int, [_P, _P, c_int64, c_int64, c_int, c_int, _P, _P, _P]),
    "gnk_mm_bf16": (c_int, [_P, c_int64, _P, c_int64, _P, c_int64, c_int64, c_int64, c_int64, _P]),
    "gnk_mm_f16": (c_int, [_P, c_int64, _P, c_int64, _P, c_int64, c_int64, c_int64, c_int64, c_int, _P]),
    "gnk_mm_i8": (c_int, [_P, c_int64, _P, c_int64, _P, c_int64, c_int64, c_int64, c_int64, _P, _P, _P, c_int, _P]),
    "gnk_mm_f8": (c_int, [_P, c_int64, _P, c_int64, _P, c_int64, c_int64, c_int64, c_int64, _P, _P, _P, _P]),
    "gnk_mm_mxfp8": (c_int, [_P, c_int64, _P, c_int64, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, _P]),
    "gnk_mm_nvfp4": (c_int, [_P, c_int64, _P, c_int64, _P, _P, c_float, _P, c_int64, c_int64, c_int64, c_int64, _P]),
    "gnk_gated_mm_nvfp4": (c_int, [_P, c_int64, _P, _P, _P, _P, _P, _P, _P, _P, c_int64, _P, _P, c_int64, _P, c_int64, c_int64, c_int64, _P]),
    "gnk_attn_fwd": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                             POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), c_int, _P]),
    "gnk_attn_varlen_fwd": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                    POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), POINTER(c_int64), c_int, _P]),
    "gnk_mm_f8_block128": (c_int, [_P, c_int64, _P, c_int64, _P, c_int64, _P, c_int64, _P, _P, c_int64, _P, c_int64, c_int64, c_int64, c_int64, _P]),
    "gnk_gemm_rs_flag_words": (c_int64, [c_int64, c_int64, c_int]),
    "gnk_gemm_rs_plan": (c_int64, [c_int64, c_int64, c_int, c_int, c_int64, POINTER(c_int32)]),
    "gnk_gemm_rs_bf16": (c_int, [_P, c_int64, _P, c_int64, POINTER(c_void_p), POINTER(c_void_p), _P, c_int64, c_int64, c_int64,
                                 c_int64, c_int, c_int, c_uint32, c_int, _P]),
    "gnk_gemm_rs_bf16_pull": (c_int, [_P, c_int64, _P, c_int64, POINTER(c_void_p), _P, POINTER(c_void_p), _P, c_int64, c_int64,
                                      c_int64, c_int64, c_int, c_int, c_uint32, c_int, _P]),
    "gnk_gemm_rs_f8": (c_int, [_P, c_int64, _P, c_int64, c_float, POINTER(c_void_p), _P, POINTER(c_void_p), _P, c_int64, c_int64,
                               c_int64, c_int64, c_int, c_int, c_uint32, c_int, _P]),
    "gnk_gemm_ar_bf16": (c_int, [_P, c_int64, _P, c_int64, POINTER(c_void_p), _P, POINTER(c_void_p), _P, _P, c_int64, c_int64,
                                 c_int64, c_int64, c_int, c_int, c_uint32, _P]),
    "gnk_debug_attn_trace": (c_int, [_P]),
    "gnk_debug_force_tile": (c_int, [c_int]),
    "gnk_debug_staged": (c_int, [c_int]),
    "gnk_debug_rs_trace": (c_int, [_P]),
    "gnk_debug_max_clusters": (c_int, [c_int]),
    "gnk_debug_trace": (c_int, [_P]),
    "gnk_debug_deep_stage": (c_int, [c_int]),
    "gnk_debug_stage_plan": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int32)]),
}


class GnkError(RuntimeError):
    def __init__(self, code: int, where: str, text: str):
        super().__init__(f"{where}: {text} (gnk status {code})")
        self.code = code


def lib() -> ctypes.CDLL:
    """Loads (building first if sources are newer and nvcc exists) and returns the library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if _build.find_nvcc() is not None and _build.is_stale():
        _build.build()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing and nvcc is not available to build it; "
            "gn_kernels_b200 has no fallback path (run `python -m gn_kernels_b200.build` on a machine with CUDA 12.9+)"
        )
    handle = ctypes.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return handle


def check(code: int, where: str) -> None:
    if code == 0:
        return
    l = lib()
    text = l.gnk_strerror(code).decode()
    if code == ERR_CUDA:
        text += ": " + l.gnk_last_cuda_error().decode()
    if code in (ERR_BAD_ARG, ERR_BAD_SHAPE, ERR_BAD_ALIGN, ERR_TOO_LARGE):
        raise ValueError(f"{where}: {text} (gnk status {code})")
    raise GnkError(code, where, text)


def device_status(clear: bool = True) -> tuple[int, int]:
    """(status, detail) of the sticky device-side status word; synchronises the device."""
    st, detail = c_int(0), c_uint32(0)
    check(lib().gnk_device_status(ctypes.byref(st), ctypes.byref(detail), int(clear)), "gnk_device_status")
    return st.value, detail.value


def raise_on_device_error() -> None:
    st, detail = device_status(clear=True)
    if st != 0:
        raise GnkError(st, "device", f"{lib().gnk_strerror(st).decode()} (detail 0x{detail:08x})")
