"""ctypes binding of libqwcuda.so (the C ABI declared in include/qwc.h).

There is no CPU fallback: if the shared library is missing, or a kernel is
asked to run without a B200, the call raises.
"""
from __future__ import annotations

import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libqwcuda.so")

OK, ERR_BLOCKED, ERR_BAD_WEIGHTS, ERR_BAD_SHAPE, ERR_BAD_GEOMETRY, ERR_CUDA = range(6)
KIND_HQ4_G32_M5, KIND_ROTATED_HQ = 0, 1
F16, F32 = 0, 1
EPI_NONE, EPI_SILU_PAIR, EPI_SILU_PAIR_FWHT = 0, 1, 2
BACKEND_BLOCKED, BACKEND_STREAM_MMA, BACKEND_TCGEN05, BACKEND_ROWWISE = 0, 1, 2, 3


class WeightViewC(ctypes.Structure):
    _fields_ = [("blocks", ctypes.c_void_p), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
                ("kind", ctypes.c_int32), ("bits", ctypes.c_int32), ("group", ctypes.c_int32)]


class PlanC(ctypes.Structure):
    _fields_ = [("family", ctypes.c_int32), ("backend", ctypes.c_int32), ("epilogue", ctypes.c_int32),
                ("threads_per_cta", ctypes.c_int32), ("kernel", ctypes.c_char * 48)]


# Every symbol include/qwc.h declares: name -> (restype, argtypes).
_i32, _i64, _vp, _sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t
_WV = ctypes.POINTER(WeightViewC)
SIGNATURES = {
    "qwc_hal_create": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(_vp)]),
    "qwc_hal_destroy": (None, [_vp]),
    "qwc_last_error": (ctypes.c_char_p, []),
    "qwc_hal_device_status": (ctypes.c_int, [_vp, ctypes.POINTER(_i32)]),
    "qwc_sm_count": (ctypes.c_int, [_vp]),
    "qwc_hal_set_static_weights": (ctypes.c_int, [_vp, _i32]),
    "qwc_weight_view_init": (ctypes.c_int, [_WV, _vp, _sz, _i64, _i64, _i32, _i32, _i32]),
    "qwc_block_bytes": (_i64, [_i32, _i32, _i32]),
    "qwc_gemm_plan": (ctypes.c_int, [_i64, _i64, _i64, _i32, _i32, _i32, _i32, _i64, ctypes.POINTER(PlanC)]),
    "qwc_fwht32_f16": (ctypes.c_int, [_vp, _vp, _vp, _i64]),
    "qwc_cast_f32_to_f16": (ctypes.c_int, [_vp, _vp, _vp, _vp, _i64]),
    "qwc_head_argmax": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "qwc_rmsnorm_fwht": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_float, _i32]),
    "qwc_dequant": (ctypes.c_int, [_vp, _vp, _WV, _vp, _i32, _i32]),
    "qwc_quantize": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _vp]),
    "qwc_gemm": (ctypes.c_int, [_vp, _vp, _WV, _vp, _i64, _i64, _vp, _i32, _i64, _i32, _i32, _vp, _sz]),
    "qwc_gemm_workspace_bytes": (_sz, [_vp, _WV, _i64, _i32, _i32]),
    "qwc_gemm_f32": (ctypes.c_int, [_vp, _vp, _WV, _vp, _i64, _i64, _vp, _i32, _i64, _i32, ctypes.c_float, _i32, _vp, _sz]),
    "qwc_gemm_f32_workspace_bytes": (_sz, [_vp, _WV, _i64, _i32]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load libqwcuda.so; raises if it was not built (python -m qwegn_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m qwegn_b200.build`. "
                "This package has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def register(name: str, restype, argtypes) -> None:
    """Declare one more exported symbol (used by the optional modules)."""
    SIGNATURES[name] = (restype, argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = restype
        fn.argtypes = argtypes


def last_error() -> str:
    return load().qwc_last_error().decode("utf-8", "replace")
