"""Binding of qwc_gemm_static_scratch: the small-M matmul door that brings its own scratch.

For hosts that cannot allocate device memory at the call site (an engine with a frozen arena, a latency-critical
thread, a fully committed memory budget).  Scratch, when the call needs any, is a fixed 2 MiB array inside the
library; larger needs are refused.  The first call on a device must happen outside stream capture; calls that could
overlap on the GPU share that array and must be ordered by the caller."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from ._lib import EPI_NONE, F16, F32, WeightViewC
from .gemm import QWGemmError, QWHal, QWWeightView, _check, _stream_ptr, check_matmul_tensors

_i32, _i64, _vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p
_lib.register("qwc_gemm_static_scratch", ctypes.c_int,
              [_vp, _vp, ctypes.POINTER(WeightViewC), _vp, _i64, _i64, _vp, _i32, _i64, _i32, _i32])
_lib.register("qwc_static_scratch_capacity", ctypes.c_size_t, [])


def static_scratch_capacity() -> int:
    return int(_lib.load().qwc_static_scratch_capacity())


def encode_static_scratch(hal: QWHal, w: QWWeightView, x: torch.Tensor, y: torch.Tensor, epi: int = EPI_NONE,
                          x_is_rotated: bool = False, stream: Optional[torch.cuda.Stream] = None) -> None:
    """Same contract as QWGemm.encode for up to 16 tokens, without a workspace argument."""
    x2, y2, m, _, ldx, ldy = check_matmul_tensors(hal, w, x, y, epi)
    _check(_lib.load().qwc_gemm_static_scratch(
        hal.handle, _stream_ptr(stream), ctypes.byref(w.c), x2.data_ptr(), m, ldx, y2.data_ptr(),
        F16 if y.dtype == torch.float16 else F32, ldy, epi, int(x_is_rotated)))
