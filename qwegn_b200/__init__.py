"""qwegn_b200: B200 (sm_100a) kernels for the reference's quantized-matmul hot path, behind a C ABI.

The kernels live in libqwcuda.so (sources in qwegn_b200/csrc, ABI in include/qwc.h).  This package is the
host-side mirror of the reference's operator interface for that path; it has no CPU or PyTorch fallback.
"""
from ._lib import (EPI_NONE, EPI_SILU_PAIR, EPI_SILU_PAIR_FWHT, F16, F32, KIND_HQ4_G32_M5, KIND_ROTATED_HQ,
                   LIB_PATH)
from .gemm import (CONTAINERS, ContainerKind, QWGemm, QWGemmError, QWGemmPlan, QWHal, QWWeightView,
                   incumbentHQ4G32, rotatedHQ)
from .moe import QWGemmMoE, QWMoEOperator
from . import noalloc  # noqa: F401  (registers qwc_gemm_static_scratch)

__all__ = [
    "EPI_NONE", "EPI_SILU_PAIR", "EPI_SILU_PAIR_FWHT", "F16", "F32", "KIND_HQ4_G32_M5", "KIND_ROTATED_HQ",
    "LIB_PATH", "CONTAINERS", "ContainerKind", "QWGemm", "QWGemmError", "QWGemmPlan", "QWHal", "QWWeightView",
    "incumbentHQ4G32", "rotatedHQ", "QWGemmMoE", "QWMoEOperator",
]
