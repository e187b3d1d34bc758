"""Host-side mirror of the reference's QWGEMM operator surface over the C ABI.

Names follow Sources/Operators/QWGEMM/QWGemm.swift: `QWGemm.plan`,
`QWGemm.encode`, `QWGemm.encodeH16`, `QWGemm.encodeFwht32`, `QWGemmError`,
`QWWeightView`.  An encoder is a CUDA stream, a tensor value is a torch CUDA
tensor (torch is used for device memory and streams only; every kernel is in
libqwcuda.so).  Encode calls allocate nothing: the caller passes the output.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import (EPI_NONE, EPI_SILU_PAIR, EPI_SILU_PAIR_FWHT, F16, F32, KIND_HQ4_G32_M5, KIND_ROTATED_HQ,
                   PlanC, WeightViewC)

_CODE_NAMES = {1: "f3Blocked", 2: "badWeights", 3: "badShape", 4: "badGeometry", 5: "cuda"}


class QWGemmError(RuntimeError):
    """QWGemmError (QWGemm.swift:66-80): .f3Blocked / .badWeights / .badShape / .badGeometry, plus .cuda."""

    def __init__(self, code: int, message: str):
        self.code = code
        self.case = _CODE_NAMES.get(code, f"code{code}")
        super().__init__(f"QWGEMM: {self.case} - {message}")


def _check(rc: int) -> None:
    if rc != 0:
        raise QWGemmError(rc, _lib.last_error())


@dataclass(frozen=True)
class ContainerKind:
    """QWWeightView.ContainerKind (Sources/Foundation/QWAlloc/QWWeightView.swift:11-31)."""
    kind: int
    bits: int
    group: int

    @property
    def block_bytes(self) -> int:
        return 20 if self.kind == KIND_HQ4_G32_M5 else self.group * self.bits // 8 + 4

    def row_bytes(self, k: int) -> int:
        return (k // self.group) * self.block_bytes


incumbentHQ4G32 = ContainerKind(KIND_HQ4_G32_M5, 4, 32)


def rotatedHQ(bits: int, group: int) -> ContainerKind:
    return ContainerKind(KIND_ROTATED_HQ, bits, group)


CONTAINERS = {"HQ4_G32": incumbentHQ4G32, "HQ8_G32": rotatedHQ(8, 32), "HQ4_G64": rotatedHQ(4, 64)}


class QWHal:
    """Device context: stands where QWHal (Sources/Foundation/QWHAL/QWHal.swift:81-235) stands in the reference."""

    def __init__(self, device: int = 0):
        lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("qwegn_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        torch.cuda.init()
        h = ctypes.c_void_p()
        _check(lib.qwc_hal_create(device, ctypes.byref(h)))
        self._h = h
        self._lib = lib

    @property
    def handle(self) -> ctypes.c_void_p:
        return self._h

    @property
    def sm_count(self) -> int:
        return int(self._lib.qwc_sm_count(self._h))

    def set_static_weights(self, enabled: bool = True) -> None:
        """Promise that weight banks are load-time data (never written by in-flight work): the decode kernels then
        prefetch their weights while the previous kernel of the stream is finishing."""
        _check(self._lib.qwc_hal_set_static_weights(self._h, int(enabled)))

    def device_status(self) -> int:
        """Synchronise and return the kernels' status word (0 = no bounded wait gave up)."""
        out = ctypes.c_int32(0)
        _check(self._lib.qwc_hal_device_status(self._h, ctypes.byref(out)))
        return int(out.value)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.qwc_hal_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> ctypes.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def check_matmul_tensors(hal: "QWHal", w: "QWWeightView", x: torch.Tensor, y: torch.Tensor, epi: int, x_dtype=torch.float16):
    """The tensor checks every matmul door makes before it hands raw pointers to the C ABI (the C side sees only
    pointers and strides, so a CPU tensor, a tensor on another device or a short y must be refused here): returns
    (x2, y2, m, n_out, ldx, ldy)."""
    if x.dtype != x_dtype or not x.is_cuda:
        raise QWGemmError(3, f"x must be a CUDA {x_dtype} tensor")
    if y.dtype not in (torch.float16, torch.float32) or not y.is_cuda:
        raise QWGemmError(3, "y must be a CUDA float16/float32 tensor")
    if x.device != hal.device or y.device != hal.device or w.bank.device != hal.device:
        raise QWGemmError(3, f"x, y and the weight bank must live on {hal.device}")
    if x.dim() not in (1, 2) or y.dim() not in (1, 2):
        raise QWGemmError(3, "x and y must be vectors or matrices")
    x2 = x if x.dim() == 2 else x.view(1, -1)
    y2 = y if y.dim() == 2 else y.view(1, -1)
    if x2.stride(1) != 1 or y2.stride(1) != 1:
        raise QWGemmError(3, "x and y rows must be contiguous")
    m = x2.shape[0]
    if x2.shape[1] != w.k:
        raise QWGemmError(3, f"x has {x2.shape[1]} columns, the bank has k={w.k}")
    n_out = w.n if epi == EPI_NONE else w.n // 2
    if y2.shape[0] != m or y2.shape[1] != n_out:
        raise QWGemmError(3, f"y is {tuple(y2.shape)}, expected ({m}, {n_out})")
    ldx = x2.stride(0) if m > 1 else max(x2.stride(0), w.k)
    ldy = y2.stride(0) if m > 1 else max(y2.stride(0), n_out)
    if m > 1 and (ldx < w.k or ldy < n_out):
        raise QWGemmError(3, "row strides smaller than the row length (overlapping rows)")
    return x2, y2, m, n_out, ldx, ldy


def check_device_tensor(hal: "QWHal", t: torch.Tensor, name: str, dtype, numel: Optional[int] = None, contiguous: bool = True):
    """One buffer of an MoE door: right device, dtype, layout and (when given) at least `numel` elements."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.device != hal.device:
        raise QWGemmError(3, f"{name} must be a CUDA tensor on {hal.device}")
    dts = dtype if isinstance(dtype, (tuple, list)) else (dtype,)
    if t.dtype not in dts:
        raise QWGemmError(3, f"{name} must be {' or '.join(str(d) for d in dts)}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise QWGemmError(3, f"{name} must be contiguous")
    if numel is not None and t.numel() < numel:
        raise QWGemmError(3, f"{name} holds {t.numel()} elements, {numel} needed")


class QWWeightView:
    """QWWeightView (QWWeightView.swift:9-152): one bank of packed blocks resident in device memory."""

    def __init__(self, blocks: torch.Tensor, n: int, k: int, container: ContainerKind = incumbentHQ4G32,
                 byte_offset: int = 0):
        if blocks.dtype != torch.uint8 or not blocks.is_cuda or not blocks.is_contiguous():
            raise QWGemmError(2, "blocks must be a contiguous CUDA uint8 tensor")
        self.bank = blocks
        self.container = container
        self.c = WeightViewC()
        avail = blocks.numel() - byte_offset
        if avail < 0:
            raise QWGemmError(2, "byte offset beyond the bank")
        _check(_lib.load().qwc_weight_view_init(ctypes.byref(self.c), ctypes.c_void_p(blocks.data_ptr() + byte_offset),
                                                avail, n, k, container.kind, container.bits, container.group))

    @property
    def n(self) -> int:
        return int(self.c.n)

    @property
    def k(self) -> int:
        return int(self.c.k)

    @property
    def isRotated(self) -> bool:
        return True

    def rows(self, r0: int, r1: int) -> "QWWeightView":
        """A view of rows [r0, r1) (column-parallel shard, or one expert of a stacked bank)."""
        rb = self.container.row_bytes(self.k)
        base = self.c.blocks - self.bank.data_ptr()
        return QWWeightView(self.bank, r1 - r0, self.k, self.container, byte_offset=base + r0 * rb)


@dataclass(frozen=True)
class QWGemmPlan:
    family: int
    backend: int
    epilogue: int
    threadsPerTG: int
    kernel: str


class QWGemm:
    """The matmul door (QWGemm.swift:82-330)."""

    @staticmethod
    def plan(m: int, n: int, k: int, container: ContainerKind = incumbentHQ4G32, epi: int = EPI_NONE,
             vocab: int = 0) -> QWGemmPlan:
        out = PlanC()
        _check(_lib.load().qwc_gemm_plan(m, n, k, container.kind, container.bits, container.group, epi, vocab,
                                         ctypes.byref(out)))
        return QWGemmPlan(out.family, out.backend, out.epilogue, out.threads_per_cta, out.kernel.decode())

    @staticmethod
    def encode(hal: QWHal, w: QWWeightView, x: torch.Tensor, y: torch.Tensor, epi: int = EPI_NONE,
               x_is_rotated: bool = False, stream: Optional[torch.cuda.Stream] = None,
               workspace: Optional[torch.Tensor] = None) -> None:
        """y[m, n_out] = epilogue(rot(x) . W_rot^T).  x f16 [m, k] (or [k]); y f16/f32 [m, n_out] (or [n_out])."""
        x2, y2, m, n_out, ldx, ldy = check_matmul_tensors(hal, w, x, y, epi)
        ws_ptr, ws_bytes = None, 0
        if workspace is not None:
            check_device_tensor(hal, workspace, "workspace", workspace.dtype)
            ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
        _check(_lib.load().qwc_gemm(hal.handle, _stream_ptr(stream), ctypes.byref(w.c), x2.data_ptr(), m, ldx, y2.data_ptr(),
                                    F16 if y.dtype == torch.float16 else F32, ldy, epi, int(x_is_rotated), ws_ptr, ws_bytes))

    # The reference's f16-store door (QWGemm.swift:137) is the same call with an f16 output tensor.
    encodeH16 = encode

    @staticmethod
    def workspaceBytes(hal: QWHal, w: QWWeightView, m: int, epi: int = EPI_NONE, x_is_rotated: bool = False) -> int:
        return int(_lib.load().qwc_gemm_workspace_bytes(hal.handle, ctypes.byref(w.c), m, epi, int(x_is_rotated)))

    @staticmethod
    def f32WorkspaceBytes(hal: QWHal, w: QWWeightView, m: int, epi: int = 0) -> int:
        return int(_lib.load().qwc_gemm_f32_workspace_bytes(hal.handle, ctypes.byref(w.c), m, epi))

    @staticmethod
    def encodeHQ4F32V4(hal: QWHal, w: QWWeightView, x: torch.Tensor, y: torch.Tensor, rows: int = 1, epi: int = 0,
                       scale: float = 1.0, x_is_rotated: bool = True, workspace: Optional[torch.Tensor] = None,
                       stream: Optional[torch.cuda.Stream] = None) -> None:
        """f32-activation matmul (QWGemmF32.swift:143-199; encodeHQ4F32BM :309-350 is the same call with more rows).
        x f32 [rows, k] in the rotated basis (the reference's dataflow; x_is_rotated=False rotates here in f32);
        epi 0 none, 1 silu(y/scale), 2 sigmoid, 3 silu(y/scale) + FWHT-32; y f16/f32 [rows, n]."""
        if x.dtype != torch.float32 or not x.is_cuda or y.dtype not in (torch.float16, torch.float32) or not y.is_cuda:
            raise QWGemmError(3, "x must be CUDA float32, y CUDA float16/float32")
        x2 = x if x.dim() == 2 else x.view(1, -1)
        y2 = y if y.dim() == 2 else y.view(1, -1)
        if x2.stride(1) != 1 or y2.stride(1) != 1 or x2.shape[0] != rows or y2.shape[0] != rows:
            raise QWGemmError(3, "x and y must hold `rows` contiguous rows")
        if x2.shape[1] != w.k or y2.shape[1] != w.n:
            raise QWGemmError(3, f"x is {tuple(x2.shape)}, y {tuple(y2.shape)}; the bank is n={w.n}, k={w.k}")
        if workspace is None:
            raise QWGemmError(3, "the f32 door needs a workspace of f32WorkspaceBytes() bytes")
        _check(_lib.load().qwc_gemm_f32(hal.handle, _stream_ptr(stream), ctypes.byref(w.c), x2.data_ptr(), rows,
                                        x2.stride(0) if rows > 1 else w.k, y2.data_ptr(),
                                        F16 if y.dtype == torch.float16 else F32, y2.stride(0) if rows > 1 else w.n,
                                        epi, float(scale), int(x_is_rotated), workspace.data_ptr(),
                                        workspace.numel() * workspace.element_size()))

    encodeHQ4F32BM = encodeHQ4F32V4

    @staticmethod
    def encodeFwht32(hal: QWHal, x: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
        """In-place activation rotation (QWGemm.swift:285-300)."""
        if x.dtype != torch.float16 or not x.is_cuda or not x.is_contiguous():
            raise QWGemmError(3, "x must be a contiguous CUDA float16 tensor")
        _check(_lib.load().qwc_fwht32_f16(hal.handle, _stream_ptr(stream), x.data_ptr(), x.numel()))

    @staticmethod
    def encodeCast(hal: QWHal, x32: torch.Tensor, y16: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
        """f32 -> f16 cast seam (QWGemm.swift:302-320)."""
        if x32.dtype != torch.float32 or y16.dtype != torch.float16 or not x32.is_contiguous() or not y16.is_contiguous():
            raise QWGemmError(2, "cast takes contiguous f32 in, f16 out")
        if y16.numel() < x32.numel():
            raise QWGemmError(2, "cast output too small")
        _check(_lib.load().qwc_cast_f32_to_f16(hal.handle, _stream_ptr(stream), x32.data_ptr(), y16.data_ptr(), x32.numel()))

    @staticmethod
    def encodeArgmax(hal: QWHal, logits: torch.Tensor, tokens: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Greedy token per row of f32 logits [rows, vocab] in the reference's key order (QWGemmF32.swift:201-307)."""
        if logits.dtype != torch.float32 or tokens.dtype != torch.int32 or not logits.is_cuda or logits.stride(-1) != 1:
            raise QWGemmError(3, "logits must be CUDA float32 with contiguous rows, tokens int32")
        l2 = logits if logits.dim() == 2 else logits.view(1, -1)
        _check(_lib.load().qwc_head_argmax(hal.handle, _stream_ptr(stream), l2.data_ptr(), l2.stride(0) if l2.shape[0] > 1 else l2.shape[1],
                                           l2.shape[0], l2.shape[1], tokens.data_ptr()))

    @staticmethod
    def encodeRMSNorm(hal: QWHal, x: torch.Tensor, gamma: torch.Tensor, out: torch.Tensor, eps: float = 1e-6,
                      residual: Optional[torch.Tensor] = None, rotate: bool = True,
                      stream: Optional[torch.cuda.Stream] = None) -> None:
        """RMSNorm with (1 + gamma) and rotated f16 output, optionally fused with residual += x (the driver's
        encodeRMSNormFast / encodeRMSNormResidualFast, Sources/Runtime/QWEngine/Driver/EncodeKernels.swift:339-404).
        Feed `out` to encode(..., x_is_rotated=True)."""
        for t in (x, gamma, out) + ((residual,) if residual is not None else ()):
            if t.dtype != torch.float16 or not t.is_cuda or not t.is_contiguous():
                raise QWGemmError(3, "norm tensors must be contiguous CUDA float16")
        x2 = x if x.dim() == 2 else x.view(1, -1)
        rows, hidden = x2.shape
        if gamma.numel() != hidden or out.numel() != x.numel() or (residual is not None and residual.numel() != x.numel()):
            raise QWGemmError(3, "shape mismatch")
        _check(_lib.load().qwc_rmsnorm_fwht(hal.handle, _stream_ptr(stream), x.data_ptr(), gamma.data_ptr(), out.data_ptr(),
                                            None if residual is None else residual.data_ptr(), rows, hidden, float(eps),
                                            int(rotate)))

    @staticmethod
    def dequant(hal: QWHal, w: QWWeightView, out: torch.Tensor, standard_domain: bool = False,
                stream: Optional[torch.cuda.Stream] = None) -> None:
        """Device twin of Pack.dequantHQ4Slab / dequantHQBlockSlab (Sources/Foundation/QWQuant/QWPack.swift:205-321)."""
        if out.dtype not in (torch.float16, torch.float32) or not out.is_cuda or not out.is_contiguous():
            raise QWGemmError(3, "out must be a contiguous CUDA float16/float32 tensor")
        if out.numel() != w.n * w.k:
            raise QWGemmError(3, f"out has {out.numel()} elements, expected {w.n * w.k}")
        _check(_lib.load().qwc_dequant(hal.handle, _stream_ptr(stream), ctypes.byref(w.c), out.data_ptr(),
                                       F16 if out.dtype == torch.float16 else F32, int(standard_domain)))

    @staticmethod
    def quantize(hal: QWHal, w: torch.Tensor, container: ContainerKind = incumbentHQ4G32,
                 out: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """Load-time quantizer (HQ4Quantizer in Sources/Foundation/QWLoad; Scripts/quantize/hq4.py:54-123):
        f32 [n, k] on the device -> packed blocks, byte-identical to the reference's Python packer."""
        if w.dtype != torch.float32 or not w.is_cuda or not w.is_contiguous() or w.dim() != 2:
            raise QWGemmError(3, "w must be a contiguous 2-D CUDA float32 tensor")
        n, k = w.shape
        if k % container.group:
            raise QWGemmError(2, f"k={k} is not a multiple of group {container.group}")
        nbytes = n * container.row_bytes(k)
        if out is None:
            out = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
        if out.dtype != torch.uint8 or out.numel() < nbytes or not out.is_contiguous():
            raise QWGemmError(3, "out must be a contiguous uint8 tensor large enough for the bank")
        _check(_lib.load().qwc_quantize(hal.handle, _stream_ptr(stream), w.data_ptr(), n, k, container.kind,
                                        container.bits, container.group, out.data_ptr()))
        return out
