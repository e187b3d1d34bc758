"""Host-side mirror of the reference's MoE operator (Sources/Operators/QWGEMM/QWMoEOperator.swift,
QWGemmMoE.swift, QWGemmMoERouter.swift) over the C ABI.  The caller owns all scratch
(`QWMoEOperator.Scratch`); nothing here allocates inside an encode call."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from ._lib import F16, F32, WeightViewC
from .gemm import QWGemmError, QWHal, QWWeightView, _check, _stream_ptr, check_device_tensor

_i32, _i64, _vp, _sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t
_WV = ctypes.POINTER(WeightViewC)


class MoeTileC(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("w_row0", "w_rows", "x_row0", "x_rows", "y_col0", "expert", "pad0", "pad1")]


_lib.register("qwc_moe_route", ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, ctypes.c_float, _vp, _vp])
_lib.register("qwc_moe_router_gemm", ctypes.c_int, [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _vp, _i32, _i64, _vp])
_lib.register("qwc_moe_group_pairs", ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _vp, _vp, _vp])
_lib.register("qwc_moe_max_tiles", _i64, [_i64, _i64, _i64])
_lib.register("qwc_moe_gather", ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _vp, _vp, _i64, _i64, _i32, _vp])
_lib.register("qwc_moe_grouped_gemm", ctypes.c_int, [_vp, _vp, _WV, _vp, _i64, _vp, _vp, _i64, _i32, _vp, _i32, _i64, _i32])
_lib.register("qwc_moe_tile_rows", _i32, [_i64, _i64])
_lib.register("qwc_moe_silu_mul", ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i32, _vp])
_lib.register("qwc_moe_combine", ctypes.c_int, [_vp, _vp, _vp, _i32, _vp, _vp, _i64, _i64, _i64, _vp, _i32])
_lib.register("qwc_moe_combine_shared", ctypes.c_int, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32])
_lib.register("qwc_moe_forward", ctypes.c_int, [_vp, _vp, _WV, _WV, _i64, _i64, _vp, _i64, _i64, _i32, _vp, _i64, _i32,
                                                ctypes.c_float, _vp, _i32, _vp, _sz])
_lib.register("qwc_moe_scratch_bytes", _sz, [_i64, _i64, _i64, _i64, _i64])


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.float32:
        return F32
    raise QWGemmError(3, "tensor must be float16 or float32")


class QWMoEOperator:
    """QWMoEOperator (QWMoEOperator.swift:10-442): experts' banks plus the resident encode chain."""

    def __init__(self, hal: QWHal, bank_gu: QWWeightView, bank_dn: QWWeightView, experts: int, inter: int, top_k: int,
                 norm_topk: bool = True, routed_scale: float = 0.0):
        self.hal, self.bank_gu, self.bank_dn = hal, bank_gu, bank_dn
        self.experts, self.inter, self.top_k = experts, inter, top_k
        self.hidden = bank_gu.k
        self.norm_topk, self.routed_scale = norm_topk, routed_scale

    def scratchBytes(self, tokens: int) -> int:
        return int(_lib.load().qwc_moe_scratch_bytes(tokens, self.experts, self.top_k, self.hidden, self.inter))

    def encodeResident(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor,
                       x_is_rotated: bool = False, stream: Optional[torch.cuda.Stream] = None) -> None:
        """x f16 [T, H]; logits f32 [T, E]; out f16/f32 [T, H]; scratch uint8 of scratchBytes(T) bytes."""
        check_device_tensor(self.hal, x, "x", torch.float16, contiguous=False)
        check_device_tensor(self.hal, logits, "logits", torch.float32)
        check_device_tensor(self.hal, out, "out", (torch.float16, torch.float32))
        check_device_tensor(self.hal, scratch, "scratch", torch.uint8, numel=self.scratchBytes(x.shape[0]) if x.dim() == 2 else None)
        if x.dim() != 2 or x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) < x.shape[1]):
            raise QWGemmError(3, "x must be a float16 [T, H] tensor with contiguous rows")
        if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.shape != (x.shape[0], self.experts):
            raise QWGemmError(3, "logits must be a contiguous float32 [T, E] tensor")
        if not out.is_contiguous() or out.shape != (x.shape[0], self.hidden):
            raise QWGemmError(3, "out must be a contiguous [T, H] tensor")
        if x.shape[1] != self.hidden:
            raise QWGemmError(3, f"x has {x.shape[1]} columns, the experts take {self.hidden}")
        _check(_lib.load().qwc_moe_forward(
            self.hal.handle, _stream_ptr(stream), ctypes.byref(self.bank_gu.c), ctypes.byref(self.bank_dn.c), self.experts,
            self.inter, x.data_ptr(), x.shape[0], x.stride(0), int(x_is_rotated), logits.data_ptr(), self.top_k,
            int(self.norm_topk), float(self.routed_scale), out.data_ptr(), _dt(out), scratch.data_ptr(), scratch.numel()))


class QWGemmMoE:
    """The individual MoE doors (QWGemmMoE.swift, QWGemmMoERouter.swift)."""

    @staticmethod
    def encodeFnRouterGemm(hal: QWHal, weight: torch.Tensor, x: torch.Tensor, y: torch.Tensor, stream=None) -> None:
        """Router logits y f32 [t, e] = x [t, h] . weight [e, h]^T (QWGemmMoERouter.swift:78-125).  weight: the raw router
        plane, bf16 / f16 / f32, un-rotated; x: plain hidden states, f16 or f32."""
        dts = {torch.float16: 0, torch.float32: 1, torch.bfloat16: 2}
        if weight.dtype not in dts or x.dtype not in (torch.float16, torch.float32) or y.dtype != torch.float32:
            raise QWGemmError(3, "router GEMM takes bf16/f16/f32 weights, f16/f32 activations and f32 logits")
        if not (weight.is_contiguous() and y.is_contiguous() and x.stride(1) == 1):
            raise QWGemmError(3, "weight and y must be contiguous, x rows contiguous")
        t, h = x.shape
        e = weight.shape[0]
        if weight.shape[1] != h or tuple(y.shape) != (t, e):
            raise QWGemmError(3, "shape mismatch")
        _check(_lib.load().qwc_moe_router_gemm(hal.handle, _stream_ptr(stream), x.data_ptr(), dts[x.dtype], x.stride(0), t, h,
                                               weight.data_ptr(), dts[weight.dtype], e, y.data_ptr()))

    @staticmethod
    def encodeFnMoeRoute(hal: QWHal, logits: torch.Tensor, top_k: int, idx: torch.Tensor, wts: torch.Tensor,
                         norm_topk: bool = True, routed_scale: float = 0.0, stream=None) -> None:
        check_device_tensor(hal, logits, "logits", torch.float32)
        if logits.dim() != 2:
            raise QWGemmError(3, "logits must be [T, E]")
        t, e = logits.shape
        check_device_tensor(hal, idx, "idx", torch.int32, numel=t * top_k)
        check_device_tensor(hal, wts, "wts", torch.float32, numel=t * top_k)
        _check(_lib.load().qwc_moe_route(hal.handle, _stream_ptr(stream), logits.data_ptr(), t, e, top_k, int(norm_topk),
                                         float(routed_scale), idx.data_ptr(), wts.data_ptr()))

    @staticmethod
    def maxTiles(pairs: int, experts: int, rows_per_expert: int) -> int:
        return int(_lib.load().qwc_moe_max_tiles(pairs, experts, rows_per_expert))

    @staticmethod
    def encodeMoEGroupPairs(hal: QWHal, idx: torch.Tensor, experts: int, gu_rows: int, dn_rows: int, stream=None,
                            gu_epilogue: int = 0):
        """Returns (expert_off, sorted_pair, sorted_tok, inv_perm, tiles_gu, tiles_dn, tile_counts), all on the device.
        gu_epilogue != 0 lists paired gate/up tiles (64 gate rows + their 64 up rows) for a SwiGLU epilogue."""
        check_device_tensor(hal, idx, "idx", torch.int32)
        if idx.dim() != 2:
            raise QWGemmError(3, "idx must be [T, K]")
        t, k = idx.shape
        pairs = t * k
        dev = idx.device
        off = torch.empty(experts + 1, dtype=torch.int32, device=dev)
        sp = torch.full((pairs,), -1, dtype=torch.int32, device=dev)
        st = torch.full((pairs,), -1, dtype=torch.int32, device=dev)
        inv = torch.empty(pairs, dtype=torch.int32, device=dev)
        tg = torch.zeros((QWGemmMoE.maxTiles(pairs, experts, gu_rows), 8), dtype=torch.int32, device=dev)
        td = torch.zeros((QWGemmMoE.maxTiles(pairs, experts, dn_rows), 8), dtype=torch.int32, device=dev)
        tc = torch.zeros(4, dtype=torch.int32, device=dev)
        _check(_lib.load().qwc_moe_group_pairs(hal.handle, _stream_ptr(stream), idx.data_ptr(), pairs, experts, k, off.data_ptr(),
                                               sp.data_ptr(), st.data_ptr(), inv.data_ptr(), gu_rows, dn_rows, gu_epilogue, tg.data_ptr(),
                                               td.data_ptr(), tc.data_ptr()))
        return off, sp, st, inv, tg, td, tc

    @staticmethod
    def encodeMoECombine(hal: QWHal, dn: torch.Tensor, inv_perm: torch.Tensor, wts: torch.Tensor, out: torch.Tensor, stream=None,
                         shared: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None):
        """out[t] = sum_k wts[t, k] * dn[inv_perm[t, k]] (+ gate[t] * shared[t], the shared-expert term: shared f32 [T, H],
        gate f32 [T]) -- QWGemm.encodeMoEDownReduceCombineF32 (QWGemmMoE.swift:298-332)."""
        check_device_tensor(hal, wts, "wts", torch.float32)
        if wts.dim() != 2 or out.dim() != 2 or dn.dim() != 2:
            raise QWGemmError(3, "wts must be [T, K], dn [P, H], out [T, H]")
        t, k = wts.shape
        h = out.shape[1]
        check_device_tensor(hal, out, "out", (torch.float16, torch.float32), numel=t * h)
        check_device_tensor(hal, dn, "dn", (torch.float16, torch.float32))
        check_device_tensor(hal, inv_perm, "inv_perm", torch.int32, numel=t * k)
        if dn.shape[1] != h or out.shape[0] != t:
            raise QWGemmError(3, f"dn is {tuple(dn.shape)}, out {tuple(out.shape)}: both must have the hidden width, out one row per token")
        if (shared is None) != (gate is None):
            raise QWGemmError(3, "shared rows and their gate come together")
        if shared is not None:
            check_device_tensor(hal, shared, "shared", torch.float32, numel=t * h)
            check_device_tensor(hal, gate, "gate", torch.float32, numel=t)
        _check(_lib.load().qwc_moe_combine_shared(hal.handle, _stream_ptr(stream), dn.data_ptr(), _dt(dn), inv_perm.data_ptr(),
                                                  wts.data_ptr(), None if shared is None else shared.data_ptr(),
                                                  None if gate is None else gate.data_ptr(), t, k, h, out.data_ptr(), _dt(out)))
