"""numpy front end of the CPU oracle (oracle/qw_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
bench's CPU-baseline leg.  The product package never imports this module.

Array conventions follow the reference's Python tooling
(Scripts/quantize/hq4.py, hq_blocks.py): blocks are uint8 [N, K/group,
block_bytes]; activations are float16 [M, K]; outputs float32.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqworacle.so")

KIND_HQ4_G32_M5 = 0
KIND_ROTATED_HQ = 1


@dataclass(frozen=True)
class Format:
    """One weight container: the reference's ContainerKind
    (Sources/Foundation/QWAlloc/QWWeightView.swift:11-31)."""
    name: str
    kind: int
    bits: int
    group: int

    @property
    def block_bytes(self) -> int:
        return 20 if self.kind == KIND_HQ4_G32_M5 else self.group * self.bits // 8 + 4

    def row_bytes(self, k: int) -> int:
        return (k // self.group) * self.block_bytes

    def plane_bytes(self, n: int, k: int) -> int:
        return n * self.row_bytes(k)


HQ4_G32 = Format("HQ4_G32", KIND_HQ4_G32_M5, 4, 32)
HQ8_G32 = Format("HQ8_G32", KIND_ROTATED_HQ, 8, 32)
HQ4_G64 = Format("HQ4_G64", KIND_ROTATED_HQ, 4, 64)
FORMATS = {f.name: f for f in (HQ4_G32, HQ8_G32, HQ4_G64)}


def build(force: bool = False) -> str:
    """Compile the C oracle in place (gcc + OpenMP) if it is missing or stale."""
    src = os.path.join(_HERE, "qw_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libqworacle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.qwo_fwht32_f32.argtypes = [vp, i64]
        L.qwo_fwht32_f16.argtypes = [vp, i64]
        L.qwo_f32_to_f16.argtypes = [vp, vp, i64]
        L.qwo_quant_hq4_g32_m5.argtypes = [vp, i64, i64, vp]
        L.qwo_quant_hq_blocks.argtypes = [vp, i64, i64, i32, i32, vp]
        L.qwo_dequant.argtypes = [vp, i64, i64, i32, i32, i32, i32, i32, vp]
        L.qwo_matmul.argtypes = [vp, i64, i64, i32, i32, i32, vp, i64, i64, i32, vp, i64]
        L.qwo_swiglu_f16.argtypes = [vp, i64, i64, i32, vp]
        L.qwo_moe_route.argtypes = [vp, i64, i64, i64, i32, ctypes.c_float, vp, vp]
        L.qwo_moe_group_pairs.argtypes = [vp, i64, i64, i64, vp, vp, vp, vp]
        L.qwo_moe_tile_plan.argtypes = [vp, i64, vp, vp]
        L.qwo_moe_tile_plan.restype = ctypes.c_int32
        L.qwo_moe_forward.argtypes = [vp, vp, i32, i32, i32, i64, i64, i64, vp, i64, i64, vp, vp, vp]
        L.qwo_moe_forward_f32.argtypes = [vp, i64, i64, i64, i64, i64, i32, vp, vp, vp, i64, vp, vp, vp, vp, vp]
        L.qwo_num_threads.restype = ctypes.c_int
        L.qwo_set_num_threads.restype = ctypes.c_int
        L.qwo_set_num_threads.argtypes = [ctypes.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().qwo_num_threads())


def set_num_threads(n: int) -> int:
    """Use n OpenMP threads from now on (launchers may export OMP_NUM_THREADS=1); returns the number in effect."""
    return int(lib().qwo_set_num_threads(int(n)))


def fwht32(x: np.ndarray) -> np.ndarray:
    """f32 orthonormal Walsh-Hadamard over aligned 32-blocks of the last axis."""
    y = _c(x, np.float32).copy()
    assert y.shape[-1] % 32 == 0
    lib().qwo_fwht32_f32(_p(y), y.size)
    return y


def fwht32_f16(x: np.ndarray) -> np.ndarray:
    """Activation rotation: f16 in, f32 butterflies, one rounding to f16."""
    y = _c(x, np.float16).copy()
    assert y.shape[-1] % 32 == 0
    lib().qwo_fwht32_f16(_p(y), y.size)
    return y


def quantize(w: np.ndarray, fmt: Format) -> np.ndarray:
    w = _c(w, np.float32)
    n, k = w.shape
    if k % fmt.group:
        raise ValueError(f"K={k} is not a multiple of group {fmt.group}")
    blocks = np.empty((n, k // fmt.group, fmt.block_bytes), dtype=np.uint8)
    if fmt.kind == KIND_HQ4_G32_M5:
        rc = lib().qwo_quant_hq4_g32_m5(_p(w), n, k, _p(blocks))
    else:
        rc = lib().qwo_quant_hq_blocks(_p(w), n, k, fmt.bits, fmt.group, _p(blocks))
    if rc:
        raise ValueError(f"quantize refused the input (code {rc})")
    return blocks


def dequant(blocks: np.ndarray, fmt: Format, f16_round: bool = False, standard: bool = False) -> np.ndarray:
    b = _c(blocks, np.uint8)
    n, nb, bb = b.shape
    assert bb == fmt.block_bytes
    out = np.empty((n, nb * fmt.group), dtype=np.float32)
    rc = lib().qwo_dequant(_p(b), n, nb * fmt.group, fmt.kind, fmt.bits, fmt.group,
                           int(f16_round), int(standard), _p(out))
    if rc:
        raise ValueError(f"dequant refused the input (code {rc})")
    return out


def matmul(blocks: np.ndarray, fmt: Format, x: np.ndarray, x_is_rotated: bool = False) -> np.ndarray:
    """y[M,N] = f16(fwht32(x)) . dequant_rot(blocks, f16_round=True)^T."""
    b = _c(blocks, np.uint8)
    n, nb, _ = b.shape
    k = nb * fmt.group
    x = _c(x, np.float16).reshape(-1, k)
    m = x.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    rc = lib().qwo_matmul(_p(b), n, k, fmt.kind, fmt.bits, fmt.group, _p(x), m, k,
                          int(x_is_rotated), _p(y), n)
    if rc:
        raise ValueError(f"matmul refused the input (code {rc})")
    return y


def matmul_f32(blocks: np.ndarray, fmt: Format, x: np.ndarray, epi: int = 0, scale: float = 1.0,
               x_is_rotated: bool = True) -> np.ndarray:
    """The f32-activation matmul (Sources/Operators/QWGEMM/QWGemmF32.swift:143-199, 309-350; kernel bodies
    Sources/QWMetal/include/qw_gemm_f32_common.metalh:59-225 with the f32 decode of include/qw_dequant_f32.metalh:9-56):
    y = epi(x_rot . W_rot^T), x f32 (rotated by encodeH32F32, QWGemmF32.swift:46-54, when it is not yet), weights
    decoded in f32, epi 0 none / 1 silu(y/scale) / 2 sigmoid(y) / 3 silu(y/scale) then FWHT-32 along n
    (qw_gemm_f32_common.metalh:15-20, 131-133)."""
    w = dequant(blocks, fmt, f16_round=False, standard=False).astype(np.float64)
    x = _c(x, np.float32).reshape(-1, w.shape[1])
    xr = x if x_is_rotated else fwht32(x)
    y = (xr.astype(np.float64) @ w.T).astype(np.float32)
    if epi in (1, 3):
        z = (y / np.float32(scale)).astype(np.float32)
        y = (z / (np.float32(1.0) + np.exp(-z, dtype=np.float32))).astype(np.float32)
    elif epi == 2:
        y = (np.float32(1.0) / (np.float32(1.0) + np.exp(-y, dtype=np.float32))).astype(np.float32)
    if epi == 3:
        y = fwht32(y)
    return y


def swiglu_f16(gu: np.ndarray, rotate: bool = False) -> np.ndarray:
    gu = _c(gu, np.float32)
    m, two_i = gu.shape
    h = np.empty((m, two_i // 2), dtype=np.float16)
    lib().qwo_swiglu_f16(_p(gu), m, two_i // 2, int(rotate), _p(h))
    return h


def rmsnorm_fwht(x: np.ndarray, gamma: np.ndarray, eps: float = 1e-6, residual: np.ndarray | None = None, rotate: bool = True):
    """RMSNorm of the reference's norm family (qwg_rmsnorm / qwg_rmsnorm_residual,
    Sources/QWMetal/mlp_norm_rope/qwnorm.metal:19-79, 200-259): s = x or f16(x + residual); y = f16(fwht32(s * rsqrt(mean(s^2)
    + eps) * (1 + gamma))) with f32 products and butterflies; the sum of squares is taken in f64 here (the device's f32
    sum differs from it in the last bits only).  Returns (y f16, new residual f16 or None)."""
    s = np.asarray(x, dtype=np.float16).astype(np.float32)
    new_res = None
    if residual is not None:
        s = (s + np.asarray(residual, dtype=np.float16).astype(np.float32)).astype(np.float16)
        new_res = s.copy()
        s = s.astype(np.float32)
    rstd = (1.0 / np.sqrt((s.astype(np.float64) ** 2).mean(axis=-1, keepdims=True) + eps)).astype(np.float32)
    f = (s * rstd) * (np.asarray(gamma, dtype=np.float16).astype(np.float32) + np.float32(1.0))
    if rotate:
        f = fwht32(f.astype(np.float32))
    return f.astype(np.float16), new_res


def head_argmax(logits: np.ndarray) -> np.ndarray:
    """Greedy token per row in the reference's key order (qw_sortable_f32_u32, Sources/QWMetal/include/qw_fastmath_safe.metalh:
    21-25; qwg_gemv_am_fold4, include/qw_gemm_f32_common.metalh:31-47): key = (sortable(value), ~column): NaN lowest,
    +0 above -0, ties to the lower column."""
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    lg = lg.reshape(-1, lg.shape[-1])
    u = lg.view(np.uint32)
    s = np.where((u & np.uint32(0x80000000)) != 0, ~u, u ^ np.uint32(0x80000000))
    s = np.where((u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000), np.uint32(0), s)
    cols = np.arange(lg.shape[1], dtype=np.uint64)
    key = (s.astype(np.uint64) << np.uint64(32)) | (np.uint64(0xFFFFFFFF) - cols)
    return key.argmax(axis=1).astype(np.int32)


def router_gemm(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """Router logits [t, e] = x [t, h] . w [e, h]^T (qwg_router_gemm, Sources/QWMetal/subsystems/qwrouter.metal:457-520):
    plain dot products of the un-rotated hidden states with the raw router plane; accumulated in f64 here, so the device's
    f32 accumulation is compared against the exact value.  bf16 planes are passed in already widened to f32."""
    return (np.asarray(x, dtype=np.float64) @ np.asarray(w, dtype=np.float64).T).astype(np.float32)


def moe_route(logits: np.ndarray, topk: int, norm_topk: bool = True, routed_scale: float = 0.0):
    lg = _c(logits, np.float32)
    t, e = lg.shape
    idx = np.empty((t, topk), dtype=np.int32)
    wts = np.empty((t, topk), dtype=np.float32)
    lib().qwo_moe_route(_p(lg), t, e, topk, int(norm_topk), float(routed_scale), _p(idx), _p(wts))
    return idx, wts


def moe_group_pairs(idx: np.ndarray, experts: int):
    idx = _c(idx, np.int32)
    t, topk = idx.shape
    pairs = t * topk
    off = np.empty(experts + 1, dtype=np.int32)
    sp = np.full(pairs, -1, dtype=np.int32)
    st = np.full(pairs, -1, dtype=np.int32)
    inv = np.empty(pairs, dtype=np.int32)
    lib().qwo_moe_group_pairs(_p(idx), pairs, experts, topk, _p(off), _p(sp), _p(st), _p(inv))
    return off, sp, st, inv


def moe_tile_plan(expert_off: np.ndarray):
    off = _c(expert_off, np.int32)
    e = off.size - 1
    cap = int(off[-1]) // 16 + e + 1
    te = np.empty(cap, dtype=np.int32)
    tr = np.empty(cap, dtype=np.int32)
    n = lib().qwo_moe_tile_plan(_p(off), e, _p(te), _p(tr))
    return te[:n].copy(), tr[:n].copy()


def moe_forward(bank_gu: np.ndarray, bank_dn: np.ndarray, fmt: Format, experts: int, hidden: int,
                inter: int, x: np.ndarray, idx: np.ndarray, wts: np.ndarray) -> np.ndarray:
    x = _c(x, np.float16)
    t = x.shape[0]
    idx = _c(idx, np.int32)
    wts = _c(wts, np.float32)
    bg = _c(bank_gu, np.uint8)
    bd = _c(bank_dn, np.uint8)
    assert bg.size == experts * 2 * inter * fmt.row_bytes(hidden)
    assert bd.size == experts * hidden * fmt.row_bytes(inter)
    out = np.empty((t, hidden), dtype=np.float32)
    rc = lib().qwo_moe_forward(_p(bg), _p(bd), fmt.kind, fmt.bits, fmt.group, experts, hidden, inter,
                               _p(x), t, idx.shape[1], _p(idx), _p(wts), _p(out))
    if rc:
        raise ValueError("moe_forward refused the input")
    return out


def moe_forward_f32(x, gate_w, gate_up, down, topk, norm_topk, sh_gate=None, sh_up=None, sh_down=None,
                    sh_scalar=None) -> np.ndarray:
    x = _c(x, np.float32)
    t, h = x.shape
    gate_w = _c(gate_w, np.float32)
    e = gate_w.shape[0]
    gate_up = _c(gate_up, np.float32)
    down = _c(down, np.float32)
    i_dim = gate_up.shape[1] // 2
    out = np.empty((t, h), dtype=np.float32)
    if sh_gate is not None:
        sh_gate, sh_up, sh_down, sh_scalar = (_c(a, np.float32) for a in (sh_gate, sh_up, sh_down, sh_scalar))
        si = sh_gate.shape[0]
        args = (_p(sh_gate), _p(sh_up), _p(sh_down), _p(sh_scalar))
    else:
        si = 0
        args = (None, None, None, None)
    lib().qwo_moe_forward_f32(_p(x), t, h, e, topk, i_dim, int(norm_topk), _p(gate_w), _p(gate_up),
                              _p(down), si, *args, _p(out))
    return out
