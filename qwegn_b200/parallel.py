"""Tensor-parallel and expert-parallel sharding of the quantized-matmul path over torch.distributed.

The reference is single-device; what it fixes is the pack format, and the format decides how a bank can be cut:

* column parallel (split N): rows are independent and groups never span rows, so a shard is a contiguous byte
  range of the plane.  A packed gate||up bank is cut in both halves alike so that gate row r and up row I + r stay
  on one rank and the SwiGLU epilogue stays local.  No collective.
* row parallel (split K): K is cut on multiples of lcm(32, group) so neither a quant group nor a Hadamard block is
  split; a shard keeps whole blocks, bytes unchanged, re-materialised contiguously per rank.  Each rank rotates only
  its own K slice of x; the partial sums are all-reduced (NCCL over NVLink).
* expert parallel: experts [r * E / R, (r + 1) * E / R) live on rank r.  Every rank routes its own tokens, the
  (token, route) rows travel to the owning rank by all-to-all, are regrouped by expert there, run through the
  grouped expert GEMMs, and travel back for the weighted combine on the source rank.

Only the plumbing (process groups, split sizes, all_reduce / all_to_all_single) uses torch; every kernel on the
data path is in libqwcuda.so.  The pure index arithmetic is kept in functions that also run on CPU tensors so it
can be tested with the gloo backend.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .gemm import ContainerKind, QWGemm, QWGemmError, QWHal, QWWeightView, _check, _stream_ptr
from ._lib import EPI_NONE, EPI_SILU_PAIR_FWHT, WeightViewC


# ---------------------------------------------------------------------------------------------------------------
# shard arithmetic on packed planes (device-agnostic: works on CPU or CUDA uint8 tensors)

def row_range(n: int, rank: int, world: int, quantum: int = 1) -> Tuple[int, int]:
    """Rows [r0, r1) of an n-row bank owned by `rank`, cut on multiples of `quantum`."""
    if n % quantum:
        raise QWGemmError(4, f"n={n} is not a multiple of {quantum}")
    q = n // quantum
    return (q * rank // world) * quantum, (q * (rank + 1) // world) * quantum


def column_shard(plane: torch.Tensor, n: int, k: int, cont: ContainerKind, rank: int, world: int, paired: bool = False,
                 quantum: int = 1) -> Tuple[torch.Tensor, int]:
    """Column-parallel shard of a packed [n, k] plane (1-D uint8).  Returns (bytes, local n).  `paired` cuts the two
    halves of a gate||up bank alike and concatenates them."""
    rb = cont.row_bytes(k)
    rows = plane.view(n, rb)
    if not paired:
        r0, r1 = row_range(n, rank, world, quantum)
        return rows[r0:r1].reshape(-1).contiguous(), r1 - r0
    half = n // 2
    r0, r1 = row_range(half, rank, world, quantum)
    return torch.cat([rows[r0:r1], rows[half + r0:half + r1]], dim=0).reshape(-1).contiguous(), 2 * (r1 - r0)


def k_range(k: int, cont: ContainerKind, rank: int, world: int) -> Tuple[int, int]:
    """K slice [k0, k1) of `rank`, cut on multiples of lcm(32, group)."""
    q = math.lcm(32, cont.group)
    if k % q:
        raise QWGemmError(4, f"k={k} is not a multiple of {q}")
    u = k // q
    return (u * rank // world) * q, (u * (rank + 1) // world) * q


def row_shard(plane: torch.Tensor, n: int, k: int, cont: ContainerKind, rank: int, world: int) -> Tuple[torch.Tensor, int]:
    """Row-parallel (K) shard: whole blocks [k0 / group, k1 / group) of every row, contiguous.  Returns (bytes, local k)."""
    k0, k1 = k_range(k, cont, rank, world)
    bb = cont.block_bytes
    blocks = plane.view(n, k // cont.group, bb)
    return blocks[:, k0 // cont.group:k1 // cont.group].reshape(-1).contiguous(), k1 - k0


# ---------------------------------------------------------------------------------------------------------------
# tensor parallel

class ColumnParallelLinear:
    """y_local[m, n_local] = epilogue(rot(x) . W_shard^T): no collective; the output stays sharded along N."""

    def __init__(self, hal: QWHal, shard: torch.Tensor, n_local: int, k: int, cont: ContainerKind, epi: int = EPI_NONE):
        self.hal, self.view, self.epi = hal, QWWeightView(shard, n_local, k, cont), epi
        self.n_out = n_local if epi == EPI_NONE else n_local // 2

    def workspace_bytes(self, m: int, x_is_rotated: bool) -> int:
        return QWGemm.workspaceBytes(self.hal, self.view, m, self.epi, x_is_rotated)

    def forward(self, x: torch.Tensor, y: torch.Tensor, x_is_rotated: bool = False, workspace: Optional[torch.Tensor] = None):
        QWGemm.encode(self.hal, self.view, x, y, epi=self.epi, x_is_rotated=x_is_rotated, workspace=workspace)


class RowParallelLinear:
    """y[m, n] = sum over ranks of rot(x[:, k_shard]) . W[:, k_shard]^T: partial sums in f32, one all-reduce."""

    def __init__(self, hal: QWHal, shard: torch.Tensor, n: int, k_local: int, cont: ContainerKind,
                 group: Optional[dist.ProcessGroup] = None):
        self.hal, self.view, self.group = hal, QWWeightView(shard, n, k_local, cont), group

    def workspace_bytes(self, m: int, x_is_rotated: bool) -> int:
        return QWGemm.workspaceBytes(self.hal, self.view, m, EPI_NONE, x_is_rotated)

    def forward(self, x_local: torch.Tensor, y: torch.Tensor, x_is_rotated: bool = False,
                workspace: Optional[torch.Tensor] = None, reduce: bool = True):
        QWGemm.encode(self.hal, self.view, x_local, y, x_is_rotated=x_is_rotated, workspace=workspace)
        if reduce and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)


class AllReduceCtxC(ctypes.Structure):
    """qwc_allreduce_ctx (include/qwc.h)."""
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("epoch", ctypes.c_uint32), ("reserved", ctypes.c_int32),
                ("inbox", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8), ("inbox_floats", ctypes.c_int64),
                ("flag_words", ctypes.c_int64)]


_lib.register("qwc_gemm_allreduce", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(WeightViewC), ctypes.c_void_p,
                                                   ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64,
                                                   ctypes.c_int32, ctypes.POINTER(AllReduceCtxC)])


class FusedRowParallelLinear(RowParallelLinear):
    """Row-parallel matmul whose kernel also does the all-reduce (decode / verify, m <= 8): every CTA pushes its partial
    sums into all ranks' inboxes over NVLink, flags, waits for the matching CTAs of the other ranks and sums in rank
    order.  The inboxes and flags live in torch symmetric memory (two buffers, alternated per call).  Shapes the fused
    form does not take fall back to the matmul + NCCL all-reduce of the base class."""

    def __init__(self, hal: QWHal, shard: torch.Tensor, n: int, k_local: int, cont: ContainerKind,
                 group: Optional[dist.ProcessGroup] = None, max_m: int = 8):
        super().__init__(hal, shard, n, k_local, cont, group)
        import torch.distributed._symmetric_memory as symm_mem
        grp = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(grp), dist.get_rank(grp)
        dev = torch.device("cuda", hal.device.index)
        self.max_m, self.sms = max_m, hal.sm_count
        self.inbox = symm_mem.empty((2, self.world, max_m, n), dtype=torch.float32, device=dev)
        self.flags = symm_mem.empty((2, self.world, self.sms), dtype=torch.int32, device=dev)
        self.flags.zero_()
        torch.cuda.synchronize(dev)
        self.h_inbox = symm_mem.rendezvous(self.inbox, grp)
        self.h_flags = symm_mem.rendezvous(self.flags, grp)
        dist.barrier(grp)   # every rank's flags are zero before anyone's first call
        self.epoch = 0

    def forward(self, x_local: torch.Tensor, y: torch.Tensor, x_is_rotated: bool = False,
                workspace: Optional[torch.Tensor] = None, reduce: bool = True):
        x2 = x_local if x_local.dim() == 2 else x_local.view(1, -1)
        m = x2.shape[0]
        if not reduce or m > self.max_m or self.world < 2 or self.world > 8:
            return super().forward(x_local, y, x_is_rotated, workspace, reduce)
        self.epoch += 1
        buf = self.epoch & 1
        ctx = AllReduceCtxC()
        ctx.rank, ctx.world, ctx.epoch = self.rank, self.world, self.epoch
        in_bytes = self.world * self.max_m * self.view.n * 4
        fl_bytes = self.world * self.sms * 4
        for r in range(self.world):
            ctx.inbox[r] = int(self.h_inbox.buffer_ptrs[r]) + buf * in_bytes
            ctx.flags[r] = int(self.h_flags.buffer_ptrs[r]) + buf * fl_bytes
        ctx.inbox_floats = self.world * self.max_m * self.view.n
        ctx.flag_words = self.world * self.sms
        y2 = y if y.dim() == 2 else y.view(1, -1)
        rc = _lib.load().qwc_gemm_allreduce(self.hal.handle, _stream_ptr(None), ctypes.byref(self.view.c), x2.data_ptr(), m,
                                            x2.stride(0) if m > 1 else max(x2.stride(0), self.view.k), y2.data_ptr(),
                                            0 if y.dtype == torch.float16 else 1,
                                            y2.stride(0) if m > 1 else max(y2.stride(0), self.view.n), int(x_is_rotated),
                                            ctypes.byref(ctx))
        if rc == 1:   # QWC_ERR_BLOCKED: a shape the fused form does not take
            self.epoch -= 1
            return super().forward(x_local, y, x_is_rotated, workspace, reduce)
        _check(rc)


class TPMlp:
    """Gate||up column parallel with the fused SwiGLU + FWHT epilogue, down row parallel, one all-reduce."""

    def __init__(self, hal: QWHal, gu_plane: torch.Tensor, dn_plane: torch.Tensor, hidden: int, inter: int,
                 cont: ContainerKind, rank: int, world: int, group: Optional[dist.ProcessGroup] = None,
                 fused_allreduce: bool = False):
        gu, n_local = column_shard(gu_plane, 2 * inter, hidden, cont, rank, world, paired=True, quantum=math.lcm(32, cont.group))
        self.inter_local = n_local // 2
        dn, k_local = row_shard(dn_plane, hidden, inter, cont, rank, world)
        if k_local != self.inter_local:
            raise QWGemmError(4, "gate/up and down shards disagree on the local intermediate size")
        dev = torch.device("cuda", hal.device.index)
        self.gate_up = ColumnParallelLinear(hal, gu.to(dev), n_local, hidden, cont, epi=EPI_SILU_PAIR_FWHT)
        fused = fused_allreduce and world > 1 and dist.is_initialized() and dist.get_backend(group) == "nccl"
        self.down = (FusedRowParallelLinear if fused else RowParallelLinear)(hal, dn.to(dev), hidden, k_local, cont, group)

    def forward(self, x: torch.Tensor, h_local: torch.Tensor, y: torch.Tensor, ws_gu=None, ws_dn=None, x_is_rotated=False):
        """x f16 [m, hidden]; h_local f16 [m, inter_local] (rotated, scratch); y f32 [m, hidden] (all-reduced)."""
        self.gate_up.forward(x, h_local, x_is_rotated=x_is_rotated, workspace=ws_gu)
        self.down.forward(h_local, y, x_is_rotated=True, workspace=ws_dn)


# ---------------------------------------------------------------------------------------------------------------
# expert parallel: index arithmetic (device-agnostic) + the exchange

@dataclass
class EPPlan:
    """Split sizes of one dispatch (host integers) and the per-(source, local expert) row counts on the receiver."""
    send_rows: list          # rows this rank sends to each rank (in expert-sorted order)
    recv_rows: list          # rows this rank receives from each rank
    recv_counts: torch.Tensor  # int32 [world, experts_local]: rows per (source rank, local expert)


def ep_send_rows(expert_off: torch.Tensor, experts: int, world: int) -> torch.Tensor:
    """Rows per destination rank from the local expert offsets (experts are contiguous per rank)."""
    per = experts // world
    bounds = expert_off[::per][: world + 1].to(torch.int64)
    return bounds[1:] - bounds[:-1]


def ep_exchange_counts(expert_off: torch.Tensor, experts: int, world: int, group=None) -> EPPlan:
    """All-to-all of the per-expert row counts; one host read for the split sizes."""
    per = experts // world
    counts = (expert_off[1:] - expert_off[:-1]).to(torch.int32).view(world, per).contiguous()
    recv = torch.empty_like(counts)
    if world > 1:
        dist.all_to_all_single(recv, counts, group=group)
    else:
        recv.copy_(counts)
    host = torch.stack([counts.sum(dim=1), recv.sum(dim=1)]).cpu()
    return EPPlan(send_rows=[int(v) for v in host[0]], recv_rows=[int(v) for v in host[1]], recv_counts=recv)


def ep_received_expert_ids(plan: EPPlan) -> torch.Tensor:
    """Local expert id of every received row (rows arrive source-major, expert-sorted inside a source)."""
    w, per = plan.recv_counts.shape
    ids = torch.arange(per, dtype=torch.int32, device=plan.recv_counts.device).repeat(w)
    return torch.repeat_interleave(ids, plan.recv_counts.reshape(-1).to(torch.int64))


def ep_dispatch(rows: torch.Tensor, plan: EPPlan, group=None) -> torch.Tensor:
    """Send expert-sorted rows [sum(send_rows), h] to their owners; returns [sum(recv_rows), h] source-major."""
    out = torch.empty((sum(plan.recv_rows), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(out, rows[: sum(plan.send_rows)].contiguous(), plan.recv_rows, plan.send_rows, group=group)
    else:
        out.copy_(rows[: sum(plan.send_rows)])
    return out


def ep_return(rows: torch.Tensor, plan: EPPlan, group=None) -> torch.Tensor:
    """Inverse of ep_dispatch: expert outputs travel back to the rank that sent the row, same order."""
    out = torch.empty((sum(plan.send_rows), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(out, rows.contiguous(), plan.send_rows, plan.recv_rows, group=group)
    else:
        out.copy_(rows)
    return out


class EPMoE:
    """Expert-parallel sparse MoE block over the library's MoE doors.

    route -> sort by expert -> gather+rotate -> all-to-all -> regroup by local expert -> grouped gate/up ->
    SwiGLU+FWHT -> grouped down -> undo regroup -> all-to-all back -> weighted combine.
    """

    def __init__(self, hal: QWHal, gu_plane: torch.Tensor, dn_plane: torch.Tensor, experts: int, hidden: int, inter: int,
                 top_k: int, cont: ContainerKind, rank: int, world: int, norm_topk: bool = True, group=None):
        if experts % world:
            raise QWGemmError(4, f"{experts} experts do not divide over {world} ranks")
        self.hal, self.experts, self.hidden, self.inter, self.top_k = hal, experts, hidden, inter, top_k
        self.rank, self.world, self.group, self.norm_topk, self.cont = rank, world, group, norm_topk, cont
        self.per = experts // world
        dev = torch.device("cuda", hal.device.index)
        gu, _ = column_shard(gu_plane, experts * 2 * inter, hidden, cont, rank, world, quantum=2 * inter)
        dn, _ = column_shard(dn_plane, experts * hidden, inter, cont, rank, world, quantum=hidden)
        self.bank_gu = QWWeightView(gu.to(dev), self.per * 2 * inter, hidden, cont)
        self.bank_dn = QWWeightView(dn.to(dev), self.per * hidden, inter, cont)

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """x f16 [t_local, hidden] (standard basis); logits f32 [t_local, experts].  Returns f32 [t_local, hidden]."""
        import ctypes
        from . import _lib
        from .moe import QWGemmMoE
        from .gemm import _check, _stream_ptr
        lib = _lib.load()
        hal, dev = self.hal, x.device
        t, k, h, inter = x.shape[0], self.top_k, self.hidden, self.inter
        pairs = t * k
        idx = torch.empty((t, k), dtype=torch.int32, device=dev)
        wts = torch.empty((t, k), dtype=torch.float32, device=dev)
        QWGemmMoE.encodeFnMoeRoute(hal, logits, k, idx, wts, norm_topk=self.norm_topk)
        off, _, sorted_tok, inv_perm, _, _, _ = QWGemmMoE.encodeMoEGroupPairs(hal, idx, self.experts, 2 * inter, h)
        xs = torch.empty((pairs, h), dtype=torch.float16, device=dev)
        _check(lib.qwc_moe_gather(hal.handle, _stream_ptr(None), x.data_ptr(), x.stride(0), h, sorted_tok.data_ptr(),
                                  off.data_ptr(), self.experts, pairs, 0, xs.data_ptr()))
        plan = ep_exchange_counts(off, self.experts, self.world, self.group)
        recv = ep_dispatch(xs, plan, self.group)
        r = recv.shape[0]
        out_rows = torch.zeros((max(r, 1), h), dtype=torch.float16, device=dev)
        if r > 0:
            # regroup the received rows by local expert (K = 1 pair sort), run the experts, undo the regroup
            eid = ep_received_expert_ids(plan).view(r, 1).contiguous()
            fused = 2 if inter % 64 == 0 else 0   # SwiGLU + FWHT in the gate/up GEMM's epilogue
            loff, _, lsorted, linv, tg, td, tc = QWGemmMoE.encodeMoEGroupPairs(hal, eid, self.per, 2 * inter, h, gu_epilogue=fused)
            xg = torch.empty((r, h), dtype=torch.float16, device=dev)
            _check(lib.qwc_moe_gather(hal.handle, _stream_ptr(None), recv.data_ptr(), recv.stride(0), h, lsorted.data_ptr(),
                                      loff.data_ptr(), self.per, r, 1, xg.data_ptr()))
            hs = torch.empty((r, inter), dtype=torch.float16, device=dev)
            if fused:
                _check(lib.qwc_moe_grouped_gemm(hal.handle, _stream_ptr(None), ctypes.byref(self.bank_gu.c), xg.data_ptr(), r,
                                                tg.data_ptr(), tc.data_ptr(), tg.shape[0], lib.qwc_moe_tile_rows(r, self.per),
                                                hs.data_ptr(), 0, inter, fused))
            else:
                gu = torch.empty((r, 2 * inter), dtype=torch.float16, device=dev)
                _check(lib.qwc_moe_grouped_gemm(hal.handle, _stream_ptr(None), ctypes.byref(self.bank_gu.c), xg.data_ptr(), r,
                                                tg.data_ptr(), tc.data_ptr(), tg.shape[0], lib.qwc_moe_tile_rows(r, self.per),
                                                gu.data_ptr(), 0, 2 * inter, 0))
                _check(lib.qwc_moe_silu_mul(hal.handle, _stream_ptr(None), gu.data_ptr(), r, inter, 1, hs.data_ptr()))
            dn = torch.empty((r, h), dtype=torch.float16, device=dev)
            _check(lib.qwc_moe_grouped_gemm(hal.handle, _stream_ptr(None), ctypes.byref(self.bank_dn.c), hs.data_ptr(), r,
                                            td.data_ptr(), tc[1:].data_ptr(), td.shape[0], lib.qwc_moe_tile_rows(r, self.per), dn.data_ptr(), 0, h, 0))
            ones = torch.ones((r, 1), dtype=torch.float32, device=dev)
            QWGemmMoE.encodeMoECombine(hal, dn, linv, ones, out_rows[:r])
        back = ep_return(out_rows[:r], plan, self.group)
        full = torch.empty((pairs, h), dtype=torch.float16, device=dev)
        full[: back.shape[0]] = back
        out = torch.empty((t, h), dtype=torch.float32, device=dev)
        QWGemmMoE.encodeMoECombine(hal, full, inv_perm, wts, out)
        return out
