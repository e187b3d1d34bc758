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


def section_column_shard(plane: torch.Tensor, sections, k: int, cont: ContainerKind, rank: int, world: int,
                         quantum: int = 1) -> Tuple[torch.Tensor, list]:
    """Column-parallel shard of a plane whose rows come in sections that are each cut over the ranks (a fused QKV
    plane: query rows, key rows, value rows -- every rank keeps its heads of each).  Returns (bytes, local rows per
    section); the local plane is the concatenation of the sections' shards."""
    rb = cont.row_bytes(k)
    rows = plane.view(sum(sections), rb)
    parts, local, base = [], [], 0
    for n_sec in sections:
        r0, r1 = row_range(n_sec, rank, world, quantum)
        parts.append(rows[base + r0:base + r1])
        local.append(r1 - r0)
        base += n_sec
    return torch.cat(parts, dim=0).reshape(-1).contiguous(), local


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
    """y[m, n] = sum over ranks of rot(x[:, k_shard]) . W[:, k_shard]^T: partial sums in f32, one all-reduce.  `world`
    (default: the size of `group`) says over how many ranks the bank was cut; 1 means no collective at all."""

    def __init__(self, hal: QWHal, shard: torch.Tensor, n: int, k_local: int, cont: ContainerKind,
                 group: Optional[dist.ProcessGroup] = None, world: Optional[int] = None):
        self.hal, self.view, self.group = hal, QWWeightView(shard, n, k_local, cont), group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)

    def workspace_bytes(self, m: int, x_is_rotated: bool) -> int:
        return QWGemm.workspaceBytes(self.hal, self.view, m, EPI_NONE, x_is_rotated)

    def forward(self, x_local: torch.Tensor, y: torch.Tensor, x_is_rotated: bool = False,
                workspace: Optional[torch.Tensor] = None, reduce: bool = True):
        QWGemm.encode(self.hal, self.view, x_local, y, x_is_rotated=x_is_rotated, workspace=workspace)
        if reduce and self.world > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)


_lib.register("qwc_peer_alloc", ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p])
_lib.register("qwc_peer_open", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)])
_lib.register("qwc_peer_close", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p])
_lib.register("qwc_peer_free", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p])


class PeerBuffer:
    """One zero-initialised device buffer per rank, each mapped into every other rank's address space (qwc_peer_alloc /
    qwc_peer_open): ptrs[r] is rank r's buffer as seen from this rank.  The 64-byte handles travel by an all-gather of
    the process group.  With world == 1 (or no process group) the buffer is plain local memory."""

    def __init__(self, hal: QWHal, nbytes: int, group: Optional[dist.ProcessGroup] = None):
        lib = _lib.load()
        self.hal, self.nbytes = hal, int(nbytes)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        local, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        _check(lib.qwc_peer_alloc(hal.handle, self.nbytes, ctypes.byref(local), handle))
        self.local = int(local.value)
        self.ptrs = [0] * self.world
        self.ptrs[self.rank] = self.local
        self._opened = []
        if self.world > 1:
            mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=hal.device)
            every = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(every, mine, group=group)
            for r in range(self.world):
                if r == self.rank:
                    continue
                h = (ctypes.c_ubyte * 64)(*every[r].cpu().tolist())
                p = ctypes.c_void_p()
                _check(lib.qwc_peer_open(hal.handle, h, ctypes.byref(p)))
                self.ptrs[r] = int(p.value)
                self._opened.append(int(p.value))
            dist.barrier(group)   # every rank has mapped every buffer (and they are all zero) before anyone's first call

    def close(self):
        lib = _lib.load()
        if getattr(self, "hal", None) is None or getattr(self.hal, "_h", None) is None:
            return
        for p in self._opened:
            lib.qwc_peer_close(self.hal.handle, ctypes.c_void_p(p))
        self._opened = []
        if self.local:
            lib.qwc_peer_free(self.hal.handle, ctypes.c_void_p(self.local))
            self.local = 0


class AllReduceCtxC(ctypes.Structure):
    """qwc_allreduce_ctx (include/qwc.h)."""
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("epoch", ctypes.c_uint32), ("reserved", ctypes.c_int32),
                ("inbox", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8), ("inbox_floats", ctypes.c_int64),
                ("flag_words", ctypes.c_int64), ("epoch_state", ctypes.c_void_p)]


_lib.register("qwc_gemm_allreduce", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(WeightViewC), ctypes.c_void_p,
                                                   ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64,
                                                   ctypes.c_int32, ctypes.POINTER(AllReduceCtxC)])


class FusedRowParallelLinear(RowParallelLinear):
    """Row-parallel matmul whose kernel also does the all-reduce (decode / verify, m <= 8): every CTA pushes its partial
    sums into all ranks' inboxes over NVLink as (value, call number) pairs, waits until the slots of its own rows carry the
    call's number and sums them in rank order.  The inboxes are peer-mapped buffers (PeerBuffer; two, used in turn); the call
    number is counted on the device, so the calls can be captured in a CUDA graph and replayed.  Shapes the fused form does not take fall
    back to the matmul + NCCL all-reduce of the base class."""

    def __init__(self, hal: QWHal, shard: torch.Tensor, n: int, k_local: int, cont: ContainerKind,
                 group: Optional[dist.ProcessGroup] = None, max_m: int = 8):
        super().__init__(hal, shard, n, k_local, cont, group)
        grp = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(grp)
        dev = torch.device("cuda", hal.device.index)
        self.max_m, self.sms = max_m, hal.sm_count
        in_floats = 2 * self.world * max_m * n                    # a slot is (f32 value, u32 call number)
        self.inbox = PeerBuffer(hal, 2 * in_floats * 4, grp)     # two buffers, used in turn
        self.state = torch.zeros(2, dtype=torch.int32, device=dev)   # device-side call counter + ticket
        torch.cuda.synchronize(dev)
        self.ctx = AllReduceCtxC()
        self.ctx.rank, self.ctx.world, self.ctx.epoch = self.rank, self.world, 0
        for r in range(self.world):
            self.ctx.inbox[r] = self.inbox.ptrs[r]
        self.ctx.inbox_floats, self.ctx.flag_words = in_floats, 0
        self.ctx.epoch_state = self.state.data_ptr()

    def forward(self, x_local: torch.Tensor, y: torch.Tensor, x_is_rotated: bool = False,
                workspace: Optional[torch.Tensor] = None, reduce: bool = True):
        x2 = x_local if x_local.dim() == 2 else x_local.view(1, -1)
        m = x2.shape[0]
        if not reduce or m > self.max_m or self.world < 2 or self.world > 8:
            return super().forward(x_local, y, x_is_rotated, workspace, reduce)
        y2 = y if y.dim() == 2 else y.view(1, -1)
        rc = _lib.load().qwc_gemm_allreduce(self.hal.handle, _stream_ptr(None), ctypes.byref(self.view.c), x2.data_ptr(), m,
                                            x2.stride(0) if m > 1 else max(x2.stride(0), self.view.k), y2.data_ptr(),
                                            0 if y.dtype == torch.float16 else 1,
                                            y2.stride(0) if m > 1 else max(y2.stride(0), self.view.n), int(x_is_rotated),
                                            ctypes.byref(self.ctx))
        if rc == 1:   # QWC_ERR_BLOCKED: a shape the fused form does not take (nothing was launched)
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
        self.down = (FusedRowParallelLinear(hal, dn.to(dev), hidden, k_local, cont, group) if fused
                     else RowParallelLinear(hal, dn.to(dev), hidden, k_local, cont, group, world=world))

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


# ---------------------------------------------------------------------------------------------------------------
# tensor-parallel layer stack (the projections of a dense transformer layer; attention itself is another operator)

class TPLayer:
    """The four projections of one dense layer under tensor parallelism, in the order the reference's engine runs them
    (Sources/Runtime/QWEngine/Module/QWDenseLayerKernels.swift:96-177 decode, :200-297 prefill):
    QKV column parallel (every rank keeps its query / key / value heads), O row parallel + all-reduce, gate||up column
    parallel with SwiGLU + FWHT fused, down row parallel + all-reduce; RMSNorm with fused residual and rotation between
    them.  The attention operator between QKV and O is not part of this path: O takes the rank's query columns of the QKV
    output as its input, which has the shape and the sharding of an attention output."""

    def __init__(self, hal: QWHal, planes: dict, hidden: int, inter: int, q_heads: int, kv_heads: int, head_dim: int,
                 attn_cont: ContainerKind, mlp_cont: ContainerKind, rank: int, world: int, group=None, fused_allreduce=True):
        dev = torch.device("cuda", hal.device.index)
        self.hal, self.hidden, self.rank, self.world, self.group = hal, hidden, rank, world, group
        qn, kvn = q_heads * head_dim, kv_heads * head_dim
        qkv, loc = section_column_shard(planes["qkv"], [qn, kvn, kvn], hidden, attn_cont, rank, world, quantum=head_dim)
        self.q_local, self.qkv_local = loc[0], sum(loc)
        self.qkv = ColumnParallelLinear(hal, qkv.to(dev), self.qkv_local, hidden, attn_cont)
        o, ok_local = row_shard(planes["o"], hidden, qn, attn_cont, rank, world)
        if ok_local != self.q_local:
            raise QWGemmError(4, "the query shard and the K shard of O disagree")
        gu, n_local = column_shard(planes["gate_up"], 2 * inter, hidden, mlp_cont, rank, world, paired=True,
                                   quantum=math.lcm(32, mlp_cont.group))
        self.inter_local = n_local // 2
        dn, dk_local = row_shard(planes["down"], hidden, inter, mlp_cont, rank, world)
        if dk_local != self.inter_local:
            raise QWGemmError(4, "gate/up and down shards disagree on the local intermediate size")
        self.gate_up = ColumnParallelLinear(hal, gu.to(dev), n_local, hidden, mlp_cont, epi=EPI_SILU_PAIR_FWHT)
        fused = fused_allreduce and world > 1 and dist.is_initialized() and dist.get_backend(group) == "nccl"
        if fused:
            self.o = FusedRowParallelLinear(hal, o.to(dev), hidden, ok_local, attn_cont, group)
            self.down = FusedRowParallelLinear(hal, dn.to(dev), hidden, dk_local, mlp_cont, group)
        else:
            self.o = RowParallelLinear(hal, o.to(dev), hidden, ok_local, attn_cont, group, world=world)
            self.down = RowParallelLinear(hal, dn.to(dev), hidden, dk_local, mlp_cont, group, world=world)
        self.gamma1 = torch.zeros(hidden, dtype=torch.float16, device=dev)
        self.gamma2 = torch.zeros(hidden, dtype=torch.float16, device=dev)


class TPLayerStack:
    """A stack of TPLayer.  forward(): xn = rotated, normed input of the first layer; res = residual stream; both f16
    [m, hidden], updated in place (res ends as the stack's output).  The caller's buffers come from buffers(m).
    Decode / verify (m <= 8): every row-parallel projection is the fused matmul + all-reduce kernel.  Prefill: the
    tokens are cut into chunks that run through a layer one after the other, so that the NCCL all-reduce of one chunk
    (on a second stream) overlaps the matmuls of the next."""

    def __init__(self, layers, hal: QWHal, group=None):
        self.layers, self.hal, self.group = layers, hal, group
        self.world = layers[0].world
        self.comm = torch.cuda.Stream(device=hal.device) if self.world > 1 else None

    def buffers(self, m: int) -> dict:
        l0, dev = self.layers[0], self.hal.device
        f16 = dict(dtype=torch.float16, device=dev)
        ws_o = max(l.o.workspace_bytes(m, False) for l in self.layers)
        return {"qkv": torch.empty((m, l0.qkv_local), **f16), "y": torch.empty((m, l0.hidden), **f16),
                "h": torch.empty((m, l0.inter_local), **f16),
                "ws": torch.empty(max(ws_o, 16), dtype=torch.uint8, device=dev)}

    def forward(self, xn: torch.Tensor, res: torch.Tensor, buf: dict, chunk: int = 0) -> None:
        m = xn.shape[0]
        if m <= 8 or self.world == 1 or chunk <= 0 or chunk >= m:
            for l in self.layers:
                self._layer(l, xn, res, buf["qkv"], buf["y"], buf["h"], buf["ws"], None)
            return
        # prefill under tensor parallelism: chunks of tokens, all-reduces on the second stream
        main = torch.cuda.current_stream()
        spans = [(c0, min(c0 + chunk, m)) for c0 in range(0, m, chunk)]
        for l in self.layers:
            for half in (0, 1):
                done = []
                for c0, c1 in spans:
                    sl = slice(c0, c1)
                    if half == 0:
                        l.qkv.forward(xn[sl], buf["qkv"][sl], x_is_rotated=True)
                        l.o.forward(buf["qkv"][sl, :l.q_local], buf["y"][sl], x_is_rotated=False, workspace=buf["ws"], reduce=False)
                    else:
                        l.gate_up.forward(xn[sl], buf["h"][sl], x_is_rotated=True)
                        l.down.forward(buf["h"][sl], buf["y"][sl], x_is_rotated=True, reduce=False)
                    ev = torch.cuda.Event()
                    ev.record(main)
                    self.comm.wait_event(ev)
                    with torch.cuda.stream(self.comm):
                        dist.all_reduce(buf["y"][sl], op=dist.ReduceOp.SUM, group=self.group)
                        ev2 = torch.cuda.Event()
                        ev2.record(self.comm)
                    done.append(ev2)
                for (c0, c1), ev2 in zip(spans, done):
                    main.wait_event(ev2)
                    sl = slice(c0, c1)
                    QWGemm.encodeRMSNorm(self.hal, buf["y"][sl], l.gamma1 if half == 0 else l.gamma2, xn[sl], residual=res[sl])

    def _layer(self, l, xn, res, qkv, y, h, ws, _):
        l.qkv.forward(xn, qkv, x_is_rotated=True)
        l.o.forward(qkv[:, :l.q_local], y, x_is_rotated=False, workspace=ws)
        QWGemm.encodeRMSNorm(self.hal, y, l.gamma1, xn, residual=res)
        l.gate_up.forward(xn, h, x_is_rotated=True)
        l.down.forward(h, y, x_is_rotated=True)
        QWGemm.encodeRMSNorm(self.hal, y, l.gamma2, xn, residual=res)


# ---------------------------------------------------------------------------------------------------------------
# expert parallel with the exchange inside the library (peer stores + flags, no NCCL, no host synchronisation)

class EpCtxC(ctypes.Structure):
    """qwc_ep_ctx (include/qwc.h)."""
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("epoch", ctypes.c_uint32), ("wait_us", ctypes.c_int32),
                ("capacity_rows", ctypes.c_int64), ("recv", ctypes.c_void_p * 8), ("counts", ctypes.c_void_p * 8),
                ("ret", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8), ("epoch_state", ctypes.c_void_p)]


_EP = ctypes.POINTER(EpCtxC)
_vp, _i32, _i64, _sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
_lib.register("qwc_ep_recv_bytes", _sz, [_i32, _i64, _i64])
_lib.register("qwc_ep_ret_bytes", _sz, [_i64, _i64])
_lib.register("qwc_ep_counts_bytes", _sz, [_i32, _i64])
_lib.register("qwc_ep_flags_bytes", _sz, [_i32])
_lib.register("qwc_ep_scratch_bytes", _sz, [_EP, _i64, _i64, _i64, _i64, _i64])
_lib.register("qwc_ep_dispatch", ctypes.c_int, [_vp, _vp, _EP, _i64, _vp, _i64, _i64, _i64, _i32, _vp, _i64, _i32, ctypes.c_float,
                                                _vp, _sz, _i64])
_lib.register("qwc_ep_experts", ctypes.c_int, [_vp, _vp, _EP, ctypes.POINTER(WeightViewC), ctypes.POINTER(WeightViewC), _i64, _i64, _i64,
                                               _i64, _vp, _sz])
_lib.register("qwc_ep_combine", ctypes.c_int, [_vp, _vp, _EP, _i64, _i64, _i64, _i64, _i64, _vp, _i32, _vp, _sz])
_lib.register("qwc_ep_moe", ctypes.c_int, [_vp, _vp, _EP, ctypes.POINTER(WeightViewC), ctypes.POINTER(WeightViewC), _i64, _i64, _vp, _i64,
                                           _i64, _i32, _vp, _i64, _i32, ctypes.c_float, _vp, _i32, _vp, _sz])


class EPMoEFused:
    """Expert-parallel sparse MoE block through qwc_ep_moe: route and sort on the source rank, rows stored straight into
    the owning rank's receive buffer, grouped expert GEMMs there, results stored straight back, weighted combine on the
    source rank.  The peer buffers are allocated once (capacity = the most (token, route) pairs any rank brings to one
    call); forward() allocates nothing and never synchronises with the host.  The call number is counted on the device,
    so forward() can be captured in a CUDA graph."""

    def __init__(self, hal: QWHal, gu_plane: torch.Tensor, dn_plane: torch.Tensor, experts: int, hidden: int, inter: int,
                 top_k: int, cont: ContainerKind, rank: int, world: int, max_tokens: int, norm_topk: bool = True, group=None):
        if experts % world:
            raise QWGemmError(4, f"{experts} experts do not divide over {world} ranks")
        lib = _lib.load()
        self.hal, self.experts, self.hidden, self.inter, self.top_k = hal, experts, hidden, inter, top_k
        self.rank, self.world, self.norm_topk, self.max_tokens = rank, world, norm_topk, max_tokens
        dev = torch.device("cuda", hal.device.index)
        per = experts // world
        gu, _ = column_shard(gu_plane, experts * 2 * inter, hidden, cont, rank, world, quantum=2 * inter)
        dn, _ = column_shard(dn_plane, experts * hidden, inter, cont, rank, world, quantum=hidden)
        self.bank_gu = QWWeightView(gu.to(dev), per * 2 * inter, hidden, cont)
        self.bank_dn = QWWeightView(dn.to(dev), per * hidden, inter, cont)
        cap = max_tokens * top_k
        self.recv = PeerBuffer(hal, lib.qwc_ep_recv_bytes(world, cap, hidden), group)
        self.counts = PeerBuffer(hal, lib.qwc_ep_counts_bytes(world, experts), group)
        self.ret = PeerBuffer(hal, lib.qwc_ep_ret_bytes(cap, hidden), group)
        self.flags = PeerBuffer(hal, lib.qwc_ep_flags_bytes(world), group)
        self.state = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ctx = EpCtxC()
        self.ctx.rank, self.ctx.world, self.ctx.epoch, self.ctx.wait_us, self.ctx.capacity_rows = rank, world, 0, 0, cap
        for r in range(world):
            self.ctx.recv[r], self.ctx.counts[r] = self.recv.ptrs[r], self.counts.ptrs[r]
            self.ctx.ret[r], self.ctx.flags[r] = self.ret.ptrs[r], self.flags.ptrs[r]
        self.ctx.epoch_state = self.state.data_ptr()
        nbytes = lib.qwc_ep_scratch_bytes(ctypes.byref(self.ctx), max_tokens, experts, top_k, hidden, inter)
        self.scratch = torch.empty(nbytes + 256, dtype=torch.uint8, device=dev)
        self._sc_ptr = (self.scratch.data_ptr() + 255) // 256 * 256
        self._sc_bytes = nbytes
        torch.cuda.synchronize(dev)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor, x_is_rotated: bool = False) -> None:
        """x f16 [t, hidden]; logits f32 [t, experts]; out f16/f32 [t, hidden] (t <= max_tokens, may be 0)."""
        from .gemm import check_device_tensor
        t = x.shape[0]
        if t > self.max_tokens:
            raise QWGemmError(3, f"{t} tokens exceed the {self.max_tokens} this block was sized for")
        if t > 0:
            check_device_tensor(self.hal, x, "x", torch.float16, contiguous=False)
            check_device_tensor(self.hal, logits, "logits", torch.float32, numel=t * self.experts)
            check_device_tensor(self.hal, out, "out", (torch.float16, torch.float32), numel=t * self.hidden)
            if x.dim() != 2 or x.shape[1] != self.hidden or x.stride(1) != 1:
                raise QWGemmError(3, "x must be [t, hidden] with contiguous rows")
        _check(_lib.load().qwc_ep_moe(
            self.hal.handle, _stream_ptr(None), ctypes.byref(self.ctx), ctypes.byref(self.bank_gu.c), ctypes.byref(self.bank_dn.c),
            self.experts, self.inter, x.data_ptr() if t else None, t, x.stride(0) if t else self.hidden, int(x_is_rotated),
            logits.data_ptr() if t else None, self.top_k, int(self.norm_topk), 0.0, out.data_ptr() if t else None,
            0 if out.dtype == torch.float16 else 1, ctypes.c_void_p(self._sc_ptr), self._sc_bytes))
