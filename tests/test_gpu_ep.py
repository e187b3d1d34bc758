"""The expert-parallel exchange (qwc_ep_dispatch / qwc_ep_experts / qwc_ep_combine) on ONE GPU: the ranks of a group are
emulated by running each phase rank after rank on the same device, every rank with its own buffers, so every wait finds
its flags already raised and no kernel ever waits for a kernel that is not running.  Checked against the oracle's
single-device MoE block on the same tokens."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import assert_matmul_close

pytestmark = pytest.mark.gpu


def _emulated_group(q, hal, oracle, name, world, e, k, hidden, inter, t_per_rank, seed, calls=2, host_epoch=False):
    from qwegn_b200 import _lib, parallel as par
    from qwegn_b200.gemm import _stream_ptr
    lib = _lib.load()
    fmt, cont = oracle.FORMATS[name], q.CONTAINERS[name]
    rng = np.random.default_rng(seed)
    gu = oracle.quantize(rng.normal(0.0, 0.05, (e * 2 * inter, hidden)).astype(np.float32), fmt)
    dn = oracle.quantize(rng.normal(0.0, 0.05, (e * hidden, inter)).astype(np.float32), fmt)
    per = e // world
    cap = max(t_per_rank) * k
    dev = "cuda"
    bufs = []
    for r in range(world):
        b = {"recv": torch.zeros(lib.qwc_ep_recv_bytes(world, cap, hidden), dtype=torch.uint8, device=dev),
             "counts": torch.zeros(lib.qwc_ep_counts_bytes(world, e), dtype=torch.uint8, device=dev),
             "ret": torch.zeros(lib.qwc_ep_ret_bytes(cap, hidden), dtype=torch.uint8, device=dev),
             "flags": torch.zeros(lib.qwc_ep_flags_bytes(world), dtype=torch.uint8, device=dev),
             "state": torch.zeros(1, dtype=torch.int32, device=dev)}
        bufs.append(b)
    ranks = []
    for r in range(world):
        ctx = par.EpCtxC()
        ctx.rank, ctx.world, ctx.epoch, ctx.wait_us, ctx.capacity_rows = r, world, 0, 50000, cap
        for p in range(world):
            ctx.recv[p], ctx.counts[p] = bufs[p]["recv"].data_ptr(), bufs[p]["counts"].data_ptr()
            ctx.ret[p], ctx.flags[p] = bufs[p]["ret"].data_ptr(), bufs[p]["flags"].data_ptr()
        ctx.epoch_state = None if host_epoch else bufs[r]["state"].data_ptr()
        gu_l = np.ascontiguousarray(gu[r * per * 2 * inter:(r + 1) * per * 2 * inter])
        dn_l = np.ascontiguousarray(dn[r * per * hidden:(r + 1) * per * hidden])
        bank_gu = q.QWWeightView(torch.from_numpy(gu_l.reshape(-1)).cuda(), per * 2 * inter, hidden, cont)
        bank_dn = q.QWWeightView(torch.from_numpy(dn_l.reshape(-1)).cuda(), per * hidden, inter, cont)
        nsc = lib.qwc_ep_scratch_bytes(ctypes.byref(ctx), max(t_per_rank), e, k, hidden, inter)
        scratch = torch.empty(nsc + 256, dtype=torch.uint8, device=dev)
        sc_ptr = (scratch.data_ptr() + 255) // 256 * 256
        ranks.append({"ctx": ctx, "gu": bank_gu, "dn": bank_dn, "scratch": scratch, "sc": ctypes.c_void_p(sc_ptr), "nsc": nsc})
    st = _stream_ptr(None)
    for call in range(calls):
        xs = [rng.standard_normal((t, hidden)).astype(np.float16) for t in t_per_rank]
        lgs = [rng.standard_normal((t, e)).astype(np.float32) for t in t_per_rank]
        xd = [torch.from_numpy(x).cuda() if x.size else None for x in xs]
        ld = [torch.from_numpy(l).cuda() if l.size else None for l in lgs]
        outs = [torch.full((max(t, 1), hidden), float("nan"), dtype=torch.float32, device=dev) for t in t_per_rank]
        for r, R in enumerate(ranks):
            if host_epoch:
                R["ctx"].epoch = call + 1
            t = t_per_rank[r]
            rc = lib.qwc_ep_dispatch(hal.handle, st, ctypes.byref(R["ctx"]), e, xd[r].data_ptr() if t else None, t, hidden, hidden, 0,
                                     ld[r].data_ptr() if t else None, k, 1, 0.0, R["sc"], R["nsc"], inter)
            assert rc == 0, _lib.last_error()
        for r, R in enumerate(ranks):
            rc = lib.qwc_ep_experts(hal.handle, st, ctypes.byref(R["ctx"]), ctypes.byref(R["gu"].c), ctypes.byref(R["dn"].c), e, inter,
                                    t_per_rank[r], k, R["sc"], R["nsc"])
            assert rc == 0, _lib.last_error()
        for r, R in enumerate(ranks):
            t = t_per_rank[r]
            rc = lib.qwc_ep_combine(hal.handle, st, ctypes.byref(R["ctx"]), e, inter, t, k, hidden, outs[r].data_ptr() if t else None, 1,
                                    R["sc"], R["nsc"])
            assert rc == 0, _lib.last_error()
        assert hal.device_status() == 0
        for r in range(world):
            t = t_per_rank[r]
            if t == 0:
                continue
            ridx, rwts = oracle.moe_route(lgs[r], k, norm_topk=True)
            ref = oracle.moe_forward(gu, dn, fmt, e, hidden, inter, xs[r], ridx, rwts)
            assert_matmul_close(outs[r][:t].cpu().numpy(), ref, tight=6e-3)


@pytest.mark.parametrize("name", ["HQ4_G32", "HQ8_G32"])
@pytest.mark.parametrize("world,e,k,hidden,inter,tokens", [(2, 8, 2, 256, 128, (40, 40)), (4, 16, 4, 256, 128, (33, 0, 7, 64)),
                                                           (1, 8, 2, 128, 128, (50,)), (8, 32, 8, 256, 256, (9, 9, 9, 9, 9, 9, 9, 9))])
def test_expert_parallel_phases_match_the_single_device_block(hal, oracle, name, world, e, k, hidden, inter, tokens):
    import qwegn_b200 as q
    _emulated_group(q, hal, oracle, name, world, e, k, hidden, inter, list(tokens), seed=world * 100 + e)


def test_expert_parallel_with_host_counted_calls(hal, oracle):
    import qwegn_b200 as q
    _emulated_group(q, hal, oracle, "HQ4_G32", 2, 8, 2, 256, 128, [16, 24], seed=5, calls=3, host_epoch=True)


def test_expert_parallel_refusals_come_before_any_launch(hal, oracle):
    import qwegn_b200 as q
    from qwegn_b200 import _lib, parallel as par
    from qwegn_b200.gemm import _stream_ptr
    lib = _lib.load()
    ctx = par.EpCtxC()
    ctx.rank, ctx.world, ctx.capacity_rows = 0, 3, 64
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    for p in range(3):
        ctx.recv[p] = ctx.counts[p] = ctx.ret[p] = ctx.flags[p] = buf.data_ptr()
    # 8 experts do not divide over 3 ranks
    rc = lib.qwc_ep_dispatch(hal.handle, _stream_ptr(None), ctypes.byref(ctx), 8, buf.data_ptr(), 4, 128, 128, 0, buf.data_ptr(), 2, 1, 0.0,
                             buf.data_ptr(), buf.numel(), 128)
    assert rc == 4 and b"divide" in lib.qwc_last_error()
    ctx.world = 2
    # more rows than the context was sized for
    rc = lib.qwc_ep_dispatch(hal.handle, _stream_ptr(None), ctypes.byref(ctx), 8, buf.data_ptr(), 64, 128, 128, 0, buf.data_ptr(), 2, 1, 0.0,
                             buf.data_ptr(), buf.numel(), 128)
    assert rc == 3 and b"capacity" in lib.qwc_last_error()
    torch.cuda.synchronize()
    assert bool((buf == 0).all())
