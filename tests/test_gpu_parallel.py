"""Tensor-parallel MLP and expert-parallel MoE on 2 GPUs (NCCL) against the single-device oracle.
Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, results):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import qwegn_b200 as q
        from qwegn_b200 import parallel as par
        from oracle import qw_oracle as qo
        hal = q.QWHal(rank)
        fmt, cont = qo.HQ4_G32, q.CONTAINERS["HQ4_G32"]
        rng = np.random.default_rng(9)   # identical data on every rank

        # ---- tensor-parallel MLP: column-parallel gate||up (SwiGLU + FWHT fused), row-parallel down, all-reduce
        hidden, inter = 512, 1024
        gu = qo.quantize(rng.normal(0, 0.05, (2 * inter, hidden)).astype(np.float32), fmt)
        dn = qo.quantize(rng.normal(0, 0.05, (hidden, inter)).astype(np.float32), fmt)
        mlp = par.TPMlp(hal, torch.from_numpy(gu.reshape(-1)), torch.from_numpy(dn.reshape(-1)), hidden, inter, cont, rank, world)
        for m in (1, 8):
            x = rng.standard_normal((m, hidden)).astype(np.float16)
            h_loc = torch.empty((m, mlp.inter_local), dtype=torch.float16, device="cuda")
            y = torch.empty((m, hidden), dtype=torch.float32, device="cuda")
            mlp.forward(torch.from_numpy(x).cuda(), h_loc, y)
            ref = qo.matmul(dn, fmt, qo.swiglu_f16(qo.matmul(gu, fmt, x), rotate=True), x_is_rotated=True)
            err = np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max()
            assert err < 3e-3, ("tp mlp", m, err)

        # ---- the same MLP with the all-reduce fused into the down projection's kernel (peer stores + flags over symmetric
        # memory): same answer as the oracle, identical bits on every rank, and stable over many calls (two buffers in turn)
        mlp_f = par.TPMlp(hal, torch.from_numpy(gu.reshape(-1)), torch.from_numpy(dn.reshape(-1)), hidden, inter, cont, rank, world,
                          fused_allreduce=True)
        assert isinstance(mlp_f.down, par.FusedRowParallelLinear)
        for it_ in range(6):
            m = (1, 8, 3)[it_ % 3]
            x = rng.standard_normal((m, hidden)).astype(np.float16)
            h_loc = torch.empty((m, mlp_f.inter_local), dtype=torch.float16, device="cuda")
            y = torch.full((m, hidden), float("nan"), dtype=torch.float32, device="cuda")
            mlp_f.forward(torch.from_numpy(x).cuda(), h_loc, y)
            ref = qo.matmul(dn, fmt, qo.swiglu_f16(qo.matmul(gu, fmt, x), rotate=True), x_is_rotated=True)
            err = np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max()
            assert err < 3e-3, ("tp mlp fused", m, err)
            gathered = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(gathered, y)
            assert all(torch.equal(gathered[0], g) for g in gathered), "ranks disagree bitwise"
        assert hal.device_status() == 0

        # ---- expert-parallel MoE: tokens sharded over ranks, experts sharded over ranks
        e, k, hid, it, t_total = 16, 4, 256, 128, 96
        bgu = qo.quantize(rng.normal(0, 0.05, (e * 2 * it, hid)).astype(np.float32), fmt)
        bdn = qo.quantize(rng.normal(0, 0.05, (e * hid, it)).astype(np.float32), fmt)
        xs = rng.standard_normal((t_total, hid)).astype(np.float16)
        lg = rng.standard_normal((t_total, e)).astype(np.float32)
        ep = par.EPMoE(hal, torch.from_numpy(bgu.reshape(-1)), torch.from_numpy(bdn.reshape(-1)), e, hid, it, k, cont, rank, world)
        t0, t1 = t_total * rank // world, t_total * (rank + 1) // world
        out = ep.forward(torch.from_numpy(xs[t0:t1]).cuda(), torch.from_numpy(lg[t0:t1]).cuda())
        ridx, rwts = qo.moe_route(lg[t0:t1], k, norm_topk=True)
        ref = qo.moe_forward(bgu, bdn, fmt, e, hid, it, xs[t0:t1], ridx, rwts)
        err = np.abs(out.cpu().numpy() - ref).max() / np.abs(ref).max()
        assert err < 8e-3, ("ep moe", err)
        assert hal.device_status() == 0

        # ---- the same block with the exchange inside the library (peer stores + flags; no NCCL, no host read), twice
        # eagerly and once more as a replayed CUDA graph (the call number is counted on the device)
        epf = par.EPMoEFused(hal, torch.from_numpy(bgu.reshape(-1)), torch.from_numpy(bdn.reshape(-1)), e, hid, it, k, cont, rank, world,
                             max_tokens=t1 - t0)
        xd, ld = torch.from_numpy(xs[t0:t1]).cuda(), torch.from_numpy(lg[t0:t1]).cuda()
        outf = torch.full((t1 - t0, hid), float("nan"), dtype=torch.float32, device="cuda")
        for _ in range(2):
            epf.forward(xd, ld, outf)
            err = np.abs(outf.cpu().numpy() - ref).max() / np.abs(ref).max()
            assert err < 8e-3, ("ep moe fused", err)
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                epf.forward(xd, ld, outf)
        for _ in range(3):
            outf.fill_(float("nan"))
            g.replay()
            torch.cuda.synchronize()
            err = np.abs(outf.cpu().numpy() - ref).max() / np.abs(ref).max()
            assert err < 8e-3, ("ep moe fused, graph replay", err)
        assert hal.device_status() == 0

        # ---- tensor-parallel layer stack (HQ8_G32 attention projections, HQ4_G32 MLP) against the same stack on one device
        hidden, inter, qh, kvh, hd = 512, 1024, 8, 2, 64
        c8 = q.CONTAINERS["HQ8_G32"]
        planes = []
        for _ in range(2):
            planes.append({
                "qkv": torch.from_numpy(qo.quantize(rng.normal(0, 0.05, ((qh + 2 * kvh) * hd, hidden)).astype(np.float32), qo.HQ8_G32).reshape(-1)),
                "o": torch.from_numpy(qo.quantize(rng.normal(0, 0.05, (hidden, qh * hd)).astype(np.float32), qo.HQ8_G32).reshape(-1)),
                "gate_up": torch.from_numpy(qo.quantize(rng.normal(0, 0.05, (2 * inter, hidden)).astype(np.float32), fmt).reshape(-1)),
                "down": torch.from_numpy(qo.quantize(rng.normal(0, 0.05, (hidden, inter)).astype(np.float32), fmt).reshape(-1))})
        one = par.TPLayerStack([par.TPLayer(hal, pl, hidden, inter, qh, kvh, hd, c8, cont, 0, 1, fused_allreduce=False) for pl in planes], hal)
        tp = par.TPLayerStack([par.TPLayer(hal, pl, hidden, inter, qh, kvh, hd, c8, cont, rank, world, fused_allreduce=True) for pl in planes], hal)
        for mtok, chunk in ((1, 0), (5, 0), (300, 128)):
            x0 = torch.from_numpy(rng.standard_normal((mtok, hidden)).astype(np.float16)).cuda()
            xn_a, res_a = torch.empty_like(x0), x0.clone()
            q.QWGemm.encodeRMSNorm(hal, x0, one.layers[0].gamma1, xn_a)
            xn_b, res_b = xn_a.clone(), res_a.clone()
            one.forward(xn_a, res_a, one.buffers(mtok))
            tp.forward(xn_b, res_b, tp.buffers(mtok), chunk=chunk)
            torch.cuda.synchronize()
            a, b = res_a.float().cpu().numpy(), res_b.float().cpu().numpy()
            err = np.abs(a - b).max() / np.abs(a).max()
            assert np.isfinite(b).all() and err < 1e-2, ("tp layer stack", mtok, err)
        assert hal.device_status() == 0
        results[rank] = True
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_mlp_and_ep_moe_on_two_gpus():
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert all(results.get(r) for r in range(world))
