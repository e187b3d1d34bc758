"""Host-side sharding and expert-parallel exchange logic on CPU (gloo, world size 2); no GPU, no kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import qwegn_b200 as q
from qwegn_b200 import parallel as par

FMTS = ["HQ4_G32", "HQ8_G32", "HQ4_G64"]


@pytest.mark.parametrize("name", FMTS)
def test_column_and_row_shards_are_byte_slices(oracle, name):
    fmt, cont = oracle.FORMATS[name], q.CONTAINERS[name]
    n, k, world = 96, 512, 4
    rng = np.random.default_rng(1)
    blocks = oracle.quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32), fmt)
    plane = torch.from_numpy(blocks.reshape(-1))
    full = oracle.dequant(blocks, fmt)
    x = rng.standard_normal((3, k)).astype(np.float16)
    xr = oracle.fwht32_f16(x)
    y_full = oracle.matmul(blocks, fmt, xr, x_is_rotated=True)
    y_sum = np.zeros_like(y_full)
    for r in range(world):
        sh, n_loc = par.column_shard(plane, n, k, cont, r, world)
        r0, r1 = par.row_range(n, r, world)
        assert n_loc == r1 - r0
        got = oracle.dequant(sh.numpy().reshape(n_loc, k // fmt.group, fmt.block_bytes), fmt)
        assert np.array_equal(got, full[r0:r1])
        shk, k_loc = par.row_shard(plane, n, k, cont, r, world)
        k0, k1 = par.k_range(k, cont, r, world)
        assert k_loc == k1 - k0 and k0 % 32 == 0 and k0 % fmt.group == 0
        bk = shk.numpy().reshape(n, k_loc // fmt.group, fmt.block_bytes)
        assert np.array_equal(oracle.dequant(bk, fmt), full[:, k0:k1])
        # each rank rotates only its own K slice: the partial products add up to the full product
        y_sum += oracle.matmul(bk, fmt, np.ascontiguousarray(x[:, k0:k1]))
    assert np.abs(y_sum - y_full).max() <= 1e-5 * np.abs(y_full).max()


def test_paired_column_shard_keeps_gate_and_up_together(oracle):
    fmt, cont = oracle.HQ4_G32, q.CONTAINERS["HQ4_G32"]
    inter, k, world = 128, 256, 4
    rng = np.random.default_rng(2)
    blocks = oracle.quantize(rng.normal(0, 0.02, (2 * inter, k)).astype(np.float32), fmt)
    plane = torch.from_numpy(blocks.reshape(-1))
    full = oracle.dequant(blocks, fmt)
    for r in range(world):
        sh, n_loc = par.column_shard(plane, 2 * inter, k, cont, r, world, paired=True, quantum=32)
        r0, r1 = par.row_range(inter, r, world, 32)
        got = oracle.dequant(sh.numpy().reshape(n_loc, k // 32, 20), fmt)
        assert np.array_equal(got[: n_loc // 2], full[r0:r1]) and np.array_equal(got[n_loc // 2:], full[inter + r0:inter + r1])
    with pytest.raises(q.QWGemmError):
        par.k_range(96, q.CONTAINERS["HQ4_G64"], 0, 2)   # 96 is not a multiple of lcm(32, 64)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ep_worker(rank, world, port, experts, top_k, tokens, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import qw_oracle as qo
        rng = np.random.default_rng(100 + rank)
        idx = rng.integers(-1, experts, size=(tokens, top_k)).astype(np.int32)
        off, sp, st, inv = qo.moe_group_pairs(idx, experts)
        valid = int(off[-1])
        # row payload: [source rank, pair index, expert id]
        rows = torch.zeros((tokens * top_k, 4), dtype=torch.float32)
        rows[:valid, 0] = rank
        rows[:valid, 1] = torch.from_numpy(sp[:valid].astype(np.float32))
        rows[:valid, 2] = torch.from_numpy(idx.reshape(-1)[sp[:valid]].astype(np.float32))
        plan = par.ep_exchange_counts(torch.from_numpy(off), experts, world)
        assert sum(plan.send_rows) == valid
        recv = par.ep_dispatch(rows, plan)
        eid = par.ep_received_expert_ids(plan)
        per = experts // world
        assert recv.shape[0] == sum(plan.recv_rows) == eid.numel()
        # every received row belongs to one of this rank's experts, in source-major, expert-sorted order
        assert torch.equal(recv[:, 2].to(torch.int32) - rank * per, eid)
        src = recv[:, 0]
        assert torch.all(src[1:] >= src[:-1])
        # a stand-in for the expert compute: mark the row with the local expert that served it
        recv[:, 3] = eid.float() + rank * per + 0.5
        back = par.ep_return(recv, plan)
        assert back.shape[0] == valid
        assert torch.equal(back[:, 1], rows[:valid, 1]) and torch.all(back[:, 0] == rank)
        assert torch.equal(back[:, 3], rows[:valid, 2] + 0.5)
        results[rank] = True
    finally:
        dist.destroy_process_group()


def test_expert_parallel_exchange_world2():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_ep_worker, args=(world, _free_port(), 8, 2, 37, results), nprocs=world, join=True)
    assert all(results.get(r) for r in range(world))


def _tp_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import qw_oracle as qo
        fmt, cont = qo.HQ4_G32, q.CONTAINERS["HQ4_G32"]
        hidden, inter, m = 128, 256, 3
        rng = np.random.default_rng(5)   # same data on every rank
        gu = qo.quantize(rng.normal(0, 0.05, (2 * inter, hidden)).astype(np.float32), fmt)
        dn = qo.quantize(rng.normal(0, 0.05, (hidden, inter)).astype(np.float32), fmt)
        x = rng.standard_normal((m, hidden)).astype(np.float16)
        # the tensor-parallel MLP with the oracle standing in for the kernels
        sh_gu, n_loc = par.column_shard(torch.from_numpy(gu.reshape(-1)), 2 * inter, hidden, cont, rank, world, paired=True, quantum=32)
        sh_dn, k_loc = par.row_shard(torch.from_numpy(dn.reshape(-1)), hidden, inter, cont, rank, world)
        assert k_loc == n_loc // 2
        g = qo.matmul(sh_gu.numpy().reshape(n_loc, hidden // 32, 20), fmt, x)
        h_loc = qo.swiglu_f16(g, rotate=True)
        part = qo.matmul(sh_dn.numpy().reshape(hidden, k_loc // 32, 20), fmt, h_loc, x_is_rotated=True)
        y = torch.from_numpy(part)
        dist.all_reduce(y)
        h_full = qo.swiglu_f16(qo.matmul(gu, fmt, x), rotate=True)
        ref = qo.matmul(dn, fmt, h_full, x_is_rotated=True)
        assert np.abs(y.numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
        results[rank] = True
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_mlp_world2():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_tp_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert all(results.get(r) for r in range(world))


def test_section_column_shard_keeps_every_ranks_heads(oracle):
    # A fused QKV plane: query, key and value rows are each cut over the ranks on head boundaries.
    fmt, cont = oracle.HQ8_G32, q.CONTAINERS["HQ8_G32"]
    heads, kv, hd, k, world = 8, 4, 32, 256, 4
    sections = [heads * hd, kv * hd, kv * hd]
    rng = np.random.default_rng(4)
    blocks = oracle.quantize(rng.normal(0, 0.02, (sum(sections), k)).astype(np.float32), fmt)
    plane = torch.from_numpy(blocks.reshape(-1))
    full = oracle.dequant(blocks, fmt)
    for r in range(world):
        sh, local = par.section_column_shard(plane, sections, k, cont, r, world, quantum=hd)
        assert local == [heads * hd // world, kv * hd // world, kv * hd // world]
        got = oracle.dequant(sh.numpy().reshape(sum(local), k // fmt.group, fmt.block_bytes), fmt)
        base, at = 0, 0
        for n_sec, n_loc in zip(sections, local):
            assert np.array_equal(got[at:at + n_loc], full[base + r * n_loc:base + (r + 1) * n_loc])
            base += n_sec
            at += n_loc
