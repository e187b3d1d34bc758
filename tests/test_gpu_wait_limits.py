"""A bounded device wait that runs out: the kernel must return by itself, report through the status word and leave the
context usable.  The failure is made on the host side of the protocol (a peer that never makes the call), never by a
fault: the fused row-parallel matmul + all-reduce is called for a world of two with both ranks' inboxes and flags in
local memory, and the second rank is simply never launched, so its slots never carry the call's number."""
import ctypes
import time

import numpy as np
import pytest
import torch

from conftest import assert_matmul_close

pytestmark = pytest.mark.gpu


def test_peer_wait_runs_out_and_the_context_stays_usable(oracle):
    import qwegn_b200 as q
    from qwegn_b200 import _lib
    from qwegn_b200.gemm import _stream_ptr
    from qwegn_b200.parallel import AllReduceCtxC
    lib = _lib.load()
    hal = q.QWHal(0)          # a context of its own: its status word will be non-zero at the end
    n, k, m = 512, 1024, 1
    rng = np.random.default_rng(5)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), oracle.HQ4_G32)
    view = q.QWWeightView(torch.from_numpy(blocks.reshape(-1)).cuda(), n, k, q.CONTAINERS["HQ4_G32"])
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).cuda()
    y = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    world, sms = 2, hal.sm_count
    inbox = torch.zeros((world, world, m, n, 2), dtype=torch.float32, device="cuda")    # [owner rank][source rank][m][n] slots of (value, call number)
    ctx = AllReduceCtxC()
    ctx.rank, ctx.world, ctx.epoch = 0, world, 1
    ctx.reserved = 20000     # wait limit in microseconds: 20 ms instead of the default second
    for r in range(world):
        ctx.inbox[r] = inbox[r].data_ptr()
    ctx.inbox_floats = 2 * world * m * n
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = lib.qwc_gemm_allreduce(hal.handle, _stream_ptr(None), ctypes.byref(view.c), x.data_ptr(), m, k, y.data_ptr(), 1, n, 0,
                                ctypes.byref(ctx))
    assert rc == 0, _lib.last_error()
    status = hal.device_status()          # synchronises: the kernel has returned
    elapsed = time.perf_counter() - t0
    assert status == 105, status          # QWC_DEV_WAIT_PEER_TIMEOUT
    assert elapsed < 5.0, elapsed         # it gave up after the limit, not after the default second per CTA wave
    # rank 0's own partial sums did arrive in its inbox slot: the matmul itself ran
    yref = oracle.matmul(blocks, oracle.HQ4_G32, x.cpu().numpy())
    assert_matmul_close(inbox[0, 0, :, :, 0].cpu().numpy(), yref)
    assert (inbox[0, 0, :, :, 1].view(torch.int32) == 1).all()       # every slot of rank 0 carries the call's number
    hal.close()
    # the context is intact: a fresh hal computes the same product
    hal2 = q.QWHal(0)
    y2 = torch.empty((m, n), dtype=torch.float32, device="cuda")
    q.QWGemm.encode(hal2, view, x, y2)
    assert_matmul_close(y2.cpu().numpy(), yref)
    assert hal2.device_status() == 0
    hal2.close()
