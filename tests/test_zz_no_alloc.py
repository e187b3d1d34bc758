"""The scratch-free small-M door, qwc_gemm_static_scratch, through the C ABI.

It exists for hosts that cannot allocate device memory where they call the library (a frozen arena, a thread that
must not synchronise the device, a committed memory budget): the scratch of a K-sliced call lives in a fixed 2 MiB
array inside the library.  The test compares it with the ordinary door (caller workspace) on two calls in a row --
the array is shared and keeps the previous call's contents, so the second call must not be disturbed by the first --
and checks that a need beyond the array is refused.  This file sorts last so that every other test has run before it."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_door_matches_the_workspace_door_twice_in_a_row(hal, oracle):
    import qwegn_b200 as q
    from qwegn_b200 import noalloc
    n, k, m = 300, 5120, 16          # 16 tokens x K = 5120: K is sliced, the raw sums go through scratch
    fmt = oracle.HQ4_G32
    rng = np.random.default_rng(21)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), fmt)
    view = q.QWWeightView(torch.from_numpy(blocks.reshape(-1)).cuda(), n, k)
    need = q.QWGemm.workspaceBytes(hal, view, m)
    assert 0 < need <= noalloc.static_scratch_capacity() == 2 << 20
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    for call in range(2):
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).cuda()
        want = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        q.QWGemm.encode(hal, view, x, want, workspace=ws)
        got = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        noalloc.encode_static_scratch(hal, view, x, got)
        torch.cuda.synchronize()
        w_np, g_np = want.cpu().numpy(), got.cpu().numpy()
        assert np.isfinite(g_np).all()
        # same kernel, same arithmetic order: the tolerance of the matmul tests (max rel 2e-3) is met with room to spare
        assert np.abs(g_np - w_np).max() <= 2e-3 * np.abs(w_np).max(), f"call {call}"
        ref = oracle.matmul(blocks, fmt, x.cpu().numpy())
        assert np.abs(g_np - ref).max() <= 2e-3 * np.abs(ref).max(), f"call {call}"
    # the fused SwiGLU + FWHT epilogue takes the same path
    gu = oracle.quantize(rng.normal(0.0, 0.03, (256, k)).astype(np.float32), fmt)
    gview = q.QWWeightView(torch.from_numpy(gu.reshape(-1)).cuda(), 256, k)
    x = torch.from_numpy(rng.standard_normal((12, k)).astype(np.float16)).cuda()
    want = torch.empty((12, 128), dtype=torch.float16, device="cuda")
    got = torch.empty((12, 128), dtype=torch.float16, device="cuda")
    q.QWGemm.encode(hal, gview, x, want, epi=q.EPI_SILU_PAIR_FWHT, workspace=torch.empty(q.QWGemm.workspaceBytes(hal, gview, 12), dtype=torch.uint8, device="cuda"))
    noalloc.encode_static_scratch(hal, gview, x, got, epi=q.EPI_SILU_PAIR_FWHT)
    torch.cuda.synchronize()
    assert np.abs(got.float().cpu().numpy() - want.float().cpu().numpy()).max() <= 3e-3 * np.abs(want.float().cpu().numpy()).max()
    # a call that needs no scratch (one token) goes straight through
    y1 = torch.empty((1, n), dtype=torch.float32, device="cuda")
    y2 = torch.empty((1, n), dtype=torch.float32, device="cuda")
    q.QWGemm.encode(hal, view, x[:1], y1)
    noalloc.encode_static_scratch(hal, view, x[:1], y2)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)


def test_static_scratch_door_refuses_what_does_not_fit(hal):
    import qwegn_b200 as q
    from qwegn_b200 import noalloc
    n, k, m = 40000, 5120, 16        # 16 x 40000 x 4 B = 2.56 MB > 2 MiB
    bank = torch.zeros(n * (k // 32) * 20, dtype=torch.uint8, device="cuda")
    view = q.QWWeightView(bank, n, k)
    x = torch.zeros((m, k), dtype=torch.float16, device="cuda")
    y = torch.full((m, n), 3.0, dtype=torch.float32, device="cuda")
    with pytest.raises(q.QWGemmError) as e:
        noalloc.encode_static_scratch(hal, view, x, y)
    assert e.value.case == "badShape" and "scratch" in str(e.value)
    with pytest.raises(q.QWGemmError):     # more than 16 tokens belongs to the other door
        noalloc.encode_static_scratch(hal, view, torch.zeros((17, k), dtype=torch.float16, device="cuda"),
                                      torch.zeros((17, n), dtype=torch.float32, device="cuda"))
    torch.cuda.synchronize()
    assert (y == 3.0).all()
