"""Prefill GEMM (tcgen05 path, M > 16) through the C ABI against the oracle."""
import numpy as np
import pytest
import torch

from conftest import assert_matmul_close

pytestmark = pytest.mark.gpu


def _bank(q, blocks, name):
    n, nb, _ = blocks.shape
    k = nb * q.CONTAINERS[name].group
    return q.QWWeightView(torch.from_numpy(np.ascontiguousarray(blocks).reshape(-1)).cuda(), n, k, q.CONTAINERS[name])


def _run(q, hal, view, x, out_dtype=torch.float16, rotated=False):
    m = x.shape[0]
    y = torch.full((m, view.n), float("nan"), dtype=out_dtype, device="cuda")
    nws = q.QWGemm.workspaceBytes(hal, view, m, 0, rotated)
    ws = torch.empty(nws, dtype=torch.uint8, device="cuda") if nws else None
    q.QWGemm.encode(hal, view, torch.from_numpy(np.ascontiguousarray(x)).cuda(), y, x_is_rotated=rotated, workspace=ws)
    return y.float().cpu().numpy()


def _tensor_path(name, k):
    """The tensor-core kernel takes K in whole raw steps: 128 k (blocks of 32), 256 k (HQ4_G64's blocks of 64)."""
    return k % (256 if name == "HQ4_G64" else 128) == 0


@pytest.mark.parametrize("name", ["HQ4_G32", "HQ8_G32", "HQ4_G64"])
@pytest.mark.parametrize("shape", [(16, 128, 128), (17, 128, 128), (17, 128, 256), (64, 200, 512), (129, 136, 768), (256, 128, 1024),
                                   (300, 1000, 640), (300, 264, 1280), (1024, 384, 2560)])
def test_prefill_vs_oracle(hal, oracle, name, shape):
    # HQ4_G64 rows are 16-byte aligned exactly when K % 256 == 0; the other shapes take the row-wise kernel (backend 3),
    # whatever the token count: covered here too.
    import qwegn_b200 as q
    m, n, k = shape
    assert q.QWGemm.plan(m, n, k, q.CONTAINERS[name]).backend == (2 if _tensor_path(name, k) else 3)
    fmt = oracle.FORMATS[name]
    rng = np.random.default_rng(m + n + k)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), fmt)
    x = rng.standard_normal((m, k)).astype(np.float16)
    view = _bank(q, blocks, name)
    yref = oracle.matmul(blocks, fmt, x)
    assert_matmul_close(_run(q, hal, view, x, out_dtype=torch.float32), yref)
    assert_matmul_close(_run(q, hal, view, x), yref, tight=3e-3)
    xr = oracle.fwht32_f16(x)
    assert_matmul_close(_run(q, hal, view, xr, rotated=True, out_dtype=torch.float32), yref)


@pytest.mark.parametrize("name", ["HQ4_G32", "HQ8_G32", "HQ4_G64"])
@pytest.mark.parametrize("shape", [(17, 64, 128), (64, 64, 256), (100, 192, 512), (300, 512, 640), (513, 128, 2048)])
def test_prefill_fused_swiglu_epilogues(hal, oracle, name, shape):
    # Fused gate/up GEMM + SwiGLU (+ FWHT-32) on the tensor path: gate rows [0, I), up rows [I, 2I) of one bank
    # (the reference's gemmBatchedH16SwiGLU, EncodeKernels.swift:156-228); oracle as gen_mlp_fixtures.py:71-79.
    import qwegn_b200 as q
    m, inter, k = shape
    if not _tensor_path(name, k):
        pytest.skip("HQ4_G64 rows are 16-byte aligned only for K % 256 == 0; the fused FWHT epilogue needs that")
    fmt = oracle.FORMATS[name]
    rng = np.random.default_rng(m + inter + k)
    blocks = oracle.quantize(rng.normal(0.0, 0.03, (2 * inter, k)).astype(np.float32), fmt)
    x = rng.standard_normal((m, k)).astype(np.float16)
    view = _bank(q, blocks, name)
    gu = oracle.matmul(blocks, fmt, x)
    xd = torch.from_numpy(x).cuda()
    for epi, rotate, tight in ((q.EPI_SILU_PAIR, False, 4e-3), (q.EPI_SILU_PAIR_FWHT, True, 5e-3)):
        href = oracle.swiglu_f16(gu, rotate=rotate).astype(np.float32)
        for dt in (torch.float16, torch.float32):
            y = torch.full((m, inter), float("nan"), dtype=dt, device="cuda")
            ws = torch.empty(q.QWGemm.workspaceBytes(hal, view, m, epi, False), dtype=torch.uint8, device="cuda")
            q.QWGemm.encode(hal, view, xd, y, epi=epi, workspace=ws)
            assert_matmul_close(y.float().cpu().numpy(), href, tight=tight)
    assert hal.device_status() == 0


def test_prefill_matches_the_gemv_path_row_by_row(hal, oracle):
    # Twin test (Tests/QWGEMMTests/QWBatchedGemmTests.swift:37-140: batched GEMM vs per-row GEMV, max |d| < 0.05).
    import qwegn_b200 as q
    m, n, k = 96, 512, 1024
    rng = np.random.default_rng(12)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), oracle.HQ4_G32)
    x = rng.standard_normal((m, k)).astype(np.float16)
    view = _bank(q, blocks, "HQ4_G32")
    y = _run(q, hal, view, x, out_dtype=torch.float32)
    rows = np.concatenate([_run(q, hal, view, x[i:i + 8], out_dtype=torch.float32) for i in range(0, m, 8)])
    assert np.abs(y - rows).max() < 1e-3


def test_prefill_needs_workspace_for_plain_activations(hal, oracle):
    import qwegn_b200 as q
    m, n, k = 64, 128, 256
    blocks = oracle.quantize(np.ones((n, k), dtype=np.float32), oracle.HQ4_G32)
    view = _bank(q, blocks, "HQ4_G32")
    # standard-basis activations are rotated into the workspace (short ones with a padded row stride); rotated ones are
    # read in place from 16 tokens on and staged below that
    assert q.QWGemm.workspaceBytes(hal, view, m, 0, False) >= m * k * 2
    assert q.QWGemm.workspaceBytes(hal, view, 4096, 0, False) == 4096 * k * 2
    assert q.QWGemm.workspaceBytes(hal, view, m, 0, True) == 0
    assert q.QWGemm.workspaceBytes(hal, view, 12, 0, True) >= 12 * k * 2
    x = torch.zeros((m, k), dtype=torch.float16, device="cuda")
    y = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    with pytest.raises(q.QWGemmError):
        q.QWGemm.encode(hal, view, x, y)
