"""RMSNorm + FWHT-32 (the step before every quantized matmul in the reference's engine) against the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,hidden", [(1, 5120), (7, 2048), (33, 8192), (300, 256)])
@pytest.mark.parametrize("with_residual", [False, True])
@pytest.mark.parametrize("rotate", [True, False])
def test_rmsnorm_fwht_matches_the_oracle(hal, oracle, rows, hidden, with_residual, rotate):
    import qwegn_b200 as q
    rng = np.random.default_rng(rows + hidden)
    x = (rng.standard_normal((rows, hidden)) * 3.0).astype(np.float16)
    gamma = (rng.standard_normal(hidden) * 0.1).astype(np.float16)
    res = (rng.standard_normal((rows, hidden)) * 2.0).astype(np.float16) if with_residual else None
    yref, rref = oracle.rmsnorm_fwht(x, gamma, 1e-6, res, rotate)
    xd, gd = torch.from_numpy(x).cuda(), torch.from_numpy(gamma).cuda()
    rd = torch.from_numpy(res).cuda() if with_residual else None
    y = torch.full((rows, hidden), float("nan"), dtype=torch.float16, device="cuda")
    q.QWGemm.encodeRMSNorm(hal, xd, gd, y, 1e-6, rd, rotate)
    got = y.float().cpu().numpy()
    ref = yref.astype(np.float32)
    assert np.isfinite(got).all()
    # f16 outputs: at most one unit in the last place apart (the device sums the squares in f32, the oracle in f64)
    assert np.abs(got - ref).max() <= 2.0 ** -10 * np.maximum(np.abs(ref), 2.0 ** -14).max()
    assert (got == ref).mean() > 0.98
    if with_residual:
        assert np.array_equal(rd.cpu().numpy(), rref)   # residual += x, rounded to f16 once


def test_rmsnorm_feeds_the_matmul(hal, oracle):
    # norm -> GEMV with x_is_rotated=1 equals GEMV on the un-rotated normalised activations
    import qwegn_b200 as q
    n, k = 512, 1024
    rng = np.random.default_rng(5)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), oracle.HQ4_G32)
    view = q.QWWeightView(torch.from_numpy(blocks.reshape(-1)).cuda(), n, k, q.CONTAINERS["HQ4_G32"])
    x = rng.standard_normal((3, k)).astype(np.float16)
    gamma = (rng.standard_normal(k) * 0.1).astype(np.float16)
    xd, gd = torch.from_numpy(x).cuda(), torch.from_numpy(gamma).cuda()
    xrot = torch.empty_like(xd)
    xplain = torch.empty_like(xd)
    q.QWGemm.encodeRMSNorm(hal, xd, gd, xrot, rotate=True)
    q.QWGemm.encodeRMSNorm(hal, xd, gd, xplain, rotate=False)
    y1 = torch.empty((3, n), dtype=torch.float32, device="cuda")
    y2 = torch.empty((3, n), dtype=torch.float32, device="cuda")
    q.QWGemm.encode(hal, view, xrot, y1, x_is_rotated=True)
    q.QWGemm.encode(hal, view, xplain, y2, x_is_rotated=False)
    a, b = y1.cpu().numpy(), y2.cpu().numpy()
    assert np.abs(a - b).max() <= 4e-3 * np.abs(b).max()   # the two differ by one extra f16 rounding of the activations


def test_rmsnorm_refusals(hal):
    import qwegn_b200 as q
    x = torch.zeros((2, 1000), dtype=torch.float16, device="cuda")
    with pytest.raises(q.QWGemmError) as e:   # EncodeKernels.swift:350-357: hidden must be a multiple of 256
        q.QWGemm.encodeRMSNorm(hal, x, torch.zeros(1000, dtype=torch.float16, device="cuda"), torch.empty_like(x))
    assert e.value.case == "badGeometry"


@pytest.mark.parametrize("rows,n", [(1, 248320), (4, 151936), (3, 1000), (2, 7)])
def test_head_argmax_matches_the_oracle(hal, oracle, rows, n):
    import qwegn_b200 as q
    rng = np.random.default_rng(rows + n)
    lg = rng.standard_normal((rows, n)).astype(np.float32)
    lg[0, n // 2] = lg[0].max()          # a tie: the lower column wins
    lg[0, n // 3] = lg[0].max()
    if n > 10:
        lg[-1, 5] = np.nan               # NaN sorts lowest
        lg[-1, 6] = np.inf
    tok = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    q.QWGemm.encodeArgmax(hal, torch.from_numpy(lg).cuda(), tok)
    assert np.array_equal(tok.cpu().numpy(), oracle.head_argmax(lg))
    allnan = torch.full((1, n), float("nan"), dtype=torch.float32, device="cuda")
    q.QWGemm.encodeArgmax(hal, allnan, tok[:1])
    assert int(tok[0]) == 0
    zeros = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    zeros[0, 0] = -0.0
    q.QWGemm.encodeArgmax(hal, zeros, tok[:1])
    assert int(tok[0]) == int(oracle.head_argmax(zeros.cpu().numpy())[0])


def test_cast_seam(hal):
    import qwegn_b200 as q
    x = torch.randn(4096 + 8, device="cuda") * 300.0
    x[:4] = torch.tensor([65504.0, 70000.0, -1e-8, float("nan")], device="cuda")
    y = torch.empty(x.numel(), dtype=torch.float16, device="cuda")
    q.QWGemm.encodeCast(hal, x, y)
    ref = x.to(torch.float16)
    assert torch.equal(y[:3], ref[:3]) and torch.equal(y[4:], ref[4:]) and bool(torch.isnan(y[3]))
    with pytest.raises(q.QWGemmError) as e:   # QWGemm.swift:308-311
        q.QWGemm.encodeCast(hal, x[:12].contiguous(), y[:12].contiguous())
    assert e.value.case == "badWeights"
