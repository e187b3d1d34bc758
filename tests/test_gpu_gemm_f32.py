"""The f32-activation matmul door (the reference's encodeHQ4F32V4 / encodeHQ4F32BM) against the oracle's f32 restatement.
Tolerance: the matmul bar (max error <= 1e-2 of the output scale, cosine >= 0.9999); the device rounds the rotated
activations once to f16, the reference keeps them in f32."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(got, ref):
    assert np.isfinite(got).all()
    err = np.abs(got - ref).max() / (np.abs(ref).max() + 1e-30)
    cos = float((got.astype(np.float64) * ref).sum() / (np.linalg.norm(got.astype(np.float64)) * np.linalg.norm(ref) + 1e-30))
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)


def _run(q, hal, view, x, m, epi, scale, rotated, dtype=torch.float32):
    y = torch.full((m, view.n), float("nan"), dtype=dtype, device="cuda")
    ws = torch.empty(q.QWGemm.f32WorkspaceBytes(hal, view, m, epi) + 256, dtype=torch.uint8, device="cuda")
    q.QWGemm.encodeHQ4F32V4(hal, view, x, y, rows=m, epi=epi, scale=scale, x_is_rotated=rotated, workspace=ws)
    return y


@pytest.mark.parametrize("name", ["HQ4_G32", "HQ8_G32", "HQ4_G64"])
@pytest.mark.parametrize("m", [1, 3, 4, 7, 24])
@pytest.mark.parametrize("epi", [0, 1, 2, 3])
def test_f32_door_matches_the_oracle(hal, oracle, name, m, epi):
    import qwegn_b200 as q
    n, k = 384, 1024
    fmt = getattr(oracle, name)
    rng = np.random.default_rng(100 * m + epi)
    blocks = oracle.quantize(rng.normal(0.0, 0.05, (n, k)).astype(np.float32), fmt)
    view = q.QWWeightView(torch.from_numpy(blocks.reshape(-1)).cuda(), n, k, q.CONTAINERS[name])
    x = rng.standard_normal((m, k)).astype(np.float32)
    scale = 1.5 if epi in (1, 3) else 1.0
    for rotated in (True, False):
        ref = oracle.matmul_f32(blocks, fmt, x, epi, scale, rotated)
        y = _run(q, hal, view, torch.from_numpy(x).cuda(), m, epi, scale, rotated)
        _check(y.cpu().numpy(), ref)
    y16 = _run(q, hal, view, torch.from_numpy(x).cuda(), m, epi, scale, True, torch.float16)
    _check(y16.float().cpu().numpy(), oracle.matmul_f32(blocks, fmt, x, epi, scale, True))
    assert hal.device_status() == 0


def test_f32_door_equals_the_f16_door_on_f16_inputs(hal, oracle):
    # activations that are exact in f16 and already rotated: both doors must give the same bits
    import qwegn_b200 as q
    n, k, m = 512, 2048, 2
    rng = np.random.default_rng(8)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), oracle.HQ4_G32)
    view = q.QWWeightView(torch.from_numpy(blocks.reshape(-1)).cuda(), n, k, q.CONTAINERS["HQ4_G32"])
    x16 = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).cuda()
    y16 = torch.empty((m, n), device="cuda")
    q.QWGemm.encode(hal, view, x16, y16, x_is_rotated=True)
    y32 = _run(q, hal, view, x16.float(), m, 0, 1.0, True)
    assert torch.equal(y16, y32)


def test_f32_door_refusals(hal, oracle):
    import qwegn_b200 as q
    n, k = 64, 256
    blocks = oracle.quantize(np.zeros((n, k), dtype=np.float32) + 0.01, oracle.HQ4_G32)
    view = q.QWWeightView(torch.from_numpy(blocks.reshape(-1)).cuda(), n, k, q.CONTAINERS["HQ4_G32"])
    x = torch.zeros((1, k), device="cuda")
    y = torch.zeros((1, n), device="cuda")
    ws = torch.empty(1 << 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(q.QWGemmError):
        q.QWGemm.encodeHQ4F32V4(hal, view, x, y, epi=4, workspace=ws)
    with pytest.raises(q.QWGemmError):
        q.QWGemm.encodeHQ4F32V4(hal, view, x, y, epi=1, scale=0.0, workspace=ws)
    with pytest.raises(q.QWGemmError):
        q.QWGemm.encodeHQ4F32V4(hal, view, x, y, workspace=ws[:64])
    with pytest.raises(q.QWGemmError):
        q.QWGemm.encodeHQ4F32V4(hal, view, x.half(), y, workspace=ws)


def test_f32_door_back_to_back_with_static_weights(hal, oracle):
    # the decode-loop promise lets the library launch kernels ahead of their predecessors' end: a chain of calls that
    # share one workspace and feed each other must give the bits of the same chain run one call at a time
    import qwegn_b200 as q
    n = k = 1024
    rng = np.random.default_rng(12)
    blocks = oracle.quantize(rng.normal(0.0, 0.03, (n, k)).astype(np.float32), oracle.HQ4_G32)
    view = q.QWWeightView(torch.from_numpy(blocks.reshape(-1)).cuda(), n, k, q.CONTAINERS["HQ4_G32"])
    x0 = torch.from_numpy(rng.standard_normal((2, k)).astype(np.float32)).cuda()
    ws = torch.empty(q.QWGemm.f32WorkspaceBytes(hal, view, 2, 3) + 256, dtype=torch.uint8, device="cuda")

    def chain(sync):
        a, b = x0.clone(), torch.empty_like(x0)
        for _ in range(6):
            q.QWGemm.encodeHQ4F32V4(hal, view, a, b, rows=2, epi=3, scale=0.5, workspace=ws)
            if sync:
                torch.cuda.synchronize()
            a, b = b, a
        torch.cuda.synchronize()
        return a.clone()

    ref = chain(True)
    torch.cuda.synchronize()
    hal.set_static_weights(True)
    try:
        got = chain(False)
    finally:
        torch.cuda.synchronize()
        hal.set_static_weights(False)
    assert torch.isfinite(ref).all() and torch.equal(ref, got)
    assert hal.device_status() == 0
