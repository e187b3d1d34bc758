"""Decode GEMV / small-M verify GEMM through the C ABI against the oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

from conftest import assert_matmul_close

pytestmark = pytest.mark.gpu

FMTS = ["HQ4_G32", "HQ8_G32", "HQ4_G64"]


def _bank(q, blocks, name):
    n, nb, _ = blocks.shape
    k = nb * q.CONTAINERS[name].group
    bank = torch.from_numpy(np.ascontiguousarray(blocks).reshape(-1)).cuda()
    return q.QWWeightView(bank, n, k, q.CONTAINERS[name])


def _run(q, hal, view, x, epi=0, out_dtype=torch.float32, rotated=False):
    m = x.shape[0]
    n_out = view.n if epi == 0 else view.n // 2
    y = torch.full((m, n_out), float("nan"), dtype=out_dtype, device="cuda")
    nws = q.QWGemm.workspaceBytes(hal, view, m, epi, rotated)
    ws = torch.empty(nws, dtype=torch.uint8, device="cuda") if nws else None
    q.QWGemm.encode(hal, view, torch.from_numpy(np.ascontiguousarray(x)).cuda(), y, epi=epi, x_is_rotated=rotated,
                    workspace=ws)
    return y.float().cpu().numpy()


def test_s1_gemv_fixture(hal, golden):
    # gen_s1_q4_fixtures.py recipe (Tests/QWGEMMTests/QWGEMMTests.swift:108-119 uses |d| <= 2e-2).
    import qwegn_b200 as q
    g = golden["matmul"]
    x = g["s1_x"].reshape(1, -1)
    for n in (32, 96):
        y = _run(q, hal, _bank(q, g[f"s1_N{n}_blocks"], "HQ4_G32"), x, rotated=True)
        assert np.abs(y[0] - g[f"s1_N{n}_y"]).max() <= 2e-2
        assert_matmul_close(y[0], g[f"s1_N{n}_y"])


def test_f5_skinny_fixture(hal, golden):
    # gen_f5_fixtures.py recipe, M in {2,3,4,8} (QWGEMMTests.swift:167-219: <= 5e-4 or one f16 spacing).
    import qwegn_b200 as q
    g = golden["matmul"]
    for nm in ("f5a", "f5b"):
        view = _bank(q, g[f"{nm}_blocks"], "HQ4_G32")
        for m in (2, 3, 4, 8):
            y = _run(q, hal, view, g[f"{nm}_x_M{m}"], rotated=True)
            assert np.abs(y - g[f"{nm}_y_M{m}"]).max() <= 5e-4
            y16 = _run(q, hal, view, g[f"{nm}_x_M{m}"], out_dtype=torch.float16, rotated=True)
            ref = g[f"{nm}_y_M{m}"]
            assert (np.abs(y16 - ref) <= np.maximum(5e-4, np.abs(ref) * 2.0 ** -10)).all()


def test_mlp_fixture_chain(hal, golden):
    # gen_mlp_fixtures.py recipe: fused gate||up + SwiGLU (f16 h), then the down GEMV on that h.
    import qwegn_b200 as q
    g = golden["matmul"]
    gu = _bank(q, g["mlp_gu_blocks"], "HQ4_G32")
    dn = _bank(q, g["mlp_dn_blocks"], "HQ4_G32")
    for m in (1, 2, 8):
        h = _run(q, hal, gu, g[f"mlp_x_M{m}"], epi=q.EPI_SILU_PAIR, out_dtype=torch.float16, rotated=True)
        href = g[f"mlp_h_M{m}"].astype(np.float32)
        assert (np.abs(h - href) <= np.abs(href) * 2.0 ** -9 + 1e-6).all()
        y = _run(q, hal, dn, g[f"mlp_h_M{m}"], rotated=True)
        assert np.abs(y - g[f"mlp_y_M{m}"]).max() <= 5e-4


@pytest.mark.parametrize("name", FMTS)
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16])
def test_small_m_sweep_vs_oracle(hal, oracle, name, m):
    import qwegn_b200 as q
    n, k = 1000, 5120   # ragged N; K of the verify sweep
    fmt = oracle.FORMATS[name]
    rng = np.random.default_rng(100 + m)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), fmt)
    x = rng.standard_normal((m, k)).astype(np.float16)
    view = _bank(q, blocks, name)
    yref = oracle.matmul(blocks, fmt, x)
    assert_matmul_close(_run(q, hal, view, x), yref)
    assert_matmul_close(_run(q, hal, view, x, out_dtype=torch.float16), yref, tight=3e-3)
    # pre-rotated activations (the reference's dataflow) give the same answer
    xr = oracle.fwht32_f16(x)
    assert_matmul_close(_run(q, hal, view, xr, rotated=True), yref)


@pytest.mark.parametrize("name", FMTS)
@pytest.mark.parametrize("shape", [(1, 256), (17, 128), (16, 4096), (4097, 512), (300, 17408), (64, 28672)])
def test_shapes_incl_ragged_and_large_k(hal, oracle, name, shape):
    import qwegn_b200 as q
    n, k = shape
    if name == "HQ4_G64" and k % 256:
        k = 256 * ((k + 255) // 256)
    fmt = oracle.FORMATS[name]
    rng = np.random.default_rng(n + k)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), fmt)
    x = rng.standard_normal((3, k)).astype(np.float16)
    assert_matmul_close(_run(q, hal, _bank(q, blocks, name), x), oracle.matmul(blocks, fmt, x))


@pytest.mark.parametrize("name", FMTS)
def test_rowwise_fallback_for_unaligned_rows(hal, oracle, name):
    # K % 128 != 0: rows are not 16-byte aligned; the plan says ROWWISE and the answer is the same.
    import qwegn_b200 as q
    k = 192 if name == "HQ4_G64" else 96
    n = 37
    fmt = oracle.FORMATS[name]
    assert q.QWGemm.plan(2, n, k, q.CONTAINERS[name]).backend == 3
    rng = np.random.default_rng(9)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), fmt)
    x = rng.standard_normal((2, k)).astype(np.float16)
    assert_matmul_close(_run(q, hal, _bank(q, blocks, name), x), oracle.matmul(blocks, fmt, x))


@pytest.mark.parametrize("name", FMTS)
@pytest.mark.parametrize("m", [1, 4, 12])
def test_silu_pair_epilogues(hal, oracle, name, m):
    import qwegn_b200 as q
    inter, k = 1504 if name != "HQ4_G64" else 1504, 2048   # inter % 32 == 0, ragged against the 148-CTA split
    fmt = oracle.FORMATS[name]
    rng = np.random.default_rng(50 + m)
    blocks = oracle.quantize(rng.normal(0.0, 0.03, (2 * inter, k)).astype(np.float32), fmt)
    x = rng.standard_normal((m, k)).astype(np.float16)
    view = _bank(q, blocks, name)
    gu = oracle.matmul(blocks, fmt, x)
    href = oracle.swiglu_f16(gu).astype(np.float32)
    h = _run(q, hal, view, x, epi=q.EPI_SILU_PAIR, out_dtype=torch.float16)
    assert_matmul_close(h, href, tight=3e-3)
    hrot_ref = oracle.swiglu_f16(gu, rotate=True).astype(np.float32)
    hrot = _run(q, hal, view, x, epi=q.EPI_SILU_PAIR_FWHT, out_dtype=torch.float16)
    assert_matmul_close(hrot, hrot_ref, tight=4e-3)


def test_row_views_and_strided_activations(hal, oracle):
    # Column-parallel shard = a row range of the same bank; x and y rows may be strided.
    import qwegn_b200 as q
    n, k = 512, 1024
    fmt = oracle.HQ4_G32
    rng = np.random.default_rng(4)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), fmt)
    view = _bank(q, blocks, "HQ4_G32")
    xw = torch.from_numpy(rng.standard_normal((4, k + 64)).astype(np.float16)).cuda()
    x = xw[:, :k]
    yw = torch.zeros((4, n + 8), dtype=torch.float32, device="cuda")
    q.QWGemm.encode(hal, view.rows(128, 384), x, yw[:, :256])
    yref = oracle.matmul(blocks[128:384], fmt, x.cpu().numpy())
    assert_matmul_close(yw[:, :256].cpu().numpy(), yref)
    assert (yw[:, 256:] == 0).all()


def test_refusals_leave_the_stream_clean(hal, oracle):
    # Tests/QWGEMMTests/QWGEMMTests.swift:221-248: a refused encode throws before anything is launched.
    import qwegn_b200 as q
    fmt = oracle.HQ4_G32
    blocks = oracle.quantize(np.ones((5, 128), dtype=np.float32), fmt)
    view = _bank(q, blocks, "HQ4_G32")
    x = torch.zeros((1, 128), dtype=torch.float16, device="cuda")
    y = torch.full((1, 5), 7.0, dtype=torch.float32, device="cuda")
    with pytest.raises(q.QWGemmError) as e:
        q.QWGemm.encode(hal, view, x, y[:, :2], epi=q.EPI_SILU_PAIR)  # odd packed bank
    assert e.value.case == "badWeights"
    with pytest.raises(q.QWGemmError) as e:
        q.QWGemm.encode(hal, view, torch.zeros((1, 96), dtype=torch.float16, device="cuda"), y)
    assert e.value.case == "badShape"
    with pytest.raises(q.QWGemmError):
        q.QWGemm.encode(hal, view, x.float(), y)
    with pytest.raises(q.QWGemmError) as e:
        q.QWWeightView(torch.zeros(10, dtype=torch.uint8, device="cuda"), 5, 128)  # bank too short
    assert e.value.case == "badWeights"
    torch.cuda.synchronize()
    assert (y == 7.0).all()
    # empty batch is a no-op
    q.QWGemm.encode(hal, view, torch.zeros((0, 128), dtype=torch.float16, device="cuda"),
                    torch.zeros((0, 5), dtype=torch.float32, device="cuda"))


def test_decode_gemv_bench_shape_properties(hal, oracle):
    # Full-size config (N=12288, K=4096, seed 0): oracle parity, linearity in x and determinism.
    import qwegn_b200 as q
    n, k = 12288, 4096
    rng = np.random.default_rng(0)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), oracle.HQ4_G32)
    x = rng.standard_normal((1, k)).astype(np.float16)
    view = _bank(q, blocks, "HQ4_G32")
    y = _run(q, hal, view, x)
    assert_matmul_close(y, oracle.matmul(blocks, oracle.HQ4_G32, x))
    y2 = _run(q, hal, view, x)
    assert np.array_equal(y, y2), "split-K reduction must be deterministic"
    xa = rng.standard_normal((1, k)).astype(np.float16)
    xr = oracle.fwht32_f16(np.concatenate([x, xa]))
    s = (xr[0].astype(np.float32) + xr[1].astype(np.float32)).astype(np.float16).reshape(1, -1)
    ys = _run(q, hal, view, s, rotated=True)
    ya = _run(q, hal, view, xa)
    assert np.abs(ys - (y + ya)).max() <= 4e-3 * np.abs(ys).max()


def test_k_sliced_call_needs_and_uses_the_workspace(hal, oracle):
    # 15 tokens x K = 5120 on the stream kernel: the staged activations exceed their shared-memory share, K is processed
    # in slices and the raw sums travel through the caller's workspace.  From 9 tokens on the plain call takes the tensor
    # path, so the stream kernel is reached here through a SwiGLU epilogue whose halves are not whole 64-row tiles.
    import qwegn_b200 as q
    k, m, inter = 5120, 15, 96
    fmt = oracle.HQ4_G32
    rng = np.random.default_rng(8)
    x = rng.standard_normal((m, k)).astype(np.float16)
    gu = oracle.quantize(rng.normal(0.0, 0.03, (2 * inter, k)).astype(np.float32), fmt)
    view = _bank(q, gu, "HQ4_G32")
    assert q.QWGemm.plan(m, 2 * inter, k, q.CONTAINERS["HQ4_G32"], epi=q.EPI_SILU_PAIR_FWHT).backend == 1
    assert q.QWGemm.workspaceBytes(hal, view, m, q.EPI_SILU_PAIR_FWHT) == m * 2 * inter * 4
    assert q.QWGemm.workspaceBytes(hal, view, 1, q.EPI_SILU_PAIR_FWHT) == 0
    xd = torch.from_numpy(x).cuda()
    h = torch.zeros((m, inter), dtype=torch.float16, device="cuda")
    with pytest.raises(q.QWGemmError) as e:
        q.QWGemm.encode(hal, view, xd, h, epi=q.EPI_SILU_PAIR_FWHT)
    assert e.value.case == "badShape"
    href = oracle.swiglu_f16(oracle.matmul(gu, fmt, x), rotate=True).astype(np.float32)
    assert_matmul_close(_run(q, hal, view, x, epi=q.EPI_SILU_PAIR_FWHT, out_dtype=torch.float16), href, tight=4e-3)


def test_nine_to_fifteen_tokens_take_the_tensor_path_through_a_staged_copy(hal, oracle):
    # Below 16 tokens the activations are always staged into the workspace (rotated, or copied when they come rotated),
    # with a row stride that spreads the few rows over 136 KiB of addresses.
    import qwegn_b200 as q
    n, k = 200, 5120
    fmt = oracle.HQ4_G32
    rng = np.random.default_rng(18)
    blocks = oracle.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), fmt)
    view = _bank(q, blocks, "HQ4_G32")
    for m in (9, 12, 15):
        assert q.QWGemm.plan(m, n, k, q.CONTAINERS["HQ4_G32"]).backend == 2
        x = rng.standard_normal((m, k)).astype(np.float16)
        for rotated in (False, True):
            need = q.QWGemm.workspaceBytes(hal, view, m, 0, rotated)
            assert need >= max(m * k * 2, 136 * 1024)
            y = torch.zeros((m, n), dtype=torch.float32, device="cuda")
            with pytest.raises(q.QWGemmError) as e:
                q.QWGemm.encode(hal, view, torch.from_numpy(x).cuda(), y, x_is_rotated=rotated)
            assert e.value.case == "badShape"
        yref = oracle.matmul(blocks, fmt, x)
        assert_matmul_close(_run(q, hal, view, x), yref)
        assert_matmul_close(_run(q, hal, view, oracle.fwht32_f16(x), rotated=True), yref)
    assert hal.device_status() == 0


def test_static_weights_mode_gives_identical_results(oracle):
    # qwc_hal_set_static_weights: the kernels prefetch weights before the previous kernel of the stream has
    # finished; results must not change, including for back-to-back dependent calls (y of one call is x of the next).
    import qwegn_b200 as q
    hal2 = q.QWHal(0)
    n, k = 1024, 1024
    fmt = oracle.HQ4_G32
    rng = np.random.default_rng(31)
    blocks = oracle.quantize(rng.normal(0.0, 0.03, (n, k)).astype(np.float32), fmt)
    view = _bank(q, blocks, "HQ4_G32")
    x = torch.from_numpy(rng.standard_normal((1, k)).astype(np.float16)).cuda()
    outs = []
    for mode in (False, True):
        torch.cuda.synchronize()
        hal2.set_static_weights(mode)
        a = x.clone()
        for _ in range(6):   # a chain: each call consumes the previous call's output
            y = torch.empty((1, n), dtype=torch.float16, device="cuda")
            q.QWGemm.encode(hal2, view, a, y)
            a = y
        torch.cuda.synchronize()
        outs.append(a.float().cpu().numpy())
    assert np.array_equal(outs[0], outs[1])
    assert hal2.device_status() == 0
    hal2.close()
