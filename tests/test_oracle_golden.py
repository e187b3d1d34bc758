"""The CPU oracle against the reference's golden vectors (no GPU).

ref_fixtures.npz re-encodes the reference's own committed known-answer tests; formats.npz / matmul.npz hold outputs
of the reference's Python quantizer, dequantizer and fixture recipes (tests/golden/gen_golden.py).
"""
import numpy as np
import pytest

FMTS = ["HQ4_G32", "HQ8_G32", "HQ4_G64"]


def test_selfpack_blocks_and_dq4_bit_exact(oracle, golden):
    # Tests/QWQuantTests/QWQuantTests.swift:69-85: HQ4 dequant must be bit-identical to the numpy golden.
    g = golden["ref_fixtures"]
    blocks = oracle.quantize(g["selfpack_w"], oracle.HQ4_G32)
    assert np.array_equal(blocks, g["selfpack_blocks"])
    dq = oracle.dequant(g["selfpack_blocks"], oracle.HQ4_G32, standard=True)
    assert np.array_equal(dq.view(np.uint32), g["selfpack_dq4"].view(np.uint32))


def test_aq_quantizer_golden(oracle, golden):
    # Scripts/quantize/test_aq_golden.py:33-38: 4x64 bf16 values -> exact HQ4_G32_M5 block bytes.
    g = golden["ref_fixtures"]
    vals = (g["aqq_bf16"].astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(oracle.quantize(vals, oracle.HQ4_G32), g["aqq_blocks"])


def test_repack_golden_linear_nibble_order(oracle, golden):
    # aq_repack_golden.json: the 4-bit group-64 linear bit-stream order (byte b holds elements 2b, 2b+1).
    g = golden["ref_fixtures"]
    packed, codes = g["repack_packed"], g["repack_codes"]
    rows, cols = codes.shape
    blocks = np.zeros((rows, cols // 64, 36), dtype=np.uint8)
    blocks[..., 0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    blocks[..., 4:] = packed.reshape(rows, cols // 64, 32)
    dq = oracle.dequant(blocks, oracle.HQ4_G64)
    assert np.array_equal(dq, codes.astype(np.float32))
    # and MLX's own dequantized values: code * scale + bias
    want = g["repack_values"]
    got = codes.reshape(rows, -1, 64) * g["repack_scales"][..., None] + g["repack_biases"][..., None]
    assert np.abs(got.reshape(rows, cols) - want).max() < 1e-5


@pytest.mark.parametrize("name", FMTS)
def test_formats_vs_reference_python(oracle, golden, name):
    g = golden["formats"]
    fmt = oracle.FORMATS[name]
    blocks = oracle.quantize(g["w"], fmt)
    assert np.array_equal(blocks, g[f"{name}_blocks"])
    assert np.array_equal(oracle.dequant(blocks, fmt).view(np.uint32), g[f"{name}_rot"].view(np.uint32))
    assert np.array_equal(oracle.dequant(blocks, fmt, f16_round=True).view(np.uint32), g[f"{name}_rot16"].view(np.uint32))
    assert np.array_equal(oracle.dequant(blocks, fmt, standard=True).view(np.uint32), g[f"{name}_std"].view(np.uint32))


def test_fwht_vs_reference_python(oracle, golden):
    g = golden["formats"]
    assert np.array_equal(oracle.fwht32(g["fwht_in"]).view(np.uint32), g["fwht_out"].view(np.uint32))
    # involution: H(H(x)) == x up to rounding
    assert np.abs(oracle.fwht32(oracle.fwht32(g["fwht_in"])) - g["fwht_in"]).max() < 1e-5


def test_matmul_recipes(oracle, golden):
    # The fixture recipes feed activations that are used as they are (already in the weights' basis).
    g = golden["matmul"]
    x = g["s1_x"]
    for n in (32, 96):
        y = oracle.matmul(g[f"s1_N{n}_blocks"], oracle.HQ4_G32, x, x_is_rotated=True)
        np.testing.assert_allclose(y[0], g[f"s1_N{n}_y"], rtol=0, atol=2e-6)
    for nm in ("f5a", "f5b"):
        for m in (2, 3, 4, 8):
            y = oracle.matmul(g[f"{nm}_blocks"], oracle.HQ4_G32, g[f"{nm}_x_M{m}"], x_is_rotated=True)
            np.testing.assert_allclose(y, g[f"{nm}_y_M{m}"], rtol=0, atol=2e-5)


def test_mlp_recipe(oracle, golden):
    g = golden["matmul"]
    for m in (1, 2, 8):
        x = g[f"mlp_x_M{m}"]
        gu = oracle.matmul(g["mlp_gu_blocks"], oracle.HQ4_G32, x, x_is_rotated=True)
        h = oracle.swiglu_f16(gu)
        # h is a f16 rounding of an f32 value computed in a different summation order: allow one f16 ulp
        hd = np.abs(h.astype(np.float32) - g[f"mlp_h_M{m}"].astype(np.float32))
        assert (hd <= np.abs(g[f"mlp_h_M{m}"].astype(np.float32)) * 2.0 ** -10 + 1e-7).all()
        y = oracle.matmul(g["mlp_dn_blocks"], oracle.HQ4_G32, g[f"mlp_h_M{m}"], x_is_rotated=True)
        np.testing.assert_allclose(y, g[f"mlp_y_M{m}"], rtol=0, atol=1e-6)


def test_rotation_identity(oracle, golden):
    # x . H(W_rot)^T == H(x) . W_rot^T (Sources/Operators/QWGEMM/QWGemm.swift:285-287): plain x against the
    # standard-domain weights equals the rotated product within the f16 rounding of x_rot.
    g = golden["formats"]
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 256)).astype(np.float16)
    for name in FMTS:
        fmt = oracle.FORMATS[name]
        y = oracle.matmul(g[f"{name}_blocks"], fmt, x)
        w_std = oracle.dequant(g[f"{name}_blocks"], fmt, standard=True)
        yref = x.astype(np.float64) @ w_std.astype(np.float64).T
        assert np.abs(y - yref).max() <= 2e-3 * np.abs(yref).max()


def test_sparse_moe_golden(oracle, golden):
    # Tests/QWFlashNextTests/FNGoldenTests.swift:82: the HF module's sparse-MoE output for the committed weights.
    g = golden["ref_fixtures"]
    hidden, experts, topk, inter, shared, norm = (int(v) for v in g["moe_cfg"])
    x = g["moe_input"].reshape(-1, hidden)
    out = oracle.moe_forward_f32(x, g["moe_gate"], g["moe_gate_up"], g["moe_down"], topk, bool(norm),
                                 g["moe_sh_gate"], g["moe_sh_up"], g["moe_sh_down"], g["moe_sh_scalar"])
    np.testing.assert_allclose(out, g["moe_output"].reshape(-1, hidden), rtol=1e-4, atol=1e-5)


def test_router_ties_and_nonfinite(oracle):
    # qwrouter.metal:84-168: ties go to the lower id; non-finite logits are never chosen; -1 when none is left.
    lg = np.array([[1.0, 3.0, 3.0, 0.5], [np.inf, np.nan, 2.0, -np.inf]], dtype=np.float32)
    idx, wts = oracle.moe_route(lg, 2, norm_topk=True)
    assert idx[0].tolist() == [1, 2]
    np.testing.assert_allclose(wts[0], [0.5, 0.5], atol=1e-6)
    assert idx[1].tolist() == [2, -1]
    np.testing.assert_allclose(wts[1], [1.0, 0.0], atol=1e-6)


def test_group_pairs_is_a_stable_counting_sort(oracle):
    rng = np.random.default_rng(5)
    idx = rng.integers(-1, 8, size=(37, 4)).astype(np.int32)
    off, sp, st, inv = oracle.moe_group_pairs(idx, 8)
    flat = idx.reshape(-1)
    valid = np.nonzero(flat >= 0)[0]
    order = valid[np.argsort(flat[valid], kind="stable")]
    assert np.array_equal(sp[: order.size], order)
    assert np.array_equal(st[: order.size], order // 4)
    assert off[-1] == order.size
    assert np.array_equal(np.diff(off), np.bincount(flat[valid], minlength=8))
    assert (inv[flat < 0] == -1).all()
    assert np.array_equal(sp[inv[valid]], valid)
    te, tr = oracle.moe_tile_plan(off)
    cover = sum({1: 16, 2: 32, 3: 64}[int(r) >> 24] for r in tr)
    assert cover >= order.size and len(te) <= 8 + order.size // 64 + 1


def test_f32_matmul_restatement_agrees_with_the_f16_one(oracle):
    # same bank, f16-exact rotated activations: the f32 restatement (f32 decode) and the f16 one (f16-rounded decode)
    # differ only by the weight rounding; and rotating inside equals rotating first
    rng = np.random.default_rng(3)
    n, k = 96, 512
    for fmt in (oracle.HQ4_G32, oracle.HQ8_G32, oracle.HQ4_G64):
        blocks = oracle.quantize(rng.normal(0.0, 0.05, (n, k)).astype(np.float32), fmt)
        x = rng.standard_normal((3, k)).astype(np.float16)
        a = oracle.matmul(blocks, fmt, x, x_is_rotated=True)
        b = oracle.matmul_f32(blocks, fmt, x.astype(np.float32), 0, 1.0, True)
        assert np.abs(a - b).max() <= 2e-3 * np.abs(a).max()
        c = oracle.matmul_f32(blocks, fmt, x.astype(np.float32), 0, 1.0, False)
        d = oracle.matmul_f32(blocks, fmt, oracle.fwht32(x.astype(np.float32)), 0, 1.0, True)
        assert np.array_equal(c, d)
        s = oracle.matmul_f32(blocks, fmt, x.astype(np.float32), 2, 1.0, True)
        assert np.allclose(s, 1.0 / (1.0 + np.exp(-b.astype(np.float64))), atol=1e-6)
        e3 = oracle.matmul_f32(blocks, fmt, x.astype(np.float32), 3, 2.0, True)
        e1 = oracle.matmul_f32(blocks, fmt, x.astype(np.float32), 1, 2.0, True)
        assert np.allclose(oracle.fwht32(e3), e1, atol=1e-5)   # the rotation is an involution
