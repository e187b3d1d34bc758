"""Device decode against the oracle and the golden vectors: bit-exact (integer/byte work, f32 results compared as bits)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FMTS = ["HQ4_G32", "HQ8_G32", "HQ4_G64"]


def _view(q, blocks, name):
    n, nb, _ = blocks.shape
    k = nb * q.CONTAINERS[name].group
    bank = torch.from_numpy(np.ascontiguousarray(blocks).reshape(-1)).cuda()
    return q.QWWeightView(bank, n, k, q.CONTAINERS[name]), n, k


def _dequant(q, hal, view, n, k, dtype=torch.float32, standard=False):
    out = torch.full((n, k), float("nan"), dtype=dtype, device="cuda")
    q.QWGemm.dequant(hal, view, out, standard_domain=standard)
    return out.cpu().numpy()


@pytest.mark.parametrize("name", FMTS)
def test_golden_formats_bit_exact(hal, golden, name):
    import qwegn_b200 as q
    g = golden["formats"]
    view, n, k = _view(q, g[f"{name}_blocks"], name)
    assert np.array_equal(_dequant(q, hal, view, n, k).view(np.uint32), g[f"{name}_rot"].view(np.uint32))
    assert np.array_equal(_dequant(q, hal, view, n, k, standard=True).view(np.uint32), g[f"{name}_std"].view(np.uint32))
    got16 = _dequant(q, hal, view, n, k, dtype=torch.float16)
    assert np.array_equal(got16.astype(np.float32).view(np.uint32), g[f"{name}_rot16"].view(np.uint32))


def test_selfpack_dq4_bit_exact(hal, golden):
    # Tests/QWQuantTests/QWQuantTests.swift:69-85 on the device.
    import qwegn_b200 as q
    g = golden["ref_fixtures"]
    view, n, k = _view(q, g["selfpack_blocks"], "HQ4_G32")
    got = _dequant(q, hal, view, n, k, standard=True)
    assert np.array_equal(got.view(np.uint32), g["selfpack_dq4"].view(np.uint32))


def test_repack_codes(hal, golden):
    import qwegn_b200 as q
    g = golden["ref_fixtures"]
    packed, codes = g["repack_packed"], g["repack_codes"]
    rows, cols = codes.shape
    blocks = np.zeros((rows, cols // 64, 36), dtype=np.uint8)
    blocks[..., 0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    blocks[..., 4:] = packed.reshape(rows, cols // 64, 32)
    view, n, k = _view(q, blocks, "HQ4_G64")
    assert np.array_equal(_dequant(q, hal, view, n, k), codes.astype(np.float32))


@pytest.mark.parametrize("name", FMTS)
@pytest.mark.parametrize("shape", [(1, 64), (7, 192), (333, 1024), (2048, 5120)])
def test_random_banks_bit_exact(hal, oracle, name, shape):
    import qwegn_b200 as q
    n, k = shape
    fmt = oracle.FORMATS[name]
    rng = np.random.default_rng(n * 131 + k)
    w = rng.normal(0.0, 0.02, (n, k)).astype(np.float32)
    w[0, :32] = 0.0
    blocks = oracle.quantize(w, fmt)
    view, n, k = _view(q, blocks, name)
    assert np.array_equal(_dequant(q, hal, view, n, k).view(np.uint32), oracle.dequant(blocks, fmt).view(np.uint32))
    assert np.array_equal(_dequant(q, hal, view, n, k, standard=True).view(np.uint32),
                          oracle.dequant(blocks, fmt, standard=True).view(np.uint32))


@pytest.mark.parametrize("name", FMTS)
def test_every_code_and_arbitrary_headers(hal, oracle, name):
    # Arbitrary block bytes (all codes, random f16 scale/bias incl. subnormals): decode is a pure function of bytes.
    import qwegn_b200 as q
    fmt = oracle.FORMATS[name]
    rng = np.random.default_rng(11)
    n, k = 64, 512
    blocks = rng.integers(0, 256, size=(n, k // fmt.group, fmt.block_bytes), dtype=np.uint8)
    hdr = rng.normal(0.0, 0.05, size=(n, k // fmt.group, 2)).astype(np.float16)
    hdr[0, 0, 0] = np.float16(6e-8)
    blocks[..., 0:4] = hdr.view(np.uint8).reshape(n, k // fmt.group, 4)
    view, n, k = _view(q, blocks, name)
    assert np.array_equal(_dequant(q, hal, view, n, k).view(np.uint32), oracle.dequant(blocks, fmt).view(np.uint32))


def test_fwht32_f16(hal, oracle):
    import qwegn_b200 as q
    rng = np.random.default_rng(2)
    x = rng.standard_normal((37, 1024)).astype(np.float16)
    xd = torch.from_numpy(x).cuda()
    q.QWGemm.encodeFwht32(hal, xd)
    assert np.array_equal(xd.cpu().numpy().view(np.uint16), oracle.fwht32_f16(x).view(np.uint16))
    with pytest.raises(q.QWGemmError):
        q.QWGemm.encodeFwht32(hal, torch.zeros(33, dtype=torch.float16, device="cuda"))
    q.QWGemm.encodeFwht32(hal, torch.zeros(0, dtype=torch.float16, device="cuda"))


def test_dequant_round_trip_full_size(hal, oracle):
    # Size-independent property at the decode-GEMV bench shape: quantize(dequant_std(blocks)) reproduces the
    # blocks' decoded values (idempotence of the codec on its own output), checked on the device's decode.
    import qwegn_b200 as q
    n, k = 12288, 4096
    rng = np.random.default_rng(0)
    w = rng.normal(0.0, 0.02, (n, k)).astype(np.float32)
    blocks = oracle.quantize(w, oracle.HQ4_G32)
    view, n, k = _view(q, blocks, "HQ4_G32")
    rot = _dequant(q, hal, view, n, k)
    std = _dequant(q, hal, view, n, k, standard=True)
    # inverse rotation of the standard-domain decode returns to the rotated decode (H is an involution)
    back = oracle.fwht32(std)
    assert np.abs(back - rot).max() <= 1e-6
    # quantization error bound: |w_rot - decode| <= scale/2 + |bias rounding| per group
    wrot = oracle.fwht32(w)
    scale = blocks[..., 0:2].copy().view(np.float16).astype(np.float32)
    err = np.abs(wrot - rot).reshape(n, k // 32, 32).max(axis=-1)
    assert (err <= scale[..., 0] * 0.5 + 1032 * scale[..., 0] * 2.0 ** -11 + 1e-7).all()


@pytest.mark.parametrize("name", FMTS)
def test_device_quantizer_bytes_equal_the_packer(hal, oracle, golden, name):
    # qwc_quantize must write the bytes the reference's Python packer writes (golden) and the oracle writes.
    import qwegn_b200 as q
    g = golden["formats"]
    got = q.QWGemm.quantize(hal, torch.from_numpy(g["w"]).cuda(), q.CONTAINERS[name]).cpu().numpy()
    assert np.array_equal(got, g[f"{name}_blocks"].reshape(-1))
    rng = np.random.default_rng(77)
    w = rng.normal(0.0, 0.02, (777, 2048)).astype(np.float32)
    w[5] = 0.0
    w[6, 3] = 500.0   # drives the HQ4_G32 scale clamp
    got = q.QWGemm.quantize(hal, torch.from_numpy(w).cuda(), q.CONTAINERS[name]).cpu().numpy()
    assert np.array_equal(got, oracle.quantize(w, oracle.FORMATS[name]).reshape(-1))


def test_aq_quantizer_golden_on_device(hal, golden):
    import qwegn_b200 as q
    g = golden["ref_fixtures"]
    vals = (g["aqq_bf16"].astype(np.uint32) << 16).view(np.float32)
    got = q.QWGemm.quantize(hal, torch.from_numpy(np.ascontiguousarray(vals)).cuda()).cpu().numpy()
    assert np.array_equal(got, g["aqq_blocks"].reshape(-1))
