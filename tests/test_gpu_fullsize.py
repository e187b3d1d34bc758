"""The benchmark configurations at their full sizes, through properties that do not need the (slow) CPU oracle:
determinism, exact scaling by a power of two, and agreement with a plain f32 matmul over the weights the device
dequantizer produces (that dequantizer is pinned bit-for-bit against the oracle in test_gpu_dequant.py)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(y, ref, tight):
    y, ref = y.double(), ref.double()
    assert torch.isfinite(y).all()
    err = float((y - ref).abs().max() / (ref.abs().max() + 1e-30))
    cos = float((y * ref).sum() / (y.norm() * ref.norm() + 1e-30))
    assert err <= 1e-2 and cos >= 0.9999 and err <= tight, (err, cos)


def _bank(q, hal, n, k, name, seed):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    w = torch.randn((n, k), generator=gen, device="cuda") * 0.02
    cont = q.CONTAINERS[name]
    view = q.QWWeightView(q.QWGemm.quantize(hal, w, cont), n, k, cont)
    del w
    wq = torch.empty((n, k), dtype=torch.float32, device="cuda")
    q.QWGemm.dequant(hal, view, wq, standard_domain=False)   # rotated-domain weights, f16-representable values
    return view, wq


def _encode(q, hal, view, x, dtype=torch.float32, epi=0):
    m = x.shape[0]
    n_out = view.n if epi == 0 else view.n // 2
    y = torch.full((m, n_out), float("nan"), dtype=dtype, device="cuda")
    nws = q.QWGemm.workspaceBytes(hal, view, m, epi, False)
    ws = torch.empty(max(nws, 16), dtype=torch.uint8, device="cuda")
    q.QWGemm.encode(hal, view, x, y, epi=epi, workspace=ws)
    return y


@pytest.mark.parametrize("name", ["HQ4_G32", "HQ8_G32", "HQ4_G64"])
def test_verify_sweep_shape_n17408_k5120(hal, name):
    # C2: N = 17408, K = 5120, M in {1, 2, 4, 8, 16}
    import qwegn_b200 as q
    n, k = 17408, 5120
    view, wq = _bank(q, hal, n, k, name, seed=2)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    for m in (1, 2, 4, 8, 16):
        x = torch.randn((m, k), generator=gen, device="cuda").to(torch.float16)
        y = _encode(q, hal, view, x)
        assert torch.equal(y, _encode(q, hal, view, x)), "not deterministic"
        # scaling x by 2 scales y by 2 (exactly, but for the few rotated activations that round as f16 subnormals)
        assert float((_encode(q, hal, view, x * 2) - y * 2).abs().max()) <= 1e-5 * float(y.abs().max())
        xr = x.clone()
        q.QWGemm.encodeFwht32(hal, xr)
        _close(y, xr.float() @ wq.t(), 3e-3)
    assert hal.device_status() == 0


def test_prefill_shapes_m4096(hal):
    # C3: M = 4096, K = 5120 with N = 34816 (gate||up, plain and fused SwiGLU + FWHT) and K = 17408, N = 5120 (down)
    import qwegn_b200 as q
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4)
    m = 4096
    view, wq = _bank(q, hal, 34816, 5120, "HQ4_G32", seed=5)
    x = torch.randn((m, 5120), generator=gen, device="cuda").to(torch.float16)
    xr = x.clone()
    q.QWGemm.encodeFwht32(hal, xr)
    ref = xr.float() @ wq.t()
    y = _encode(q, hal, view, x, dtype=torch.float16)
    assert torch.equal(y, _encode(q, hal, view, x, dtype=torch.float16)), "not deterministic"
    _close(y.float(), ref, 3e-3)
    inter = 17408
    g, u = ref[:, :inter].half().float(), ref[:, inter:].half().float()   # the reference rounds gate and up to f16 first
    h = (torch.nn.functional.silu(g) * u).half()
    href = h.clone()
    q.QWGemm.encodeFwht32(hal, href)
    del ref, g, u
    _close(_encode(q, hal, view, x, dtype=torch.float16, epi=q.EPI_SILU_PAIR).float(), h.float(), 5e-3)
    _close(_encode(q, hal, view, x, dtype=torch.float16, epi=q.EPI_SILU_PAIR_FWHT).float(), href.float(), 6e-3)
    del view, wq, y
    torch.cuda.empty_cache()
    view, wq = _bank(q, hal, 5120, 17408, "HQ4_G32", seed=6)
    x = torch.randn((m, 17408), generator=gen, device="cuda").to(torch.float16)
    xr = x.clone()
    q.QWGemm.encodeFwht32(hal, xr)
    _close(_encode(q, hal, view, x), xr.float() @ wq.t(), 3e-3)
    assert hal.device_status() == 0


# C5: one 70B-class layer (hidden 8192, intermediate 28672, 64 query + 8 key/value heads of 128): QKV and O in HQ8_G32, the MLP
# in HQ4_G32, whole and as the 1/8 shards of tensor parallelism (column shards cut N, row shards cut K)
_LAYER_BANKS = [
    ("HQ8_G32", 10240, 8192), ("HQ8_G32", 8192, 8192), ("HQ4_G32", 57344, 8192), ("HQ4_G32", 8192, 28672),
    ("HQ8_G32", 1280, 8192), ("HQ8_G32", 8192, 1024), ("HQ4_G32", 7168, 8192), ("HQ4_G32", 8192, 3584),
]


@pytest.mark.parametrize("name,n,k", _LAYER_BANKS)
def test_layer_bank_shapes_h8192_i28672(hal, name, n, k):
    import qwegn_b200 as q
    view, wq = _bank(q, hal, n, k, name, seed=n + k)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(n ^ k)
    for m in (1, 8192):
        x = torch.randn((m, k), generator=gen, device="cuda").to(torch.float16)
        dt = torch.float32 if m == 1 else torch.float16
        y = _encode(q, hal, view, x, dtype=dt)
        assert torch.equal(y, _encode(q, hal, view, x, dtype=dt)), "not deterministic"
        if m == 1:
            assert float((_encode(q, hal, view, x * 2, dtype=dt) - y * 2).abs().max()) <= 1e-5 * float(y.abs().max())
        xr = x.clone()
        q.QWGemm.encodeFwht32(hal, xr)
        _close(y.float(), xr.float() @ wq.t(), 3e-3)
        del x, xr, y
    assert hal.device_status() == 0


@pytest.mark.parametrize("tokens", [2048, 8])
def test_moe_block_t2048_e256_top8(hal, tokens):
    # C4: 256 experts, top-8, hidden 2048, expert intermediate 512; 2048 tokens (grouped tensor path) and 8 (decode path)
    import qwegn_b200 as q
    t, e, k, hid, inter = tokens, 256, 8, 2048, 512
    bgu, wgu = _bank(q, hal, e * 2 * inter, hid, "HQ4_G32", seed=7)
    bdn, wdn = _bank(q, hal, e * hid, inter, "HQ4_G32", seed=8)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(9)
    x = torch.randn((t, hid), generator=gen, device="cuda").to(torch.float16)
    lg = torch.randn((t, e), generator=gen, device="cuda")
    op = q.QWMoEOperator(hal, bgu, bdn, e, inter, k, norm_topk=True)
    sc = torch.empty(op.scratchBytes(t), dtype=torch.uint8, device="cuda")
    out = torch.full((t, hid), float("nan"), device="cuda")
    op.encodeResident(x, lg, out, sc)
    out2 = torch.empty_like(out)
    op.encodeResident(x, lg, out2, sc)
    assert torch.equal(out, out2), "not deterministic"
    # reference: route with the library's router (pinned against the oracle elsewhere), experts in plain torch
    idx = torch.empty((t, k), dtype=torch.int32, device="cuda")
    wts = torch.empty((t, k), device="cuda")
    q.QWGemmMoE.encodeFnMoeRoute(hal, lg, k, idx, wts)
    assert int((idx < 0).sum()) == 0 and torch.allclose(wts.sum(dim=1), torch.ones(t, device="cuda"), atol=1e-5)
    xr = x.clone()
    q.QWGemm.encodeFwht32(hal, xr)
    ref = torch.zeros((t, hid), device="cuda")
    flat_e = idx.reshape(-1).long()
    flat_t = torch.arange(t, device="cuda").repeat_interleave(k)
    for ex in torch.unique(flat_e).tolist():
        sel = (flat_e == ex).nonzero().squeeze(1)
        rows = flat_t[sel]
        gu = xr[rows].float() @ wgu[ex * 2 * inter:(ex + 1) * 2 * inter].t()
        g, u = gu[:, :inter].half().float(), gu[:, inter:].half().float()
        h = (torch.nn.functional.silu(g) * u).half()
        q.QWGemm.encodeFwht32(hal, h)
        dn = (h.float() @ wdn[ex * hid:(ex + 1) * hid].t()).half().float()
        ref.index_add_(0, rows, dn * wts.reshape(-1)[sel].unsqueeze(1))
    _close(out, ref, 8e-3)
    assert hal.device_status() == 0


def test_decode_moe_under_static_weights_matches_plain_launches(hal):
    # the decode loop's promise (weights never written by in-flight work) lets kernels be launched ahead of their
    # predecessors' end; back-to-back steps with changing routings must give the bits of steps run one at a time
    import qwegn_b200 as q
    t, e, k, hid, inter = 8, 256, 8, 2048, 512
    bgu, _ = _bank(q, hal, e * 2 * inter, hid, "HQ4_G32", seed=17)
    bdn, _ = _bank(q, hal, e * hid, inter, "HQ4_G32", seed=18)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(19)
    x = torch.randn((t, hid), generator=gen, device="cuda").to(torch.float16)
    lgs = [torch.randn((t, e), generator=gen, device="cuda") for _ in range(12)]
    op = q.QWMoEOperator(hal, bgu, bdn, e, inter, k, norm_topk=True)
    sc = torch.empty(op.scratchBytes(t), dtype=torch.uint8, device="cuda")

    def run(sync):
        outs = []
        for lg in lgs:
            o = torch.full((t, hid), float("nan"), device="cuda")
            op.encodeResident(x, lg, o, sc)
            if sync:
                torch.cuda.synchronize()
            outs.append(o)
        torch.cuda.synchronize()
        return outs

    ref = run(True)
    hal.set_static_weights(True)
    try:
        got = run(False)
    finally:
        torch.cuda.synchronize()
        hal.set_static_weights(False)
    for a, b in zip(ref, got):
        assert torch.isfinite(a).all() and torch.equal(a, b)
    assert hal.device_status() == 0
