"""QWP1 reader against the reference's committed selfpack fixture (tests/golden/selfpack.qwp is byte-identical to
Tests/QWQuantTests/fixtures/selfpack.qwp; see tests/golden/gen_golden.py)."""
import os

import numpy as np
import pytest

from conftest import GOLDEN


def test_selfpack_index_and_planes(oracle, golden):
    from qwegn_b200.pack import Pack
    p = Pack(os.path.join(GOLDEN, "selfpack.qwp"))
    assert set(p.entries) == {"w_test", "norm_test"}
    e = p.entries["w_test"]
    assert e.shape == (256, 1024) and e.kind == "blocks" and e.container.block_bytes == 20
    assert e.offset % 16384 == 0            # Q4G_ALIGNMENT (Scripts/quantize/pack.py:25)
    g = golden["ref_fixtures"]
    assert np.array_equal(p.plane("w_test"), g["selfpack_blocks"].reshape(-1))
    # QWQuantTests.swift:69-85: decoding the pack's plane gives the numpy golden bit for bit
    dq = oracle.dequant(np.array(p.plane("w_test")).reshape(256, 32, 20), oracle.HQ4_G32, standard=True)
    assert np.array_equal(dq.view(np.uint32), g["selfpack_dq4"].view(np.uint32))
    assert np.array_equal(p.raw_f32("norm_test").reshape(-1), g["selfpack_raw_norm"].reshape(-1))
    p.close()


def test_rejects_a_file_that_is_not_a_pack(tmp_path):
    import qwegn_b200 as q
    from qwegn_b200.pack import Pack
    f = tmp_path / "x.qwp"
    f.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(q.QWGemmError):
        Pack(str(f))


@pytest.mark.gpu
def test_load_uploads_the_plane_verbatim(hal, golden):
    import torch
    import qwegn_b200 as q
    from qwegn_b200.pack import Pack
    p = Pack(os.path.join(GOLDEN, "selfpack.qwp"))
    view = p.load(hal, "w_test")
    assert (view.n, view.k) == (256, 1024)
    assert np.array_equal(view.bank.cpu().numpy(), golden["ref_fixtures"]["selfpack_blocks"].reshape(-1))
    out = torch.empty((256, 1024), dtype=torch.float32, device="cuda")
    q.QWGemm.dequant(hal, view, out, standard_domain=True)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), golden["ref_fixtures"]["selfpack_dq4"].view(np.uint32))
    p.close()


_MOEPACK_LAYERS = {"l0": ("HQ4_G32", 4, 128, 128), "l1": ("HQ8_G32", 4, 128, 128), "l2": ("HQ4_G64", 2, 256, 256)}


def _moepack():
    from qwegn_b200.pack import Pack
    return Pack(os.path.join(GOLDEN, "moepack.qwp")), np.load(os.path.join(GOLDEN, "moepack.npz"))


def test_expert_stacks_and_rotated_containers_in_a_pack(oracle):
    # A pack written by the reference's pack_file (Scripts/quantize/pack.py:214-268): 3-D "….experts.…" stacks become one plane
    # of E slabs of e_hq4 bytes each; an "hq" entry names the rotated container (QWQuantTypes.swift:69-149).
    p, g = _moepack()
    for layer, (name, experts, hidden, inter) in _MOEPACK_LAYERS.items():
        fmt = oracle.FORMATS[name]
        for proj, key, rows, k in (("gate_up_proj", "gate_up", 2 * inter, hidden), ("down_proj", "down", hidden, inter)):
            e = p.entries[f"{layer}.mlp.experts.{proj}"]
            assert e.shape == (experts, rows, k) and e.experts == experts and e.kind == "blocks"
            assert (e.container.bits, e.container.group) == (fmt.bits, fmt.group)
            assert e.expert_bytes == rows * fmt.row_bytes(k) and e.nbytes == experts * e.expert_bytes
            assert e.offset % 16384 == 0
            w = g[f"{layer}_{key}"].astype(np.float32).reshape(experts * rows, k)
            blocks = oracle.quantize(w, fmt)
            assert np.array_equal(p.plane(e.name), blocks.reshape(-1)), "the oracle's blocks differ from the reference's plane"
            slab = np.array(p.plane(e.name)[e.expert_bytes:2 * e.expert_bytes]).reshape(rows, k // fmt.group, -1)
            dq = oracle.dequant(slab, fmt, standard=True)
            want = g[f"{layer}_{proj}_e1_dq"]
            assert np.array_equal(dq[:16].view(np.uint32), want.view(np.uint32))
    for name, key, fmt in (("l0.attn.q_proj.weight", "q_proj", oracle.HQ8_G32), ("l0.attn.o_proj.weight", "o_proj", oracle.HQ4_G64)):
        e = p.entries[name]
        assert e.experts == 0 and (e.container.bits, e.container.group) == (fmt.bits, fmt.group)
        assert np.array_equal(p.plane(name), oracle.quantize(g[key].astype(np.float32), fmt).reshape(-1))
    p.close()


@pytest.mark.gpu
@pytest.mark.parametrize("layer", sorted(_MOEPACK_LAYERS))
def test_expert_stack_from_a_pack_through_the_moe_operator(hal, oracle, layer):
    # Pack.load -> QWMoEOperator -> oracle: the expert stack is used as it lies in the file (expert e at row e * N)
    import torch
    import qwegn_b200 as q
    from conftest import assert_matmul_close
    name, experts, hidden, inter = _MOEPACK_LAYERS[layer]
    p, g = _moepack()
    bank_gu = p.load(hal, f"{layer}.mlp.experts.gate_up_proj")
    bank_dn = p.load(hal, f"{layer}.mlp.experts.down_proj")
    assert (bank_gu.n, bank_gu.k, bank_dn.n, bank_dn.k) == (experts * 2 * inter, hidden, experts * hidden, inter)
    topk = 2 if experts > 2 else 1
    x, lg = g[f"{layer}_x"], g[f"{layer}_logits"]
    op = q.QWMoEOperator(hal, bank_gu, bank_dn, experts, inter, topk, norm_topk=True)
    scratch = torch.empty(op.scratchBytes(x.shape[0]), dtype=torch.uint8, device="cuda")
    out = torch.full((x.shape[0], hidden), float("nan"), dtype=torch.float32, device="cuda")
    op.encodeResident(torch.from_numpy(x).cuda(), torch.from_numpy(lg).cuda(), out, scratch)
    ridx, rwts = oracle.moe_route(lg, topk, norm_topk=True)
    ref = oracle.moe_forward(np.array(p.plane(f"{layer}.mlp.experts.gate_up_proj")), np.array(p.plane(f"{layer}.mlp.experts.down_proj")),
                             oracle.FORMATS[name], experts, hidden, inter, x, ridx, rwts)
    assert_matmul_close(out.cpu().numpy(), ref, tight=6e-3)
    p.close()
