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
