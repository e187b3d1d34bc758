import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import qw_oracle
    qw_oracle.build()
    return qw_oracle


@pytest.fixture(scope="session")
def golden():
    return {name: np.load(os.path.join(GOLDEN, name + ".npz")) for name in ("ref_fixtures", "formats", "matmul")}


@pytest.fixture(scope="session")
def hal():
    import qwegn_b200 as q
    h = q.QWHal(0)
    yield h
    assert h.device_status() == 0, "a kernel reported a bounded wait that gave up"
    h.close()


# The stated output tolerance of the path: max relative error <= 1e-2 (relative to the largest reference
# magnitude) and cosine similarity >= 0.9999.  `tight` additionally bounds the error by what f32 accumulation of
# f16-rounded operands can produce, so that an indexing bug cannot hide inside the loose gate.
def assert_matmul_close(y, yref, tight=2e-3):
    y = np.asarray(y, dtype=np.float64)
    yref = np.asarray(yref, dtype=np.float64)
    assert y.shape == yref.shape
    assert np.isfinite(y).all()
    scale = np.abs(yref).max() + 1e-30
    err = np.abs(y - yref).max() / scale
    cos = float((y * yref).sum() / (np.linalg.norm(y) * np.linalg.norm(yref) + 1e-30))
    assert err <= 1e-2, f"max relative error {err:.3e} > 1e-2"
    assert cos >= 0.9999, f"cosine {cos:.6f} < 0.9999"
    assert err <= tight, f"max relative error {err:.3e} > tight bound {tight:.1e}"
