"""The C-ABI boundary without a GPU: the library loads, exports every symbol include/qwc.h declares, and the pure
host functions (dispatch table, weight-view validation) behave like the reference's (QWGemm.swift:92-133,
QWWeightView.swift:108-152)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    ge.build()
    from qwegn_b200 import _lib
    return _lib.load()


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(qwc_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 12
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_binding_covers_the_header(lib):
    from qwegn_b200 import _lib
    import qwegn_b200.moe  # noqa: F401  (registers the MoE entry points)
    import qwegn_b200.parallel  # noqa: F401  (registers the fused all-reduce and the expert-parallel entry points)
    assert set(_declared_symbols()) <= set(_lib.SIGNATURES), sorted(set(_declared_symbols()) - set(_lib.SIGNATURES))


def test_block_bytes(lib):
    assert lib.qwc_block_bytes(0, 4, 32) == 20
    assert lib.qwc_block_bytes(1, 8, 32) == 36
    assert lib.qwc_block_bytes(1, 4, 64) == 36
    assert lib.qwc_block_bytes(1, 2, 256) == 68


def test_plan_families_and_backends():
    import qwegn_b200 as q
    p = q.QWGemm.plan(1, 12288, 4096)
    assert (p.family, p.backend) == (1, 1) and "hq4g32m5" in p.kernel
    assert q.QWGemm.plan(1, 248320, 5120, vocab=248320).family == 2
    assert q.QWGemm.plan(3, 1024, 5120).family == 5
    assert q.QWGemm.plan(16, 17408, 5120, q.rotatedHQ(8, 32)).family == 4
    p = q.QWGemm.plan(4096, 34816, 5120)
    assert p.family == 3 and p.backend in (1, 2)
    # K not a multiple of 128: rows are not 16-byte aligned, the bulk-copy kernels cannot take them
    assert q.QWGemm.plan(1, 64, 96).backend == 3
    # a container of the family without a kernel here is blocked, not an error (QWGemm.swift:128-131)
    assert q.QWGemm.plan(1, 64, 256, q.rotatedHQ(3, 128)).backend == 0
    with pytest.raises(q.QWGemmError) as e:
        q.QWGemm.plan(0, 64, 256)
    assert e.value.case == "badShape"


def test_weight_view_refusals(lib):
    from qwegn_b200._lib import WeightViewC
    v = WeightViewC()
    fake = ctypes.c_void_p(0x10000)
    assert lib.qwc_weight_view_init(ctypes.byref(v), fake, 20 * 8, 4, 64, 0, 0, 0) == 0
    assert (v.n, v.k, v.bits, v.group) == (4, 64, 4, 32)
    # k % group != 0
    assert lib.qwc_weight_view_init(ctypes.byref(v), fake, 1 << 20, 4, 48, 0, 4, 32) == 2
    assert b"multiple of group" in lib.qwc_last_error()
    # bank too short
    assert lib.qwc_weight_view_init(ctypes.byref(v), fake, 20 * 8 - 1, 4, 64, 0, 4, 32) == 2
    # unknown kind / bits
    assert lib.qwc_weight_view_init(ctypes.byref(v), fake, 1 << 20, 4, 64, 7, 4, 32) == 2
    assert lib.qwc_weight_view_init(ctypes.byref(v), fake, 1 << 20, 4, 64, 1, 5, 32) == 2
    # HQ4_G64 needs k % 64
    assert lib.qwc_weight_view_init(ctypes.byref(v), fake, 1 << 20, 4, 96, 1, 4, 64) == 2
    assert lib.qwc_weight_view_init(ctypes.byref(v), fake, 1 << 20, 4, 128, 1, 4, 64) == 0
    # misaligned
    assert lib.qwc_weight_view_init(ctypes.byref(v), ctypes.c_void_p(0x10002), 1 << 20, 4, 64, 0, 4, 32) == 2


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "qwegn_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                for needle in ("import oracle", "from oracle", "qw_oracle", "libqworacle", "oracle/"):
                    assert needle not in text, f"{f} reaches into the oracle ({needle})"


class _FakeHal:
    """Stands in for QWHal where no GPU exists: the tensor checks only need the device the context lives on."""
    def __init__(self):
        import torch
        self.device = torch.device("cuda", 0)


class _FakeView:
    def __init__(self, n, k):
        import torch
        self.n, self.k = n, k
        self.bank = type("B", (), {"device": torch.device("cuda", 0)})()


def test_matmul_doors_refuse_bad_tensors_before_any_call():
    # The C side sees raw pointers and strides only, so a CPU tensor, a short y or overlapping rows must be refused
    # by the Python doors before the C ABI is reached (QWGemm.encode, the scratch-free door and the MoE doors share
    # these checks).  No GPU is needed to see the refusals: they come before any launch.
    import torch
    import qwegn_b200 as q
    from qwegn_b200.gemm import check_device_tensor, check_matmul_tensors
    from qwegn_b200 import noalloc
    hal, w = _FakeHal(), _FakeView(64, 128)
    x = torch.zeros((2, 128), dtype=torch.float16)
    y = torch.zeros((2, 64), dtype=torch.float32)
    for fn in (lambda: check_matmul_tensors(hal, w, x, y, 0),                      # CPU tensors
               lambda: q.QWGemm.encode(hal, w, x, y),
               lambda: noalloc.encode_static_scratch(hal, w, x, y)):
        with pytest.raises(q.QWGemmError) as e:
            fn()
        assert e.value.case == "badShape"
    with pytest.raises(q.QWGemmError):
        check_device_tensor(hal, x, "x", torch.float16)
    # shape logic (independent of the device check): reproduce it on meta tensors that claim to be on the GPU
    xm = torch.empty((2, 128), dtype=torch.float16, device="meta")
    assert not xm.is_cuda   # meta tensors are refused like CPU tensors
    with pytest.raises(q.QWGemmError):
        check_matmul_tensors(hal, w, xm, torch.empty((2, 64), dtype=torch.float32, device="meta"), 0)
