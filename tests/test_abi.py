"""The C ABI without a GPU: the library loads, exports every symbol the headers
declare, and the entry points that need no device behave."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from cswap_b200 import build
    build.build()
    import cswap_b200
    return cswap_b200.lib()


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b(\w+)\s*\([^;{]*\)\s*;", text, flags=re.M)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_every_declared_symbol_is_exported_and_bound(L):
    from cswap_b200._lib import SIGNATURES
    declared = _declared("cswap_b200.h") + _declared("cswap_compat.h")
    assert len(declared) >= 37
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in include/ but not exported"
        assert name in SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(SIGNATURES) == sorted(set(declared))


def test_sizing_and_layout_without_a_device(L):
    from cswap_b200._lib import SparseLayout
    b = C.c_size_t()
    assert L.csw_zfp_max_bytes(32, 32, 8192, 512, C.byref(b)) == 0 and b.value == 8 * 1024 * 1024
    assert L.csw_zfp_max_bytes(5, 5, 5, 300, C.byref(b)) == 0 and b.value == (8 * 300 + 63) // 64 * 8
    assert L.csw_zfp_max_bytes(32, 32, 4, 8, C.byref(b)) == 1       # header does not fit
    assert L.csw_zfp_max_bytes(0, 0, 0, 512, C.byref(b)) == 1
    nx, ny, nz = C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert L.csw_zfp_view(1 << 20, C.byref(nx), C.byref(ny), C.byref(nz)) == 0
    assert (nx.value, ny.value, nz.value) == (32, 32, 1024)
    assert L.csw_zfp_view(1000, C.byref(nx), C.byref(ny), C.byref(nz)) == 7
    lay = SparseLayout()
    assert L.csw_sparse_layout_of(4194304, C.byref(lay)) == 0
    assert lay.tile_off == 0 and lay.bitmap == 4096 and lay.values == 4096 + 524288
    assert lay.bound == lay.values + 4 * 4194304
    assert L.csw_status_string(2) == b"output capacity too small"
    assert L.csw_version().count(b".") == 2


def test_cost_decision_is_pure_host_logic(L):
    import cswap_b200 as cs
    cm = cs.CostModel(zfp_enc_b=2.5e-13, zfp_dec_b=2.5e-13, sparse_enc_b=2e-13, sparse_dec_b=1.5e-13,
                      zfp_enc_a=5e-6, zfp_dec_a=5e-6, sparse_enc_a=8e-6, sparse_dec_a=4e-6,
                      d2h_a=1e-5, d2h_bps=50e9, h2d_a=1e-5, h2d_bps=50e9, zfp_maxbits=512)
    n = 8 << 20
    pol, exposed = cm.decide([
        cs.TensorDesc(n, 0.9, False, 0.0, 0.0),
        cs.TensorDesc(n, 0.0, True, 0.0, 0.0),
        cs.TensorDesc(n, 0.0, False, 0.0, 0.0),
        cs.TensorDesc(n, 0.9, True, 1.0, 1.0),
        cs.TensorDesc(1000, 0.0, True, 0.0, 0.0),
        cs.TensorDesc(n, -1.0, False, 0.0, 0.0),
    ])
    assert pol == [3, 6, 2, 2, 2, 2]
    assert exposed[1] < exposed[2] and exposed[3] == 0.0
    # a backlog on the link makes compression worth it even inside a window
    pol2, _ = cm.decide([cs.TensorDesc(64 << 20, 0.0, False, 1e-4, 1e-4), cs.TensorDesc(n, 0.0, True, 1e-3, 1e-3)])
    assert pol2 == [2, 6]
    with pytest.raises(cs.CswapError):
        cs.CostModel().decide([cs.TensorDesc(n)])  # no link bandwidth fitted


def test_codec_refuses_cpu_tensors():
    import torch
    import cswap_b200 as cs
    with pytest.raises(ValueError):
        cs.zfp_compress(torch.zeros(1024), 512)
    with pytest.raises(ValueError):
        cs.sparse_compress(torch.zeros(1024))


def test_missing_library_fails_loudly(monkeypatch):
    import cswap_b200._lib as lib
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", "/nonexistent/libcswap_b200.so")
    with pytest.raises(lib.LibraryMissing):
        lib.lib()
