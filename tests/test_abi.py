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
    text = re.sub(r"^\s*typedef[^;{]*\([^;]*;", "", text, flags=re.M)  # function-pointer typedefs declare no symbol
    names = re.findall(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b(\w+)\s*\([^;{]*\)\s*;", text, flags=re.M)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_every_declared_symbol_is_exported_and_bound(L):
    from cswap_b200._lib import CXX_SIGNATURES, SIGNATURES
    declared = _declared("cswap_b200.h") + _declared("cswap_compat.h")
    assert len(declared) >= 41
    for name in declared:
        if name in CXX_SIGNATURES:  # C++ linkage: exported under its mangled name
            assert hasattr(L, CXX_SIGNATURES[name][0]), f"{name} is declared in include/ but not exported"
            continue
        assert hasattr(L, name), f"{name} is declared in include/ but not exported"
        assert name in SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(list(SIGNATURES) + list(CXX_SIGNATURES)) == sorted(set(declared))


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
    n = 8 << 20  # 32 MiB tensors: 0.67 ms each on the link, far more than the 1 ms forward pass can hide
    fwd = 1e-3
    tensors = [
        cs.TensorDesc(n, 0.9, False, ready_s=1e-4, need_s=1.8e-3),    # very sparse, lossless only
        cs.TensorDesc(n, 0.0, True, ready_s=3e-4, need_s=1.4e-3),     # dense, loss allowed
        cs.TensorDesc(n, 0.0, False, ready_s=5e-4, need_s=1.0e-3),    # dense, lossless: nothing applies
        cs.TensorDesc(n, -1.0, False, ready_s=7e-4, need_s=0.6e-3),   # sparsity unknown, lossless
        cs.TensorDesc(n + 8, 0.0, True, ready_s=9e-4, need_s=0.2e-3),  # not a multiple of 1024: ZFP + raw tail
        cs.TensorDesc(1000, 0.0, True, ready_s=9.5e-4, need_s=0.1e-3),  # less than one 32x32 slab: no ZFP
    ]
    pol, stall = cm.decide(tensors, fwd)
    assert pol == [3, 6, 2, 2, 6, 2]
    all_raw = [cs.TensorDesc(t.numel, -1.0, False, t.ready_s, t.need_s) for t in tensors]
    pol_raw, stall_raw = cm.decide(all_raw, fwd)
    assert pol_raw == [2] * 6 and sum(stall) < 0.75 * sum(stall_raw)
    # when the link keeps up with compute nothing stalls either way, and the tie goes to the smaller
    # payload (it leaves the link and the copy engine's queue to others): sparse at 90 % zeros, ZFP
    # where only loss helps, raw where nothing may be coded
    small = [cs.TensorDesc(1 << 18, 0.9, True, ready_s=1e-4 * i, need_s=1e-3 * (5 - i)) for i in range(5)]
    pol2, stall2 = cm.decide(small, 1e-3)
    assert pol2 == [3] * 5 and sum(stall2) == 0.0
    dense = [cs.TensorDesc(1 << 18, 0.0, i % 2 == 0, ready_s=1e-4 * i, need_s=1e-3 * (5 - i)) for i in range(5)]
    pol3, stall3 = cm.decide(dense, 1e-3)
    assert pol3 == [6, 2, 6, 2, 6] and sum(stall3) == 0.0
    assert cm.decide([], 0.0) == ([], [])
    # the prediction for a given table: keeping everything costs nothing, and raw tensors that backward
    # wants before they have left are taken back (which is why all-raw can be predicted cheaper than a
    # table with codecs in it: it frees no memory for those tensors either)
    total_keep, _ = cm.simulate(tensors, [0] * 6, fwd)
    total_dec, per = cm.simulate(tensors, pol, fwd)
    total_raw, per_raw = cm.simulate(tensors, [2] * 6, fwd)
    assert total_keep == 0.0 and total_dec > 0.0 and total_raw > 0.0 and len(per) == 6
    # six 32 MiB copies queue on a 50 GB/s link: the last ones are still on their way out when backward
    # (1 ms after the forward pass began) asks for them, so they stall nothing
    assert per_raw[4] == 0.0 and per_raw[3] == 0.0 and per_raw[0] > 0.0
    # the sparse slopes fitted at 75 % / 90 % zeros are used for a tensor that sparse: with a codec that is
    # hopeless there (but fine at 50 %) the 90 %-zero tensor stays raw
    cm2 = cs.CostModel(**cm.as_dict())
    cm2.c.sparse_enc_b75, cm2.c.sparse_enc_b90, cm2.c.sparse_dec_b75, cm2.c.sparse_dec_b90 = 2e-13, 1e-9, 1.5e-13, 1e-9
    assert cm2.decide(tensors, fwd)[0][0] == 2
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


def test_blob_header_validation_without_a_device(L):
    """csw_blob_info is host logic: sizes, policy, and for sparse payloads the
    consistency of tile offsets with the bitmap."""
    import ctypes as C
    import struct
    import numpy as np
    import cswap_b200 as cs
    from cswap_b200._lib import SparseLayout

    def blob(policy, numel, payload, maxbits=0, nnz=0, magic=0x50575343, version=1):
        return np.frombuffer(struct.pack("<IIIIQQQ3Q", magic, version, policy, maxbits, numel, len(payload), nnz,
                                         0, 0, 0) + bytes(payload), dtype=np.uint8)

    raw = blob(2, 8, bytes(32))
    assert cs.blob_info(raw) == {"policy": 2, "numel": 8, "zfp_maxbits": 0, "payload_bytes": 32, "nnz": 0,
                                 "version": 1}
    for bad in (blob(2, 8, bytes(28)), blob(2, 8, bytes(32), magic=1), blob(2, 8, bytes(32), version=2),
                blob(5, 8, bytes(32)), blob(2, 0, b""), blob(2, 8, bytes(32), nnz=1)):
        with pytest.raises(cs.CswapError):
            cs.blob_info(bad)
    with pytest.raises(cs.CswapError):
        cs.blob_info(raw[:40])                               # shorter than the header
    with pytest.raises(cs.CswapError):
        cs.blob_info(raw[:-1])                               # payload cut short
    # zfp: 4096 values = 32x32x4 = 64 blocks of 512 bits
    assert cs.blob_info(blob(6, 4096, bytes(4096), maxbits=512))["zfp_maxbits"] == 512
    assert cs.blob_info(blob(6, 4096 + 5, bytes(4096 + 20), maxbits=512))["numel"] == 4101  # stream + raw tail
    with pytest.raises(cs.CswapError):
        cs.blob_info(blob(6, 4096 + 5, bytes(4096), maxbits=512))  # the tail is missing
    with pytest.raises(cs.CswapError):
        cs.blob_info(blob(6, 1000, bytes(4000), maxbits=512))      # less than one slab never travels as ZFP
    with pytest.raises(cs.CswapError):
        cs.blob_info(blob(6, 4096, bytes(2048), maxbits=512))
    # sparse: 5000 elements, two tiles, non-zeros at 3, 40 and 4100
    n = 5000
    lay = SparseLayout()
    assert L.csw_sparse_layout_of(n, C.byref(lay)) == 0
    def sparse(tile_off, nnz):
        p = bytearray(lay.values + 4 * nnz)
        p[lay.tile_off:lay.tile_off + 8] = struct.pack("<II", *tile_off)
        words = np.zeros((n + 31) // 32, dtype=np.uint32)
        for i in (3, 40, 4100):
            words[i // 32] |= np.uint32(1 << (i % 32))
        p[lay.bitmap:lay.bitmap + 4 * words.size] = words.tobytes()
        return blob(3, n, p, nnz=nnz)
    assert cs.blob_info(sparse((0, 2), 3))["nnz"] == 3
    assert cs.blob_info(sparse((1, 0), 3))["nnz"] == 3       # segments in schedule order are fine
    for bad in (sparse((0, 3), 3), sparse((2, 0), 3), sparse((0, 2), 4), sparse((0, 2), 2)):
        with pytest.raises(cs.CswapError):
            cs.blob_info(bad)
