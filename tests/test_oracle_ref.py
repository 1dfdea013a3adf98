"""The CPU oracle against the host build of the reference's own headers,
block by block.  Only runs where that build exists (it needs the reference
tree); elsewhere the committed fixtures of test_oracle_golden.py stand in."""
import ctypes as C

import numpy as np
import pytest


@pytest.fixture(scope="module")
def ref(oracle):
    if not oracle.have_ref():
        pytest.skip("host build of the reference not present")
    return oracle.ref()


def _f32(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _u64(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint64))


def _blocks(rng, size, trial):
    kind = trial % 7
    if kind == 0:
        b = rng.standard_normal(size)
    elif kind == 1:
        b = np.tanh(rng.standard_normal(size))
    elif kind == 2:
        b = np.sin(0.1 * np.arange(size) + trial) * 10.0 ** rng.uniform(-10, 10)
    elif kind == 3:
        b = np.zeros(size)
        b[rng.integers(size)] = rng.standard_normal()
    elif kind == 4:
        b = np.full(size, rng.standard_normal())
    elif kind == 5:
        b = rng.uniform(-1, 1, size) * (rng.random(size) < 0.3)
    else:
        b = np.zeros(size)
    return b.astype(np.float32)


@pytest.mark.parametrize("dims", [1, 2, 3])
@pytest.mark.parametrize("maxbits", [16, 37, 64, 128, 256, 300, 512, 1024])
def test_blocks_match_reference(oracle, ref, dims, maxbits):
    rng = np.random.default_rng(1000 * dims + maxbits)
    size = 1 << (2 * dims)
    asis = 0
    for trial in range(120):
        blk = _blocks(rng, size, trial)
        bidx = int(rng.integers(0, 5))
        s, nmax = oracle.zfp_encode_block(blk, dims, maxbits, bidx)
        r = np.zeros(s.size, dtype=np.uint64)
        ref.ref_bs_encode_block(_f32(blk.copy()), dims, maxbits, bidx, r.ctypes.data, r.size * 8)
        assert np.array_equal(s, r)
        d = oracle.zfp_decode_block(s, dims, maxbits, bidx)
        d2 = np.zeros(size, dtype=np.float32)
        ref.ref_bs_decode_block(r.ctypes.data, r.size * 8, dims, maxbits, bidx, _f32(d2))
        assert np.array_equal(d.view(np.uint32), d2.view(np.uint32))
        if nmax < 64:
            # no full 64-bit plane was written: the reference's block code as
            # written (its own bit writer / reader) is valid on the host too
            a = np.zeros(s.size, dtype=np.uint64)
            ref.ref_asis_encode_block(_f32(blk.copy()), dims, maxbits, bidx, _u64(a))
            assert np.array_equal(a, s)
            d3 = np.zeros(size, dtype=np.float32)
            ref.ref_asis_decode_block(_u64(a), dims, maxbits, bidx, _f32(d3))
            assert np.array_equal(d.view(np.uint32), d3.view(np.uint32))
            asis += 1
    assert asis > 20


def test_tables_and_lifts(oracle, ref):
    L = oracle.lib()
    p, q = L.orc_perm3(), ref.ref_perm3()
    assert [p[i] for i in range(64)] == [q[i] for i in range(64)]
    rng = np.random.default_rng(3)
    for stride in (1, 4, 16):
        for _ in range(200):
            v = rng.integers(-2 ** 30, 2 ** 30, 64).astype(np.int32)
            a, b = v.copy(), v.copy()
            L.orc_fwd_lift(a.ctypes.data_as(C.POINTER(C.c_int32)), stride)
            ref.ref_fwd_lift(b.ctypes.data_as(C.POINTER(C.c_int32)), stride)
            assert np.array_equal(a, b)
            L.orc_inv_lift(a.ctypes.data_as(C.POINTER(C.c_int32)), stride)
            ref.ref_inv_lift(b.ctypes.data_as(C.POINTER(C.c_int32)), stride)
            assert np.array_equal(a, b)


@pytest.mark.parametrize("n,P", [(1000, 16384), (4194304, 16384), (16384 * 32 + 5, 16384), (12345, 8192)])
def test_sparse_reference_kernels(oracle, ref, n, P):
    rng = np.random.default_rng(n)
    a = (rng.standard_normal(n) * (rng.random(n) < 0.4)).astype(np.float32)
    a[rng.integers(n)] = -0.0
    b, bm, v, nnz = oracle.legacy_sparse_compress(a, P)
    rb = np.zeros(P, dtype=np.int32)
    rbm = np.zeros(bm.size, dtype=np.uint32)
    rv = np.zeros(n, dtype=np.float32)
    rn = ref.ref_sparse_compress(_f32(a.copy()), n, P // 32, 32, rb.ctypes.data_as(C.POINTER(C.c_int32)),
                                 rbm.ctypes.data_as(C.POINTER(C.c_uint32)), _f32(rv))
    _, _, _, active = oracle.legacy_sizes(n, P)
    assert rn == nnz
    assert np.array_equal(rb[:active], b[:active]) and np.array_equal(rbm, bm)
    assert np.array_equal(rv[:nnz].view(np.uint32), v.view(np.uint32))
    out = oracle.legacy_sparse_decompress(v, n, P, bm, b, prefill=7.0)
    ro = np.full(n, 7.0, dtype=np.float32)
    ref.ref_sparse_decompress(_f32(rv), _f32(ro), n, P // 32, 32, rbm.ctypes.data_as(C.POINTER(C.c_uint32)),
                              rb.ctypes.data_as(C.POINTER(C.c_int32)))
    assert np.array_equal(out.view(np.uint32), ro.view(np.uint32))
