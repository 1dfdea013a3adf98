"""csw_sparse_compress_static - the entry point for callers that cannot
allocate device memory when they need to compress (allocator locked or
exhausted, callbacks that must not synchronise, fixed memory budgets).  Its
scratch is a fixed array inside the library; this checks, through the C ABI,
that it produces exactly what csw_sparse_compress produces, on two calls in a
row that share that array."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _packed(cs, fn, t, n, out=None, nnz=None):
    """Run one compress entry point; return (tile_off, bitmap, values, nnz) as numpy."""
    import torch
    L = cs.sparse_layout(n)
    if out is None:
        out = torch.zeros(L.bound, dtype=torch.uint8, device="cuda")
        nnz = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    st = fn(t.data_ptr(), n, out.data_ptr(), L.bound, nnz.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    k = int(nnz.item())
    buf = out.cpu().numpy()
    tiles, words = (n + 4095) // 4096, (n + 31) // 32
    return (buf[L.tile_off:L.tile_off + 4 * tiles].copy(), buf[L.bitmap:L.bitmap + 4 * words].copy(),
            buf[L.values:L.values + 4 * k].copy(), k)


def test_static_scratch_entry_point_matches_the_allocating_one():
    import torch
    import cswap_b200 as cs
    lib = cs.lib()
    rng = np.random.default_rng(77)
    # second call is smaller and sparser than the first: stale counters of the
    # first call's extra tiles stay in the shared array and must not matter
    for n, keep in ((3 * 4096 * 37 + 123, 0.5), (4096 * 5 + 7, 0.1)):
        a = (rng.standard_normal(n) * (rng.random(n) < keep)).astype(np.float32)
        a[1] = -0.0
        t = torch.from_numpy(a).cuda()
        want = _packed(cs, lib.csw_sparse_compress, t, n)
        got = _packed(cs, lib.csw_sparse_compress_static, t, n)
        assert got[3] == want[3] == int(np.count_nonzero(a.view(np.uint32)))
        for g, w in zip(got[:3], want[:3]):
            assert np.array_equal(g, w)  # bit for bit
        back = cs.sparse_decompress(_repack(cs, got, n), n)
        assert np.array_equal(back.cpu().numpy().view(np.uint32), a.view(np.uint32))
    out_keep = torch.zeros(cs.sparse_layout(n).bound, dtype=torch.uint8, device="cuda")
    nnz_keep = torch.zeros(1, dtype=torch.int32, device="cuda")
    # a warmed call takes no device memory: the driver's free-memory figure does not move
    free0 = torch.cuda.mem_get_info()[0]
    got = _packed(cs, lib.csw_sparse_compress_static, t, n, out=out_keep, nnz=nnz_keep)
    assert torch.cuda.mem_get_info()[0] == free0
    # n = 0 (the warm-up form) is accepted and leaves a zero count
    z = torch.full((1,), 5, dtype=torch.int32, device="cuda")
    assert lib.csw_sparse_compress_static(None, 0, out_keep.data_ptr(), out_keep.numel(), z.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(z.item()) == 0
    # exactly the limit passes the limit check (capacity 0 then stops it before any launch)
    st = lib.csw_sparse_compress_static(t.data_ptr(), C.c_size_t(268435456), out_keep.data_ptr(), 0, z.data_ptr(), None)
    assert st == 2
    # beyond the fixed array: refused, nothing launched
    big = C.c_size_t(268435456 + 1)
    st = lib.csw_sparse_compress_static(t.data_ptr(), big, t.data_ptr(), 0, t.data_ptr(), None)
    assert st == 8 and b"fixed limit" in lib.csw_status_string(st)


def _repack(cs, parts, n):
    import torch
    L = cs.sparse_layout(n)
    buf = np.zeros(L.bound, dtype=np.uint8)
    buf[L.tile_off:L.tile_off + parts[0].size] = parts[0]
    buf[L.bitmap:L.bitmap + parts[1].size] = parts[1]
    buf[L.values:L.values + parts[2].size] = parts[2]
    return torch.from_numpy(buf).cuda()
