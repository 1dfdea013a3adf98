"""Overrun detection for every codec output (the stand-in for a memory checker):
each output buffer sits between two 4 KiB guard areas holding a fixed pattern;
after the call both guards must be untouched and the bytes between them must
be the expected ones.  Covers the slab and the generic ZFP kernels (streams and
tensors, partial slabs, ragged shapes, unaligned bit budgets) and the sparse
packed buffer, its count word and its scatter-back."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu

GUARD = 4096
PATTERN = 0xA5


@pytest.fixture(scope="module")
def cs():
    import torch
    import cswap_b200
    assert torch.cuda.is_available()
    cswap_b200.lib()
    return cswap_b200


class Guarded:
    """`nbytes` of device memory with a guard on either side."""

    def __init__(self, nbytes, fill=0xEE):
        import torch
        self.nbytes = nbytes
        self.buf = torch.full((nbytes + 2 * GUARD,), PATTERN, dtype=torch.uint8, device="cuda")
        self.buf[GUARD:GUARD + nbytes] = fill
        self.ptr = self.buf.data_ptr() + GUARD

    def body(self):
        return self.buf[GUARD:GUARD + self.nbytes]

    def check(self, what):
        import torch
        torch.cuda.synchronize()
        lo = self.buf[:GUARD]
        hi = self.buf[GUARD + self.nbytes:]
        assert bool((lo == PATTERN).all()), f"{what}: wrote below the buffer"
        assert bool((hi == PATTERN).all()), f"{what}: wrote past the buffer (first at +{int((hi != PATTERN).nonzero()[0])})"


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


ZFP_CASES = [
    # dims, maxbits
    ((32, 32, 1), 512), ((32, 32, 5), 512), ((32, 32, 8), 256), ((32, 32, 9), 1024), ((32, 32, 17), 512),
    ((32, 32, 67), 64), ((32, 32, 31), 2048), ((32, 32, 12), 96),           # slab kernels, partial groups
    ((5, 5, 5), 512), ((31, 33, 6), 300), ((9, 7, 3), 37), ((64, 16, 9), 512),  # generic 3-D
    ((13, 10, 0), 256), ((4, 4, 0), 37), ((37, 0, 0), 64), ((13, 0, 0), 96), ((1, 0, 0), 300),
]


@pytest.mark.parametrize("dims,maxbits", ZFP_CASES)
def test_zfp_stream_and_tensor_stay_inside(cs, oracle, dims, maxbits):
    import torch
    nx, ny, nz = dims
    n = nx * max(ny, 1) * max(nz, 1)
    a = util.normal(n, seed=n + maxbits)
    t = torch.from_numpy(a).cuda()
    L = cs.lib()
    need = cs.zfp_max_bytes(nx, ny, nz, maxbits)
    out = Guarded(need)
    assert L.csw_zfp_compress(t.data_ptr(), nx, ny, nz, maxbits, out.ptr, need, None, _stream()) == 0
    out.check("zfp compress")
    ref = oracle.zfp_encode(a, nx, ny, nz, maxbits)
    assert np.array_equal(out.body().cpu().numpy().view(np.uint64), ref)   # every byte between the guards written
    back = Guarded(4 * n)
    assert L.csw_zfp_decompress(out.ptr, need, nx, ny, nz, maxbits, back.ptr, _stream()) == 0
    back.check("zfp decompress")
    ref_back = oracle.zfp_decode(ref, nx, ny, nz, maxbits)
    assert np.array_equal(back.body().cpu().numpy().view(np.uint32), ref_back.view(np.uint32))


@pytest.mark.parametrize("n", [1, 31, 33, 4095, 4096, 4097, 100003, 1 << 20])
@pytest.mark.parametrize("entry", ["csw_sparse_compress", "csw_sparse_compress_onepass"])
def test_sparse_packed_buffer_stays_inside(cs, n, entry):
    import torch
    a = util.relu_normal(n, 0.5, seed=n)
    t = torch.from_numpy(a).cuda()
    L = cs.lib()
    lay = cs.sparse_layout(n)
    nnz_true = int(np.count_nonzero(a.view(np.uint32)))
    packed = Guarded(lay.bound)
    count = Guarded(4, fill=0)
    assert getattr(L, entry)(t.data_ptr(), n, packed.ptr, lay.bound, count.ptr, _stream()) == 0
    packed.check(entry)
    count.check(entry + " count word")
    assert int(count.body().view(torch.int32)[0]) == nnz_true
    # nothing is written past the bytes that have to move
    moved = cs.sparse_packed_bytes(n, nnz_true)
    tail = packed.body()[moved:]
    assert bool((tail == 0xEE).all()), "bytes past header + bitmap + nnz values were written"
    back = Guarded(4 * n)
    assert L.csw_sparse_decompress(packed.ptr, n, back.ptr, _stream()) == 0
    back.check("sparse decompress")
    assert np.array_equal(back.body().cpu().numpy().view(np.uint32), a.view(np.uint32))


@pytest.mark.parametrize("n", [5000, 70001, 1 << 20])
def test_reference_layout_sparse_stays_inside(cs, n):
    """PreGPUcompression / PreAcc / GPUcompression / GPUdecompression: the four
    caller-sized buffers of CSWAP+/Execution.h:88-99."""
    import math
    import torch
    a = util.relu_normal(n, 0.75, seed=n)
    t = torch.from_numpy(a).cuda()
    L = cs.lib()
    dimsize, blocksize = 512, 32
    P = dimsize * blocksize
    chunk = -(-n // P)
    begin = Guarded(4 * P, fill=0)
    num = Guarded(4, fill=0)
    bitmap = Guarded(4 * P * (-(-chunk // 32)), fill=0)
    nnz_true = int(np.count_nonzero(a))
    values = Guarded(4 * max(nnz_true, 1))
    s = _stream()
    L.PreGPUcompression(n, P, t.data_ptr(), begin.ptr, dimsize, blocksize, s)
    active = int(math.ceil(float(n) / math.ceil(float(n) / P)))
    L.PreAcc(begin.ptr, active, num.ptr, 1, 1, s)
    begin.check("PreGPUcompression/PreAcc")
    num.check("PreAcc")
    assert int(num.body().view(torch.int32)[0]) == nnz_true
    L.GPUcompression(n, P, t.data_ptr(), values.ptr, begin.ptr, bitmap.ptr, dimsize, blocksize, s)
    values.check("GPUcompression values")
    bitmap.check("GPUcompression bitmap")
    begin.check("GPUcompression begin")
    out = Guarded(4 * n, fill=0)
    torch.cuda.synchronize()
    L.GPUdecompression(values.ptr, out.ptr, n, P, bitmap.ptr, begin.ptr, dimsize, blocksize)
    out.check("GPUdecompression")
    assert np.array_equal(out.body().cpu().numpy().view(np.float32), a)
