"""The product's codecs against the reference's own CUDA kernels on the same GPU.

oracle/_ref/libcswap_ref_cuda.so is the reference's cuZFP.cu / compression.cu
compiled for sm_100a where the reference tree is mounted (oracle/build_ref_cuda.sh);
the built library travels with the repository.  Streams, decoded arrays and the
reference sparse layout must agree bit for bit.  Skipped where that library
has not been built."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu

SLACK = 4096  # the reference's block reader loads one word past the last block (decode.cuh:80-84)


@pytest.fixture(scope="module")
def env():
    import torch
    import cswap_b200
    from oracle import oracle as O
    if not O.have_ref_cuda():
        pytest.skip("reference CUDA build not present (oracle/build_ref_cuda.sh)")
    assert torch.cuda.is_available()
    cswap_b200.lib()
    return cswap_b200, O, O.ref_cuda()


def ref_compress(R, t, dims, maxbits, nbytes):
    import torch
    nx, ny, nz = dims
    buf = torch.zeros(nbytes + SLACK, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    got = R.refcuda_zfp_compress(t.data_ptr(), nx, ny, nz, maxbits, buf.data_ptr(), buf.numel())
    torch.cuda.synchronize()
    return buf, int(got)


def ref_decompress(R, buf, dims, maxbits, n):
    import torch
    nx, ny, nz = dims
    out = torch.full((n,), 7.0, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    R.refcuda_zfp_decompress(buf.data_ptr(), buf.numel(), nx, ny, nz, maxbits, out.data_ptr())
    torch.cuda.synchronize()
    return out


def both(env, a, dims, maxbits):
    import torch
    cs, O, R = env
    t = torch.from_numpy(a).cuda()
    mine = cs.zfp_compress(t, maxbits, dims)
    nbytes = mine.numel()
    buf, _ = ref_compress(R, t, dims, maxbits, nbytes)
    # the reference sizes 3-D streams by truncation (shared.h:73-84) but its blocks
    # add into every word they touch of the zeroed buffer: compare all of it
    got = mine.cpu().numpy()
    ref = buf.cpu().numpy()[:nbytes]
    assert np.array_equal(got, ref), f"stream differs at byte {np.flatnonzero(got != ref)[:4]}"
    back = cs.zfp_decompress(mine, a.size, maxbits, dims)
    ref_back = ref_decompress(R, buf, dims, maxbits, a.size)
    assert torch.equal(back.view(torch.int32), ref_back.view(torch.int32))
    # and across: the reference decodes the product's stream
    padded = torch.zeros(nbytes + SLACK, dtype=torch.uint8, device="cuda")
    padded[:nbytes] = mine
    cross = ref_decompress(R, padded, dims, maxbits, a.size)
    assert torch.equal(back.view(torch.int32), cross.view(torch.int32))


@pytest.mark.parametrize("maxbits", [64, 512, 1024])
def test_decode_arbitrary_streams(env, maxbits):
    """Streams no encoder wrote: the reference's decoder and the product's must
    still agree on every bit (the reference's loops are bounded by the bit
    budget whatever the content, decode.cuh:141-173)."""
    import torch
    cs, O, R = env
    dims = (32, 32, 64)
    n = 32 * 32 * 64
    nbytes = O.zfp_stream_bytes(*dims, maxbits)
    for sw in util.arbitrary_streams(nbytes // 4, maxbits):
        padded = torch.zeros(nbytes + SLACK, dtype=torch.uint8, device="cuda")
        padded[:nbytes] = torch.from_numpy(sw.view(np.uint8).copy()).cuda()
        ref_back = ref_decompress(R, padded, dims, maxbits, n)
        back = cs.zfp_decompress(padded[:nbytes].clone(), n, maxbits, dims)
        assert torch.equal(back.view(torch.int32), ref_back.view(torch.int32))


def test_config1(env):
    a = util.tanh_normal(128 * 64 * 32 * 32, seed=1)
    both(env, a, (32, 32, 8192), 512)


@pytest.mark.parametrize("rate", [4, 8, 16])
@pytest.mark.parametrize("dist", ["normal", "uniform"])
def test_rates(env, rate, dist):
    n = 1024 * 1024
    a = getattr(util, dist)(n, seed=rate)
    both(env, a, (32, 32, n // 1024), 64 * rate)


@pytest.mark.parametrize("maxbits", [64, 192, 512, 1024, 2048])
def test_awkward_blocks(env, maxbits):
    # includes blocks whose planes are written as full 64-bit words, which a
    # host build of the reference's bit writer cannot reproduce
    a = util.block_zoo(32 * 32 * 40, seed=maxbits)
    both(env, a, (32, 32, 40), maxbits)


@pytest.mark.parametrize("dims", [(32, 32, 7), (30, 17, 9), (5, 5, 5), (64, 16, 9)])
def test_partial_blocks(env, dims):
    nx, ny, nz = dims
    a = util.normal(nx * ny * nz, seed=nx + ny + nz)
    both(env, a, dims, 512)


@pytest.mark.parametrize("zero_fraction", [0.5, 0.75, 0.9])
def test_sparse_reference_layout(env, zero_fraction):
    """PreGPUcompression / PreAcc / GPUcompression / GPUdecompression of the
    product against the reference's kernels, config 2's tensor."""
    import torch
    cs, O, R = env
    n = 128 * 128 * 16 * 16
    a = util.relu_normal(n, zero_fraction, seed=3)
    t = torch.from_numpy(a).cuda()
    dimsize, blocksize = 512, 32
    P = dimsize * blocksize
    begin, bitmap, values, nnz = cs.legacy_sparse_compress(t, dimsize, blocksize)
    r_begin = torch.zeros(P, dtype=torch.int32, device="cuda")
    r_num = torch.zeros(1, dtype=torch.int32, device="cuda")
    r_bitmap = torch.zeros(bitmap.numel(), dtype=torch.int32, device="cuda")
    r_values = torch.zeros(n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    r_nnz = R.refcuda_sparse_compress(t.data_ptr(), n, dimsize, blocksize, r_begin.data_ptr(), r_num.data_ptr(),
                                      r_bitmap.data_ptr(), r_values.data_ptr())
    torch.cuda.synchronize()
    assert r_nnz == nnz == int(np.count_nonzero(a))
    assert torch.equal(begin, r_begin)
    assert torch.equal(bitmap, r_bitmap)
    assert torch.equal(values.view(torch.int32), r_values[:nnz].view(torch.int32))
    out = cs.legacy_sparse_decompress(values, n, bitmap, begin, dimsize, blocksize)
    r_out = torch.zeros(n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    R.refcuda_sparse_decompress(r_values.data_ptr(), r_out.data_ptr(), n, dimsize, blocksize, r_bitmap.data_ptr(),
                                r_begin.data_ptr())
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int32), r_out.view(torch.int32))
    assert np.array_equal(r_out.cpu().numpy(), a)
