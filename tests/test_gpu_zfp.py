"""Parity of the CUDA ZFP codec (through the C ABI) with the CPU oracle:
streams and decoded arrays must be bit-identical."""
import ctypes as C

import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cs():
    import torch
    import cswap_b200
    assert torch.cuda.is_available()
    cswap_b200.lib()
    return cswap_b200


def _roundtrip(cs, O, a, dims, maxbits):
    """compress + decompress on the GPU; compare both with the oracle."""
    import torch
    nx, ny, nz = dims
    t = torch.from_numpy(a).cuda()
    stream = cs.zfp_compress(t, maxbits, dims)
    ref = O.zfp_encode(a, nx, ny, nz, maxbits, threads=O.max_threads())
    got = stream.cpu().numpy().view(np.uint64)
    assert got.size == ref.size
    assert np.array_equal(got, ref), f"stream differs at word {np.flatnonzero(got != ref)[:4]}"
    back = cs.zfp_decompress(stream, a.size, maxbits, dims).cpu().numpy()
    ref_back = O.zfp_decode(ref, nx, ny, nz, maxbits, threads=O.max_threads())
    assert np.array_equal(back.view(np.uint32), ref_back.view(np.uint32))
    assert cs.lib().csw_device_status(None) == 0
    return back


def test_config1_tanh_rate8(cs, oracle):
    # float32 [128,64,32,32] = 32 MiB viewed 32 x 32 x 8192 at rate 8
    a = util.tanh_normal(128 * 64 * 32 * 32, seed=1)
    back = _roundtrip(cs, oracle, a, (32, 32, 8192), 512)
    err = back.astype(np.float64) - a
    assert np.abs(err).max() < 0.25 and np.sqrt((err ** 2).mean()) < 0.03


@pytest.mark.parametrize("rate", [4, 8, 16])
@pytest.mark.parametrize("dist", ["normal", "uniform"])
@pytest.mark.parametrize("kib", [64, 256, 1024, 16384])
def test_rate_sweep(cs, oracle, rate, dist, kib):
    n = kib * 256
    a = getattr(util, dist)(n, seed=kib + rate)
    _roundtrip(cs, oracle, a, (32, 32, n // 1024), 64 * rate)


@pytest.mark.parametrize("maxbits", [32, 64, 96, 160, 256, 512, 1024, 2048])
def test_awkward_blocks_all_word_rates(cs, oracle, maxbits):
    a = util.block_zoo(32 * 32 * 40, seed=maxbits)
    _roundtrip(cs, oracle, a, (32, 32, 40), maxbits)


@pytest.mark.parametrize("nz", [1, 2, 3, 5, 7, 8, 9, 12, 15, 16, 17, 18, 19, 31, 33, 67])
def test_partial_slabs(cs, oracle, nz):
    a = util.tanh_normal(1024 * nz, seed=nz)
    _roundtrip(cs, oracle, a, (32, 32, nz), 512)


@pytest.mark.parametrize("dims", [(4, 4, 4), (5, 5, 5), (9, 7, 3), (64, 16, 9), (31, 33, 6), (32, 32, 0), (13, 10, 0),
                                  (4, 4, 0), (4, 0, 0), (13, 0, 0), (1000, 0, 0), (1, 0, 0), (1, 1, 1), (2, 3, 0)])
@pytest.mark.parametrize("maxbits", [37, 64, 300, 512])
def test_generic_geometry(cs, oracle, dims, maxbits):
    nx, ny, nz = dims
    n = nx * max(ny, 1) * max(nz, 1)
    a = util.normal(n, seed=n + maxbits)
    _roundtrip(cs, oracle, a, dims, maxbits)


@pytest.mark.parametrize("dims", [(4, 0, 0), (13, 0, 0), (5, 5, 5), (4, 4, 0), (12, 4, 4)])
@pytest.mark.parametrize("maxbits", [32, 96, 160])
def test_generic_odd_word_count_writes_every_byte(cs, oracle, dims, maxbits):
    """Whole 32-bit words per block but an odd number of words in all: the last
    32 bits of the 64-bit-sized stream belong to no block and must still be
    written (as zeros), whatever the buffer held before."""
    import torch
    nx, ny, nz = dims
    n = nx * max(ny, 1) * max(nz, 1)
    a = util.normal(n, seed=n + maxbits)
    need = cs.zfp_max_bytes(nx, ny, nz, maxbits)
    out = torch.full((need,), 0xFF, dtype=torch.uint8, device="cuda")
    cs.zfp_compress(torch.from_numpy(a).cuda(), maxbits, dims, out=out)
    ref = oracle.zfp_encode(a, nx, ny, nz, maxbits)
    assert np.array_equal(out.cpu().numpy().view(np.uint64), ref)


def test_special_values(cs, oracle):
    n = 1024 * 16
    a = np.zeros(n, dtype=np.float32)
    _roundtrip(cs, oracle, a, (32, 32, 16), 512)          # all zero
    a[:] = -0.0
    _roundtrip(cs, oracle, a, (32, 32, 16), 512)          # negative zeros act as zero
    a = util.normal(n, 3) * np.float32(1e-36)             # scale factor overflows (emax < -97)
    _roundtrip(cs, oracle, a, (32, 32, 16), 512)
    a = util.normal(n, 4) * np.float32(1e30)
    _roundtrip(cs, oracle, a, (32, 32, 16), 512)
    a = np.full(n, 3.0e38, dtype=np.float32)              # near FLT_MAX
    _roundtrip(cs, oracle, a, (32, 32, 16), 256)


def test_known_answer_block(cs):
    # the 64-value block f[i] = 1.5 sin(0.37 i), rate 8, first block of a 4x4x4 field
    import torch
    blk = (1.5 * np.sin(0.37 * np.arange(64))).astype(np.float32)
    s = cs.zfp_compress(torch.from_numpy(blk).cuda(), 512, (4, 4, 4)).cpu().numpy().view(np.uint64)
    want = [0x2a08c10a20080501, 0x515654048028018c, 0xc632018a42b02a06, 0x6a341c144b518439,
            0x122b67b9050b0242, 0x89006d52210c28ca, 0xf84059df88b61197, 0x697de4eee05d0126]
    assert [int(w) for w in s] == want


@pytest.mark.parametrize("mib,rate", [(256, 8), (256, 4), (256, 16), (512, 4), (512, 8), (512, 16)])
def test_full_size_properties(cs, oracle, mib, rate):
    """256 MiB and 512 MiB tensors (the top of the size sweep) at rates 4, 8 and
    16: the stream of the whole equals the streams of its parts (blocks are
    independent), sampled groups match the oracle, the decoded tensor equals
    the oracle's decode of those groups and stays within the rate's error
    bound, and a second trip through the codec stays within that bound."""
    import torch
    n = mib * 262144
    maxbits = 64 * rate
    bound = {4: 4.0, 8: 0.25, 16: 1.5e-3}[rate]
    g = torch.Generator(device="cuda").manual_seed(7 + mib + rate)
    t = torch.tanh(torch.randn(n, device="cuda", generator=g))
    nz = n // 1024
    whole = cs.zfp_compress(t, maxbits)
    assert whole.numel() == n * rate // 8
    part = 4 * 1024 * 1024
    for k in range(0, n, part * 8):  # every 8th 16 MiB piece
        piece = cs.zfp_compress(t[k:k + part].contiguous(), maxbits)
        assert torch.equal(piece, whole[k * rate // 8:(k + part) * rate // 8])
    back = cs.zfp_decompress(whole, n, maxbits)
    rng = np.random.default_rng(mib + rate)
    picks = [0, nz - 16] + [int(z) & ~3 for z in rng.integers(0, nz - 16, 14)]
    for z0 in picks:
        a = t[z0 * 1024:(z0 + 16) * 1024].cpu().numpy()
        ref = oracle.zfp_encode(a, 32, 32, 16, maxbits)
        got = whole[z0 * 128 * rate:(z0 + 16) * 128 * rate].cpu().numpy().view(np.uint64)
        assert np.array_equal(got, ref)
        ref_back = oracle.zfp_decode(ref, 32, 32, 16, maxbits)
        assert np.array_equal(back[z0 * 1024:(z0 + 16) * 1024].cpu().numpy().view(np.uint32), ref_back.view(np.uint32))
    assert float((back - t).abs().max()) < bound
    again = cs.zfp_decompress(cs.zfp_compress(back, maxbits), n, maxbits)
    # a second trip through the codec moves values by at most the first trip's error bound
    assert float((again - back).abs().max()) < bound
    assert cs.lib().csw_device_status(None) == 0


def test_reconstruction_error_table(cs, capsys):
    import torch
    n = 8 * 1024 * 1024
    rows = []
    for dist in ("normal", "uniform", "tanh_normal"):
        a = torch.from_numpy(getattr(util, dist)(n, 11)).cuda()
        for rate in (4, 8, 16):
            b = cs.zfp_decompress(cs.zfp_compress(a, 64 * rate), n, 64 * rate)
            e = (b - a).double()
            rows.append((dist, rate, float(e.abs().max()), float(e.pow(2).mean().sqrt())))
    with capsys.disabled():
        for r in rows:
            print("recon %-12s rate %2d  max_abs %.3e  rmse %.3e" % r)
    by = {(d, r): (m, s) for d, r, m, s in rows}
    for d in ("normal", "uniform", "tanh_normal"):
        assert by[(d, 16)][1] < by[(d, 8)][1] < by[(d, 4)][1]


def test_errors_do_not_launch(cs):
    import torch
    t = torch.zeros(4096, device="cuda")
    out = torch.zeros(16, dtype=torch.uint8, device="cuda")
    L = cs.lib()
    need = C.c_size_t()
    st = L.csw_zfp_compress(t.data_ptr(), 32, 32, 4, 512, out.data_ptr(), 16, C.byref(need), None)
    assert st == 2 and need.value == 4096  # CSW_ERR_SIZE, required bytes reported
    assert L.csw_zfp_compress(t.data_ptr(), 32, 32, 4, 8, out.data_ptr(), 16, None, None) == 1  # maxbits < 9
    assert L.csw_zfp_compress(None, 32, 32, 4, 512, out.data_ptr(), 16, None, None) == 1
    assert L.csw_zfp_compress(t.data_ptr(), 0, 0, 0, 512, out.data_ptr(), 16, None, None) == 1
    assert torch.count_nonzero(out).item() == 0


def test_strided_field(cs, oracle):
    """A 3-D window of a larger array through the strided entry point."""
    import torch
    big = torch.from_numpy(util.normal(40 * 36 * 12, 5)).cuda().view(12, 36, 40)
    win = big[1:11, 2:34, 4:36]  # nz=10, ny=32, nx=32
    nx, ny, nz = 32, 32, 10
    L = cs.lib()
    need = cs.zfp_max_bytes(nx, ny, nz, 512)
    out = torch.empty(need, dtype=torch.uint8, device="cuda")
    st = L.csw_zfp_compress_strided(win.data_ptr(), nx, ny, nz, win.stride(2), win.stride(1), win.stride(0), 512,
                                    out.data_ptr(), need, None, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    ref = oracle.zfp_encode(win.contiguous().cpu().numpy(), nx, ny, nz, 512)
    assert np.array_equal(out.cpu().numpy().view(np.uint64), ref)
    dst = torch.zeros_like(big)
    dwin = dst[1:11, 2:34, 4:36]
    st = L.csw_zfp_decompress_strided(out.data_ptr(), need, nx, ny, nz, dwin.stride(2), dwin.stride(1),
                                      dwin.stride(0), 512, dwin.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    ref_back = oracle.zfp_decode(ref, nx, ny, nz, 512).reshape(nz, ny, nx)
    assert np.array_equal(dwin.cpu().numpy(), ref_back)
    mask = torch.ones_like(dst, dtype=torch.bool)
    mask[1:11, 2:34, 4:36] = False
    assert torch.count_nonzero(dst[mask]).item() == 0  # nothing outside the window was touched


@pytest.mark.parametrize("where", ["host", "device"])
def test_reference_named_entry_points(cs, oracle, where):
    """cuda_compress / cuda_decompress with zfp-layout structs (cuZFP.h:10-12)."""
    import torch
    from cswap_b200._lib import Bitstream, ZfpField, ZfpStream
    nx, ny, nz, maxbits = 32, 32, 24, 512
    a = util.tanh_normal(nx * ny * nz, 9)
    nbytes = cs.zfp_max_bytes(nx, ny, nz, maxbits)
    L = cs.lib()
    if where == "host":
        field_buf = a.copy()
        stream_buf = np.zeros(nbytes // 8, dtype=np.uint64)
        fptr, sptr = field_buf.ctypes.data, stream_buf.ctypes.data
    else:
        ft = torch.from_numpy(a).cuda()
        st_t = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        fptr, sptr = ft.data_ptr(), st_t.data_ptr()
    bs = Bitstream(0, 0, sptr, sptr, sptr + nbytes)
    zs = ZfpStream(maxbits, maxbits, 32, -1074, C.pointer(bs))
    fld = ZfpField(3, nx, ny, nz, 0, 0, 0, 0, 0, fptr)
    got_bytes = L.cuda_compress(C.byref(zs), C.byref(fld))
    assert got_bytes == nbytes
    assert bs.ptr == sptr + nbytes and bs.bits == 64
    ref = oracle.zfp_encode(a, nx, ny, nz, maxbits)
    got = stream_buf if where == "host" else st_t.cpu().numpy().view(np.uint64)
    assert np.array_equal(got, ref)
    if where == "host":
        field_buf[:] = 0
    else:
        ft.zero_()
        torch.cuda.synchronize()
    bs2 = Bitstream(0, 0, sptr, sptr, sptr + nbytes)
    zs2 = ZfpStream(maxbits, maxbits, 32, -1074, C.pointer(bs2))
    L.cuda_decompress(C.byref(zs2), C.byref(fld))
    back = field_buf if where == "host" else ft.cpu().numpy()
    assert np.array_equal(back, oracle.zfp_decode(ref, nx, ny, nz, maxbits))


def test_large_host_call_is_pipelined_and_exact(cs):
    """Host field + host stream of 100 MiB: cuda_compress / cuda_decompress cut
    the field into z-chunks and overlap copies with coding; the bytes must be
    the ones the one-shot device path produces (nz deliberately ragged)."""
    import torch
    from cswap_b200._lib import Bitstream, ZfpField, ZfpStream
    nx, ny, nz, maxbits = 32, 32, 25601 + 2, 512
    n = nx * ny * nz
    t = torch.tanh(torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)))
    want = cs.zfp_compress(t, maxbits, (nx, ny, nz))
    want_back = cs.zfp_decompress(want, n, maxbits, (nx, ny, nz))
    nbytes = cs.zfp_max_bytes(nx, ny, nz, maxbits)
    h_field = t.cpu().pin_memory()
    h_stream = torch.zeros(nbytes, dtype=torch.uint8).pin_memory()
    L = cs.lib()
    sp = h_stream.data_ptr()
    bs = Bitstream(0, 0, sp, sp, sp + nbytes)
    zs = ZfpStream(maxbits, maxbits, 32, -1074, C.pointer(bs))
    fld = ZfpField(3, nx, ny, nz, 0, 0, 0, 0, 0, h_field.data_ptr())
    assert L.cuda_compress(C.byref(zs), C.byref(fld)) == nbytes
    assert torch.equal(h_stream, want.cpu())
    h_out = torch.zeros(n, dtype=torch.float32).pin_memory()
    bs2 = Bitstream(0, 0, sp, sp, sp + nbytes)
    zs2 = ZfpStream(maxbits, maxbits, 32, -1074, C.pointer(bs2))
    fld2 = ZfpField(3, nx, ny, nz, 0, 0, 0, 0, 0, h_out.data_ptr())
    L.cuda_decompress(C.byref(zs2), C.byref(fld2))
    assert bs2.ptr == sp + nbytes
    assert torch.equal(h_out, want_back.cpu())


def test_fork_wrappers_compress_set_ratio(cs, oracle):
    """setRatio / compress / decompress, the wrappers the reference's Execution
    calls (CSWAP+/Execution.h:63,113): the buffer compress() returns holds the
    oracle's stream of the 32 x 32 x n/1024 view followed by the values past
    the last whole slab, and it comes from the allocator the caller supplied."""
    import torch
    L = cs.lib()
    held = {}

    @C.CFUNCTYPE(C.c_void_p, C.c_size_t)
    def alloc(nbytes):
        t = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        held[t.data_ptr()] = t
        return t.data_ptr()

    @C.CFUNCTYPE(None, C.c_void_p)
    def release(p):
        held.pop(p, None)

    L.csw_set_device_allocator(C.cast(alloc, C.c_void_p), C.cast(release, C.c_void_p))
    try:
        n = 1024 * 20 + 300
        a = util.tanh_normal(n, 21)
        t = torch.from_numpy(a).cuda()
        torch.cuda.synchronize()
        for maxbits in (128, 512):
            L.cxx_setRatio(maxbits)
            nbytes = C.c_size_t()
            buf = L.cxx_compress(t.data_ptr(), n, C.byref(nbytes))
            assert buf in held and nbytes.value == 20 * 16 * maxbits // 8 + 300 * 4  # 16 blocks per slab
            torch.cuda.synchronize()
            g = held[buf].cpu().numpy()[:nbytes.value]
            zb = nbytes.value - 1200
            ref = oracle.zfp_encode(a[:20480], 32, 32, 20, maxbits)
            assert np.array_equal(g[:zb].view(np.uint64), ref)
            assert np.array_equal(g[zb:].view(np.float32), a[20480:])
            back = torch.zeros(n, device="cuda")
            torch.cuda.synchronize()
            L.cxx_decompress(buf, nbytes.value, back.data_ptr(), n)
            torch.cuda.synchronize()
            want = np.concatenate([oracle.zfp_decode(ref, 32, 32, 20, maxbits), a[20480:]])
            assert np.array_equal(back.cpu().numpy().view(np.uint32), want.view(np.uint32))
            release(buf)
        assert not held
    finally:
        L.cxx_setRatio(512)
        L.csw_set_device_allocator(None, None)


@pytest.mark.parametrize("dims", [(32, 32, 64), (32, 32, 7), (20, 12, 9)])
@pytest.mark.parametrize("maxbits", [32, 64, 128, 512, 1024, 100])
def test_decode_arbitrary_streams(cs, oracle, dims, maxbits):
    """Decoding is defined for any bit string (a swapped-out tensor may come
    back from a file): slab and generic kernels must produce what the oracle
    produces, bit for bit, also for streams no encoder wrote."""
    import torch
    nx, ny, nz = dims
    nbytes = oracle.zfp_stream_bytes(nx, ny, nz, maxbits)
    for sw in util.arbitrary_streams(nbytes // 4, maxbits + nz):
        s64 = np.ascontiguousarray(sw).view(np.uint64)
        ref = oracle.zfp_decode(s64, nx, ny, nz, maxbits, threads=oracle.max_threads())
        stream = torch.from_numpy(sw.view(np.uint8).copy()).cuda()
        got = cs.zfp_decompress(stream, nx * ny * nz, maxbits, dims).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    assert cs.lib().csw_device_status(None) == 0
