"""Parity of the CUDA sparse codec (through the C ABI) with the CPU oracle."""
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


def _check_native(cs, O, a):
    import torch
    n = a.size
    t = torch.from_numpy(a).cuda()
    packed, nnz_t = cs.sparse_compress(t)
    nnz = int(nnz_t.item())
    bitmap, values, tile_off, ref_nnz = O.sparse_compress(a)
    assert nnz == ref_nnz
    L = cs.sparse_layout(n)
    buf = packed.cpu().numpy()
    tiles = (n + 4095) // 4096
    words = (n + 31) // 32
    assert np.array_equal(buf[L.tile_off:L.tile_off + 4 * tiles].view(np.uint32), tile_off)
    assert np.array_equal(buf[L.bitmap:L.bitmap + 4 * words].view(np.uint32), bitmap)
    assert np.array_equal(buf[L.values:L.values + 4 * nnz].view(np.uint32), values.view(np.uint32))
    out = cs.sparse_decompress(packed, n)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), a.view(np.uint32))  # bit-exact, incl. -0.0 / NaN
    assert cs.sparse_packed_bytes(n, nnz) == L.values + 4 * nnz
    return nnz


def _check_onepass(cs, O, a):
    """Single-pass compressor: the bitmap and the count are the oracle's, every
    tile's segment holds the oracle's values for that tile, the segments tile
    the values array without gaps or overlaps (in whatever order), and both the
    library and the oracle decode the buffer back to the input."""
    import torch
    n = a.size
    t = torch.from_numpy(a).cuda()
    packed, nnz_t = cs.sparse_compress(t, onepass=True)
    nnz = int(nnz_t.item())
    bitmap, values, tile_off, ref_nnz = O.sparse_compress(a)
    assert nnz == ref_nnz
    L = cs.sparse_layout(n)
    buf = packed.cpu().numpy()
    tiles = (n + 4095) // 4096
    words = (n + 31) // 32
    got_bitmap = buf[L.bitmap:L.bitmap + 4 * words].view(np.uint32)
    assert np.array_equal(got_bitmap, bitmap)
    got_off = buf[L.tile_off:L.tile_off + 4 * tiles].view(np.uint32).astype(np.int64)
    got_vals = buf[L.values:L.values + 4 * nnz].view(np.uint32)
    ref_off = np.append(tile_off.astype(np.int64), ref_nnz)
    cnt = np.diff(ref_off)
    order = np.argsort(got_off, kind="stable")
    nonempty = order[cnt[order] > 0]
    # segments of the non-empty tiles are disjoint and cover [0, nnz)
    starts = got_off[nonempty]
    assert np.array_equal(starts, np.concatenate(([0], np.cumsum(cnt[nonempty])[:-1]))) if nonempty.size else nnz == 0
    assert np.all(got_off <= nnz)
    ref_vals = values.view(np.uint32)
    for tl in range(tiles):
        assert np.array_equal(got_vals[got_off[tl]:got_off[tl] + cnt[tl]], ref_vals[ref_off[tl]:ref_off[tl + 1]])
    out = cs.sparse_decompress(packed, n)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), a.view(np.uint32))
    # the oracle's tile-by-tile decoder reads the same buffer
    dec = np.zeros(n, dtype=np.uint32)
    for tl in range(tiles):
        lo, hi = tl * 4096, min(n, (tl + 1) * 4096)
        bits = np.unpackbits(got_bitmap[lo // 32:(hi + 31) // 32].view(np.uint8), bitorder="little")[:hi - lo]
        dec[lo:hi][bits.astype(bool)] = got_vals[got_off[tl]:got_off[tl] + cnt[tl]]
    assert np.array_equal(dec, a.view(np.uint32))
    return nnz


@pytest.mark.parametrize("n", [1, 33, 4095, 4096, 4097, 8192 + 17, (1 << 20) + 5, 128 * 128 * 16 * 16])
def test_onepass_matches_oracle_per_tile(cs, oracle, n):
    _check_onepass(cs, oracle, util.relu_normal(n, 0.75, seed=n + 1))


def test_onepass_special_patterns(cs, oracle):
    n = 5 * 4096 + 100
    _check_onepass(cs, oracle, np.zeros(n, dtype=np.float32))
    _check_onepass(cs, oracle, util.normal(n, 1) + np.float32(10))
    a = util.relu_normal(n, 0.5, 3)
    a[::7] = -0.0
    a[5::11] = np.nan
    a.view(np.uint32)[9::17] = 0x7fc12345
    _check_onepass(cs, oracle, a)


def test_onepass_full_size_and_host_count_rejected(cs):
    """256 MiB: count and round trip; a count word outside device memory is refused."""
    import torch
    n = 64 * 1024 * 1024
    g = torch.Generator(device="cuda").manual_seed(6)
    t = torch.relu(torch.randn(n, device="cuda", generator=g))
    packed, nnz_t = cs.sparse_compress(t, onepass=True)
    assert int(nnz_t.item()) == int(torch.count_nonzero(t).item())
    out = cs.sparse_decompress(packed, n)
    assert torch.equal(out.view(torch.int32), t.view(torch.int32))
    # the multiset of packed values is that of the non-zeros
    L = cs.sparse_layout(n)
    vals = packed[L.values:L.values + 4 * int(nnz_t.item())].view(torch.float32)
    assert torch.equal(torch.sort(vals).values, torch.sort(t[t != 0]).values)
    host_word = torch.zeros(1, dtype=torch.int32).pin_memory()
    st = cs.lib().csw_sparse_compress_onepass(t.data_ptr(), n, packed.data_ptr(), packed.numel(),
                                              host_word.data_ptr(), None)
    assert st == 1  # CSW_ERR_ARG


@pytest.mark.parametrize("zf", [0.5, 0.75, 0.9])
def test_config2_relu_activations(cs, oracle, zf, capsys):
    # float32 [128,128,16,16] = 16 MiB
    n = 128 * 128 * 16 * 16
    a = util.relu_normal(n, zf, seed=2)
    nnz = _check_native(cs, oracle, a)
    measured = 1 - nnz / n
    assert abs(measured - zf) < 0.01
    ratio = 4 * n / cs.sparse_packed_bytes(n, nnz)
    with capsys.disabled():
        print(f"sparse zeros {measured:.3f}: ratio {ratio:.2f}x")
    assert ratio > {0.5: 1.8, 0.75: 3.3, 0.9: 7.0}[zf]


@pytest.mark.parametrize("n", [1, 31, 32, 33, 1000, 4095, 4096, 4097, 8192 + 17, 1 << 20, (1 << 20) + 5])
def test_ragged_sizes(cs, oracle, n):
    a = util.relu_normal(n, 0.75, seed=n)
    _check_native(cs, oracle, a)


def test_special_patterns(cs, oracle):
    n = 3 * 4096 + 100
    _check_native(cs, oracle, np.zeros(n, dtype=np.float32))                       # nothing kept
    _check_native(cs, oracle, util.normal(n, 1) + np.float32(10))                  # everything kept
    a = util.relu_normal(n, 0.5, 3)
    a[::7] = -0.0                                                                   # negative zero survives
    a[5::11] = np.nan
    a[3::13] = np.float32(1e-45)                                                    # denormal survives
    a.view(np.uint32)[9::17] = 0x7fc12345                                           # NaN payload survives
    _check_native(cs, oracle, a)


def test_empty_tensor(cs):
    import torch
    t = torch.empty(0, device="cuda")
    packed, nnz = cs.sparse_compress(t, out=torch.empty(64, dtype=torch.uint8, device="cuda"))
    assert int(nnz.item()) == 0


def test_full_size_properties(cs):
    """256 MiB tensor: bit-exact round trip, count equals torch's, values are
    the non-zeros in order."""
    import torch
    n = 64 * 1024 * 1024
    g = torch.Generator(device="cuda").manual_seed(5)
    t = torch.relu(torch.randn(n, device="cuda", generator=g) - 0.6745)
    packed, nnz_t = cs.sparse_compress(t)
    nnz = int(nnz_t.item())
    assert nnz == int(torch.count_nonzero(t).item())
    L = cs.sparse_layout(n)
    vals = packed[L.values:L.values + 4 * nnz].view(torch.float32)
    assert torch.equal(vals, t[t != 0])
    out = cs.sparse_decompress(packed, n)
    assert torch.equal(out.view(torch.int32), t.view(torch.int32))


def test_capacity_check(cs):
    import ctypes as C
    import torch
    t = torch.ones(4096, device="cuda")
    out = torch.empty(64, dtype=torch.uint8, device="cuda")
    nnz = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = cs.lib().csw_sparse_compress(t.data_ptr(), 4096, out.data_ptr(), 64, nnz.data_ptr(), None)
    assert st == 2  # CSW_ERR_SIZE


@pytest.mark.parametrize("n,dimsize", [(128 * 128 * 16 * 16, 512), (1000, 512), (16384 * 32 + 5, 512), (12345, 256),
                                       (16384 * 64, 512), (100000, 512)])
def test_reference_layout(cs, oracle, n, dimsize):
    """PreGPUcompression / PreAcc / GPUcompression / GPUdecompression with the
    reference's buffers, byte for byte."""
    import torch
    P = dimsize * 32
    a = util.relu_normal(n, 0.75, seed=n % 97)
    a[::5] = np.where(a[::5] == 0, np.float32(-0.0), a[::5])  # -0.0 is dropped by the float compare
    a[7::1001] = np.nan
    t = torch.from_numpy(a).cuda()
    begin, bitmap, values, nnz = cs.legacy_sparse_compress(t, dimsize, 32)
    rb, rbm, rv, rn = oracle.legacy_sparse_compress(a, P)
    chunk, wp, bw, active = oracle.legacy_sizes(n, P)
    assert nnz == rn
    assert np.array_equal(begin.cpu().numpy()[:active], rb[:active])
    assert np.array_equal(bitmap.cpu().numpy().view(np.uint32), rbm)
    assert np.array_equal(values.cpu().numpy().view(np.uint32), rv.view(np.uint32))
    # decompression leaves positions after the last set bit of a word untouched
    pre = torch.full((n,), 7.0, device="cuda")
    out = cs.legacy_sparse_decompress(values, n, bitmap, begin, dimsize, 32, out=pre)
    want = oracle.legacy_sparse_decompress(rv, n, P, rbm, rb, prefill=7.0)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # on a zeroed destination it is the original up to the sign of zero
    out0 = cs.legacy_sparse_decompress(values, n, bitmap, begin, dimsize, 32)
    got = out0.cpu().numpy()
    keep = ~np.isnan(a)
    assert np.array_equal(got[keep], a[keep] + np.float32(0.0)) and np.isnan(got[~keep]).all()
