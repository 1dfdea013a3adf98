"""The CPU oracle against fixtures generated from the host build of the
reference's own headers (tests/golden/make_golden.py)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import make_golden as G  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))


@pytest.mark.parametrize("case", G.CASES, ids=[c[0] for c in G.CASES])
def test_zfp_stream_and_decode(oracle, case):
    name, dims, maxbits, dist, seed = case
    nx, ny, nz = dims
    n = nx * max(ny, 1) * max(nz, 1)
    a = G.make_input(dist, n, seed)
    s = oracle.zfp_encode(a, nx, ny, nz, maxbits)
    want = GOLD[f"{name}.stream"]
    assert np.array_equal(s, want)
    # decoded blocks (including the padding lanes of partial blocks)
    blocks = GOLD[f"{name}.blocks"]
    d = 3 if nz else 2 if ny else 1
    for b in range(blocks.shape[0]):
        got = oracle.zfp_decode_block(np.concatenate([s, np.zeros(2, np.uint64)]), d, maxbits, b)
        assert np.array_equal(got.view(np.uint32), blocks[b].view(np.uint32))
    # and the assembled field
    back = oracle.zfp_decode(s, nx, ny, nz, maxbits)
    ref = np.zeros(n, dtype=np.float32)
    for b in range(blocks.shape[0]):
        _scatter(ref, dims, b, blocks[b])
    assert np.array_equal(back.view(np.uint32), ref.view(np.uint32))


def _scatter(out, dims, b, q):
    nx, ny, nz = dims
    d = 3 if nz else 2 if ny else 1
    ny1, nz1 = max(ny, 1), max(nz, 1)
    f = out.reshape(nz1, ny1, nx)
    bx, by = (nx + 3) // 4, (ny1 + 3) // 4 if d >= 2 else 1
    x0, y0, z0 = (b % bx) * 4, ((b // bx) % by) * 4 if d >= 2 else 0, (b // (bx * by)) * 4 if d >= 3 else 0
    q = q.reshape((4 if d >= 3 else 1), (4 if d >= 2 else 1), 4)
    for z in range(min(4 if d >= 3 else 1, nz1 - z0)):
        for y in range(min(4 if d >= 2 else 1, ny1 - y0)):
            for x in range(min(4, nx - x0)):
                f[z0 + z, y0 + y, x0 + x] = q[z, y, x]


def test_known_answer_block(oracle):
    blk = (1.5 * np.sin(0.37 * np.arange(64))).astype(np.float32)
    s, _ = oracle.zfp_encode_block(blk, 3, 512)
    assert np.array_equal(s[:8], GOLD["kat.stream"])
    assert [int(w) for w in s[:2]] == [0x2a08c10a20080501, 0x515654048028018c]


@pytest.mark.parametrize("name,n,dimsize,seed", [("sparse_5000", 5000, 16, 201), ("sparse_70001", 70001, 64, 202)])
def test_sparse_reference_layout(oracle, name, n, dimsize, seed):
    rng = np.random.default_rng(seed)
    a = np.maximum(0, rng.standard_normal(n) - 0.5).astype(np.float32)
    a[::7] = -0.0
    P = dimsize * 32
    begin, bitmap, values, nnz = oracle.legacy_sparse_compress(a, P)
    active = GOLD[f"{name}.begin"].size
    assert np.array_equal(begin[:active], GOLD[f"{name}.begin"])
    assert np.array_equal(bitmap, GOLD[f"{name}.bitmap"])
    assert np.array_equal(values.view(np.uint32), GOLD[f"{name}.values"].view(np.uint32))
    out = oracle.legacy_sparse_decompress(values, n, P, bitmap, begin, prefill=7.0)
    assert np.array_equal(out.view(np.uint32), GOLD[f"{name}.restored"].view(np.uint32))


def test_native_sparse_roundtrip_is_bit_exact(oracle):
    rng = np.random.default_rng(5)
    for n in (0, 1, 31, 32, 33, 4095, 4096, 4097, 100003):
        a = np.maximum(0, rng.standard_normal(n)).astype(np.float32)
        if n > 10:
            a[3] = -0.0
            a[5] = np.nan
        bitmap, values, tile_off, nnz = oracle.sparse_compress(a)
        assert nnz == int(np.count_nonzero(a.view(np.uint32)))
        if n:
            assert tile_off[0] == 0 and np.all(np.diff(tile_off.astype(np.int64)) >= 0)
        out = oracle.sparse_decompress(bitmap, values, n)
        assert np.array_equal(out.view(np.uint32), a.view(np.uint32))
