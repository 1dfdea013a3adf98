"""Generates tests/golden/golden.npz from the HOST BUILD OF THE REFERENCE's own
headers (oracle/_ref/libcswap_ref.so, built by oracle/build_ref.sh where the
reference tree is mounted).  The fixtures pin the CPU oracle - and through it
the CUDA path - to the reference on machines where the reference is absent.

    python tests/golden/make_golden.py

Inputs are regenerated from seeds by the tests (numpy default_rng), only the
reference's outputs are stored.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

CASES = [
    # name, (nx, ny, nz), maxbits, distribution, seed
    ("c1_tanh_rate8", (32, 32, 8), 512, "tanh", 101),
    ("normal_rate4", (32, 32, 4), 256, "normal", 102),
    ("normal_rate16", (32, 32, 4), 1024, "normal", 103),
    ("uniform_rate8", (32, 32, 4), 512, "uniform", 104),
    ("partial_5x5x5", (5, 5, 5), 512, "normal", 105),
    ("partial_z_32x32x6", (32, 32, 6), 512, "tanh", 106),
    ("unaligned_300bits", (8, 8, 8), 300, "normal", 107),
    ("tiny_budget_37bits", (8, 8, 4), 37, "normal", 108),
    ("field_2d", (13, 10, 0), 256, "normal", 109),
    ("field_1d", (37, 0, 0), 64, "normal", 110),
    ("sparse_blocks", (16, 16, 8), 512, "sparse", 111),
    ("smooth", (16, 16, 16), 512, "smooth", 112),
    ("wide_range", (8, 8, 8), 1024, "wide", 113),
]


def make_input(dist, n, seed):
    rng = np.random.default_rng(seed)
    if dist == "tanh":
        a = np.tanh(rng.standard_normal(n))
    elif dist == "normal":
        a = rng.standard_normal(n)
    elif dist == "uniform":
        a = rng.uniform(-1, 1, n)
    elif dist == "sparse":
        a = np.maximum(0, rng.standard_normal(n) - 1.0)
    elif dist == "smooth":
        a = np.sin(0.01 * np.arange(n)) * 3 + 0.001 * rng.standard_normal(n)
    elif dist == "wide":
        a = rng.standard_normal(n) * 10.0 ** rng.integers(-8, 8, n)
    else:
        raise KeyError(dist)
    return a.astype(np.float32)


def gather(a, dims, b):
    """block b of the field, replicate padded (CSWAP+/zfp/encode3.cuh:12-47)."""
    nx, ny, nz = dims
    d = 3 if nz else 2 if ny else 1
    ny1, nz1 = max(ny, 1), max(nz, 1)
    f = a.reshape(nz1, ny1, nx)
    bx, by = (nx + 3) // 4, (ny1 + 3) // 4 if d >= 2 else 1
    x0, y0, z0 = (b % bx) * 4, ((b // bx) % by) * 4 if d >= 2 else 0, (b // (bx * by)) * 4 if d >= 3 else 0

    def idx(o, n):
        v = min(4, n - o)
        pad = {1: [0, 0, 0, 0], 2: [0, 1, 1, 0], 3: [0, 1, 2, 0], 4: [0, 1, 2, 3]}[v]
        return [o + p for p in pad]
    xs = idx(x0, nx)
    ys = idx(y0, ny1) if d >= 2 else [0]
    zs = idx(z0, nz1) if d >= 3 else [0]
    return np.ascontiguousarray(f[np.ix_(zs, ys, xs)]).ravel().astype(np.float32), d


def ref_field(a, dims, maxbits):
    """stream and decode of the whole field through the reference's block codec"""
    R = O.ref()
    nx, ny, nz = dims
    d = 3 if nz else 2 if ny else 1
    nb = ((nx + 3) // 4) * ((max(ny, 1) + 3) // 4 if d >= 2 else 1) * ((max(nz, 1) + 3) // 4 if d >= 3 else 1)
    words = (nb * maxbits + 63) // 64
    buf = np.zeros(words + 2, dtype=np.uint64)
    nbytes = buf.size * 8
    size = 1 << (2 * d)
    dec = np.zeros((nb, size), dtype=np.float32)
    for b in range(nb):
        blk, _ = gather(a, dims, b)
        R.ref_bs_encode_block(blk.ctypes.data_as(C.POINTER(C.c_float)), d, maxbits, b, buf.ctypes.data, nbytes)
    for b in range(nb):
        R.ref_bs_decode_block(buf.ctypes.data, nbytes, d, maxbits, b, dec[b].ctypes.data_as(C.POINTER(C.c_float)))
    return buf[:words].copy(), dec


def main():
    O.build()
    assert O.have_ref(), "the reference tree is not mounted; cannot generate fixtures"
    R = O.ref()
    out = {}
    for name, dims, maxbits, dist, seed in CASES:
        n = dims[0] * max(dims[1], 1) * max(dims[2], 1)
        a = make_input(dist, n, seed)
        stream, dec = ref_field(a, dims, maxbits)
        out[f"{name}.stream"] = stream
        out[f"{name}.blocks"] = dec
    # known-answer block from the reference's zfp_encode_block as written
    blk = (1.5 * np.sin(0.37 * np.arange(64))).astype(np.float32)
    kat = np.zeros(8, dtype=np.uint64)
    R.ref_asis_encode_block(blk.ctypes.data_as(C.POINTER(C.c_float)), 3, 512, 0, kat.ctypes.data_as(C.POINTER(C.c_uint64)))
    out["kat.stream"] = kat
    # sparse, reference layout
    for name, n, dimsize, seed in (("sparse_5000", 5000, 16, 201), ("sparse_70001", 70001, 64, 202)):
        rng = np.random.default_rng(seed)
        a = np.maximum(0, rng.standard_normal(n) - 0.5).astype(np.float32)
        a[::7] = -0.0
        P = dimsize * 32
        _, _, bw, active = O.legacy_sizes(n, P)
        begin = np.zeros(P, dtype=np.int32)
        bitmap = np.zeros(bw, dtype=np.uint32)
        values = np.zeros(n, dtype=np.float32)
        nnz = R.ref_sparse_compress(a.ctypes.data_as(C.POINTER(C.c_float)), n, dimsize, 32,
                                    begin.ctypes.data_as(C.POINTER(C.c_int32)),
                                    bitmap.ctypes.data_as(C.POINTER(C.c_uint32)),
                                    values.ctypes.data_as(C.POINTER(C.c_float)))
        dst = np.full(n, 7.0, dtype=np.float32)
        R.ref_sparse_decompress(values.ctypes.data_as(C.POINTER(C.c_float)), dst.ctypes.data_as(C.POINTER(C.c_float)),
                                n, dimsize, 32, bitmap.ctypes.data_as(C.POINTER(C.c_uint32)),
                                begin.ctypes.data_as(C.POINTER(C.c_int32)))
        out[f"{name}.begin"] = begin[:active]
        out[f"{name}.bitmap"] = bitmap
        out[f"{name}.values"] = values[:nnz]
        out[f"{name}.restored"] = dst
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
