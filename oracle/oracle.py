"""ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the bench's CPU-baseline / reference legs may
import this module; the product package never does.

Two shared objects are wrapped:

* ``libcswap_oracle.so``  - the plain-C restatement (``cswap_oracle.c``), built
  by ``oracle/Makefile``; travels everywhere.
* ``_ref/libcswap_ref.so`` - the reference's own headers compiled for the host
  (``ref_shim.cpp`` + ``build_ref.sh``); only buildable where the reference
  tree is mounted, used to pin the restatement and to generate fixtures.
* ``_ref/libcswap_ref_cuda.so`` - the reference's own CUDA codec compiled for
  sm_100a (``ref_cuda_shim.cpp`` + ``build_ref_cuda.sh``); built where the
  reference tree is mounted, runs wherever a GPU is: the GPU tests compare the
  product's streams with it and the bench times it as the reference arm.

The reference checkout is found through the environment variable
``CSWAP_REFERENCE`` or, failing that, as a directory named ``reference`` next
to this repository.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libcswap_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libcswap_ref.so")
_REF_CUDA_SO = os.path.join(_HERE, "_ref", "libcswap_ref_cuda.so")

TILE = 4096


def build(force: bool = False) -> None:
    """Compile the C restatement (and the reference host build when the
    reference tree is present)."""
    src = os.path.join(_HERE, "cswap_oracle.c")
    if force or not os.path.exists(_ORACLE_SO) or os.path.getmtime(_ORACLE_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "libcswap_oracle.so"])
    ref_root = reference_root()
    if ref_root is not None:
        env = dict(os.environ, CSWAP_REFERENCE=ref_root)
        shim = os.path.join(_HERE, "ref_shim.cpp")
        if force or not os.path.exists(_REF_SO) or os.path.getmtime(_REF_SO) < os.path.getmtime(shim):
            subprocess.check_call([os.path.join(_HERE, "build_ref.sh")], stdout=subprocess.DEVNULL, env=env)
        shim = os.path.join(_HERE, "ref_cuda_shim.cpp")
        if force or not os.path.exists(_REF_CUDA_SO) or os.path.getmtime(_REF_CUDA_SO) < os.path.getmtime(shim):
            subprocess.check_call([os.path.join(_HERE, "build_ref_cuda.sh")], stdout=subprocess.DEVNULL,
                                  stderr=subprocess.DEVNULL, env=env)


def reference_root():
    """Directory of the reference checkout, or None where it is not mounted."""
    cands = [os.environ.get("CSWAP_REFERENCE"),
             os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "CSWAP+", "zfp")):
            return os.path.abspath(c)
    return None


_lib = None
_ref = None


def _f32(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _u64(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint64))


def _u32(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint32))


def _i32(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_ORACLE_SO):
            build()
        L = C.CDLL(_ORACLE_SO)
        L.orc_zfp_stream_bytes.restype = C.c_size_t
        L.orc_zfp_stream_bytes.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, C.c_uint]
        L.orc_zfp_encode.restype = C.c_size_t
        L.orc_zfp_encode.argtypes = [C.POINTER(C.c_float), C.c_size_t, C.c_size_t, C.c_size_t, C.c_uint,
                                     C.POINTER(C.c_uint64), C.c_int]
        L.orc_zfp_decode.restype = None
        L.orc_zfp_decode.argtypes = [C.POINTER(C.c_uint64), C.c_size_t, C.c_size_t, C.c_size_t, C.c_uint,
                                     C.POINTER(C.c_float), C.c_int]
        L.orc_zfp_encode_block.restype = C.c_int
        L.orc_zfp_encode_block.argtypes = [C.POINTER(C.c_float), C.c_int, C.c_uint, C.c_size_t,
                                           C.POINTER(C.c_uint64)]
        L.orc_zfp_decode_block.restype = None
        L.orc_zfp_decode_block.argtypes = [C.POINTER(C.c_uint64), C.c_int, C.c_uint, C.c_size_t,
                                           C.POINTER(C.c_float)]
        L.orc_fwd_lift.argtypes = [C.POINTER(C.c_int32), C.c_uint]
        L.orc_inv_lift.argtypes = [C.POINTER(C.c_int32), C.c_uint]
        L.orc_int2uint.restype = C.c_uint32
        L.orc_int2uint.argtypes = [C.c_int32]
        L.orc_uint2int.restype = C.c_int32
        L.orc_uint2int.argtypes = [C.c_uint32]
        L.orc_perm3.restype = C.POINTER(C.c_ubyte)
        L.orc_sparse_compress.restype = C.c_size_t
        L.orc_sparse_compress.argtypes = [C.POINTER(C.c_float), C.c_size_t, C.POINTER(C.c_uint32),
                                          C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.c_int]
        L.orc_sparse_decompress.restype = None
        L.orc_sparse_decompress.argtypes = [C.POINTER(C.c_uint32), C.POINTER(C.c_float), C.c_size_t,
                                            C.POINTER(C.c_float), C.c_int]
        L.orc_legacy_sparse_compress.restype = C.c_size_t
        L.orc_legacy_sparse_compress.argtypes = [C.POINTER(C.c_float), C.c_int, C.c_int, C.POINTER(C.c_int32),
                                                 C.POINTER(C.c_uint32), C.POINTER(C.c_float)]
        L.orc_legacy_sparse_decompress.restype = None
        L.orc_legacy_sparse_decompress.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int, C.c_int,
                                                   C.POINTER(C.c_uint32), C.POINTER(C.c_int32)]
        L.orc_max_threads.restype = C.c_int
        _lib = L
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF_SO)


def ref():
    global _ref
    if _ref is None:
        R = C.CDLL(_REF_SO)
        R.ref_asis_encode_block.argtypes = [C.POINTER(C.c_float), C.c_int, C.c_int, C.c_uint, C.POINTER(C.c_uint64)]
        R.ref_asis_decode_block.argtypes = [C.POINTER(C.c_uint64), C.c_int, C.c_int, C.c_uint, C.POINTER(C.c_float)]
        R.ref_bs_encode_block.argtypes = [C.POINTER(C.c_float), C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_size_t]
        R.ref_bs_decode_block.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_size_t, C.POINTER(C.c_float)]
        R.ref_perm3.restype = C.POINTER(C.c_ubyte)
        R.ref_perm2.restype = C.POINTER(C.c_ubyte)
        R.ref_fwd_lift.argtypes = [C.POINTER(C.c_int32), C.c_int]
        R.ref_inv_lift.argtypes = [C.POINTER(C.c_int32), C.c_int]
        R.ref_sparse_compress.restype = C.c_int
        R.ref_sparse_compress.argtypes = [C.POINTER(C.c_float), C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int32),
                                          C.POINTER(C.c_uint32), C.POINTER(C.c_float)]
        R.ref_sparse_decompress.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int, C.c_int, C.c_int,
                                            C.POINTER(C.c_uint32), C.POINTER(C.c_int32)]
        _ref = R
    return _ref


def have_ref_cuda() -> bool:
    return os.path.exists(_REF_CUDA_SO)


_ref_cuda = None


def ref_cuda():
    """The reference's CUDA codec (needs a GPU).  Arguments are raw device
    pointers; every call runs on the legacy default stream and blocks."""
    global _ref_cuda
    if _ref_cuda is None:
        R = C.CDLL(_REF_CUDA_SO, mode=os.RTLD_LOCAL)
        R.refcuda_zfp_compress.restype = C.c_size_t
        R.refcuda_zfp_compress.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_uint, C.c_void_p,
                                           C.c_size_t]
        R.refcuda_zfp_decompress.restype = None
        R.refcuda_zfp_decompress.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_uint,
                                             C.c_void_p]
        R.refcuda_sparse_compress.restype = C.c_int
        R.refcuda_sparse_compress.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p]
        R.refcuda_sparse_decompress.restype = None
        R.refcuda_sparse_decompress.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                                C.c_void_p]
        R.refcuda_sizeof_zfp_stream.restype = C.c_size_t
        R.refcuda_sizeof_zfp_field.restype = C.c_size_t
        _ref_cuda = R
    return _ref_cuda


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---------------------------------------------------------------------------
# ZFP
# ---------------------------------------------------------------------------

def zfp_stream_bytes(nx, ny, nz, maxbits) -> int:
    return int(lib().orc_zfp_stream_bytes(nx, ny, nz, maxbits))


def zfp_encode(a: np.ndarray, nx, ny, nz, maxbits, threads=1) -> np.ndarray:
    """Stream (uint64 words) of the contiguous float32 array `a` viewed nx*ny*nz."""
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    assert a.size == nx * max(ny, 1) * max(nz, 1)
    nbytes = zfp_stream_bytes(nx, ny, nz, maxbits)
    out = np.zeros(nbytes // 8 + 1, dtype=np.uint64)
    lib().orc_zfp_encode(_f32(a), nx, ny, nz, maxbits, _u64(out), threads)
    return out[: nbytes // 8]


def zfp_decode(stream: np.ndarray, nx, ny, nz, maxbits, threads=1) -> np.ndarray:
    s = np.zeros(stream.size + 2, dtype=np.uint64)
    s[: stream.size] = stream
    out = np.zeros(nx * max(ny, 1) * max(nz, 1), dtype=np.float32)
    lib().orc_zfp_decode(_u64(s), nx, ny, nz, maxbits, _f32(out), threads)
    return out


def zfp_encode_block(block: np.ndarray, dims, maxbits, block_idx=0, stream=None):
    block = np.ascontiguousarray(block, dtype=np.float32)
    if stream is None:
        stream = np.zeros(((block_idx + 1) * maxbits + 63) // 64 + 1, dtype=np.uint64)
    nmax = lib().orc_zfp_encode_block(_f32(block), dims, maxbits, block_idx, _u64(stream))
    return stream, nmax


def zfp_decode_block(stream: np.ndarray, dims, maxbits, block_idx=0) -> np.ndarray:
    out = np.zeros(1 << (2 * dims), dtype=np.float32)
    lib().orc_zfp_decode_block(_u64(stream), dims, maxbits, block_idx, _f32(out))
    return out


# ---------------------------------------------------------------------------
# sparse
# ---------------------------------------------------------------------------

def sparse_compress(a: np.ndarray, threads=1):
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    n = a.size
    bitmap = np.zeros((n + 31) // 32, dtype=np.uint32)
    values = np.zeros(max(n, 1), dtype=np.float32)
    tile_off = np.zeros(max((n + TILE - 1) // TILE, 1), dtype=np.uint32)
    nnz = lib().orc_sparse_compress(_f32(a), n, _u32(bitmap), _f32(values), _u32(tile_off), threads) if n else 0
    return bitmap, values[:nnz].copy(), tile_off[: (n + TILE - 1) // TILE], int(nnz)


def sparse_decompress(bitmap, values, n, threads=1) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    v = np.ascontiguousarray(values, dtype=np.float32)
    if v.size == 0:
        v = np.zeros(1, dtype=np.float32)
    if n:
        lib().orc_sparse_decompress(_u32(np.ascontiguousarray(bitmap)), _f32(v), n, _f32(out), threads)
    return out


def legacy_sizes(n: int, P: int):
    """(chunk, words_per_worker, bitmap_words, active) of the reference layout."""
    chunk = -(-n // P)
    words_per = -(-chunk // 32)
    import math
    active = int(math.ceil(np.float32(n) / math.ceil(np.float32(n) / np.float32(P))))
    return chunk, words_per, words_per * P, active


def legacy_sparse_compress(a: np.ndarray, P: int):
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    n = a.size
    _, _, bw, _ = legacy_sizes(n, P)
    begin = np.zeros(P, dtype=np.int32)
    bitmap = np.zeros(bw, dtype=np.uint32)
    values = np.zeros(n, dtype=np.float32)
    nnz = lib().orc_legacy_sparse_compress(_f32(a), n, P, _i32(begin), _u32(bitmap), _f32(values))
    return begin, bitmap, values[:nnz].copy(), int(nnz)


def legacy_sparse_decompress(values, n, P, bitmap, begin, prefill=0.0) -> np.ndarray:
    out = np.full(n, prefill, dtype=np.float32)
    v = np.ascontiguousarray(values, dtype=np.float32)
    if v.size == 0:
        v = np.zeros(1, dtype=np.float32)
    lib().orc_legacy_sparse_decompress(_f32(v), _f32(out), n, P, _u32(bitmap), _i32(begin))
    return out
