"""ctypes binding of libcswap_b200.so (declarations mirror include/cswap_b200.h
and include/cswap_compat.h)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcswap_b200.so")


class LibraryMissing(RuntimeError):
    pass


class CswapError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(what)


class SparseLayout(C.Structure):
    _fields_ = [("tile_off", C.c_size_t), ("bitmap", C.c_size_t), ("values", C.c_size_t), ("bound", C.c_size_t)]


class MgrConfig(C.Structure):
    _fields_ = [("device", C.c_int), ("pinned_bytes", C.c_size_t), ("staging_bytes", C.c_size_t),
                ("zfp_maxbits", C.c_uint)]


class TicketInfo(C.Structure):
    _fields_ = [("policy", C.c_int), ("numel", C.c_size_t), ("raw_bytes", C.c_size_t), ("moved_bytes", C.c_size_t),
                ("complete", C.c_int)]


class BlobHeader(C.Structure):
    _fields_ = [("magic", C.c_uint32), ("version", C.c_uint32), ("policy", C.c_uint32), ("zfp_maxbits", C.c_uint32),
                ("numel", C.c_uint64), ("payload_bytes", C.c_uint64), ("nnz", C.c_uint64),
                ("reserved", C.c_uint64 * 3)]


class MgrStats(C.Structure):
    _fields_ = [("swap_outs", C.c_uint64), ("swap_ins", C.c_uint64), ("raw_bytes_out", C.c_uint64),
                ("moved_bytes_out", C.c_uint64), ("raw_bytes_in", C.c_uint64), ("moved_bytes_in", C.c_uint64),
                ("pinned_in_use", C.c_size_t), ("pinned_high_water", C.c_size_t), ("staging_in_use", C.c_size_t),
                ("staging_high_water", C.c_size_t)]


class CostModelStruct(C.Structure):
    _fields_ = [(n, C.c_double) for n in
                ("zfp_enc_a", "zfp_enc_b", "zfp_dec_a", "zfp_dec_b", "sparse_enc_a", "sparse_enc_b", "sparse_dec_a",
                 "sparse_dec_b", "d2h_a", "d2h_bps", "h2d_a", "h2d_bps")] + [("zfp_maxbits", C.c_uint)] + \
               [(n, C.c_double) for n in ("sparse_enc_b75", "sparse_enc_b90", "sparse_dec_b75", "sparse_dec_b90",
                                          "host_swap_s")]


class TensorDescStruct(C.Structure):
    _fields_ = [("numel", C.c_size_t), ("zero_fraction", C.c_double), ("lossy_ok", C.c_int),
                ("ready_s", C.c_double), ("need_s", C.c_double)]


class Bitstream(C.Structure):
    _fields_ = [("bits", C.c_uint), ("buffer", C.c_uint64), ("ptr", C.c_void_p), ("begin", C.c_void_p),
                ("end", C.c_void_p)]


class _Omp(C.Structure):
    _fields_ = [("threads", C.c_uint), ("chunk_size", C.c_uint)]


class _Exec(C.Structure):
    _fields_ = [("policy", C.c_int), ("omp", _Omp)]


class ZfpStream(C.Structure):
    _fields_ = [("minbits", C.c_uint), ("maxbits", C.c_uint), ("maxprec", C.c_uint), ("minexp", C.c_int),
                ("stream", C.POINTER(Bitstream)), ("exec", _Exec)]


class ZfpField(C.Structure):
    _fields_ = [("type", C.c_int), ("nx", C.c_size_t), ("ny", C.c_size_t), ("nz", C.c_size_t), ("nw", C.c_size_t),
                ("sx", C.c_ssize_t), ("sy", C.c_ssize_t), ("sz", C.c_ssize_t), ("sw", C.c_ssize_t),
                ("data", C.c_void_p)]


_P = C.c_void_p
_SZ = C.c_size_t
_SSZ = C.c_ssize_t
_U = C.c_uint
_I = C.c_int

# name -> (restype, argtypes); every symbol the two headers declare
SIGNATURES = {
    "csw_status_string": (C.c_char_p, [_I]),
    "csw_last_cuda_error": (_I, []),
    "csw_version": (C.c_char_p, []),
    "csw_device_status": (_I, [_P]),
    "csw_zfp_max_bytes": (_I, [_SZ, _SZ, _SZ, _U, C.POINTER(_SZ)]),
    "csw_zfp_compress": (_I, [_P, _SZ, _SZ, _SZ, _U, _P, _SZ, C.POINTER(_SZ), _P]),
    "csw_zfp_compress_strided": (_I, [_P, _SZ, _SZ, _SZ, _SSZ, _SSZ, _SSZ, _U, _P, _SZ, C.POINTER(_SZ), _P]),
    "csw_zfp_decompress": (_I, [_P, _SZ, _SZ, _SZ, _SZ, _U, _P, _P]),
    "csw_zfp_decompress_strided": (_I, [_P, _SZ, _SZ, _SZ, _SZ, _SSZ, _SSZ, _SSZ, _U, _P, _P]),
    "csw_zfp_view": (_I, [_SZ, C.POINTER(_SZ), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "csw_sparse_layout_of": (_I, [_SZ, C.POINTER(SparseLayout)]),
    "csw_sparse_compress": (_I, [_P, _SZ, _P, _SZ, _P, _P]),
    "csw_sparse_compress_static": (_I, [_P, _SZ, _P, _SZ, _P, _P]),
    "csw_sparse_compress_onepass": (_I, [_P, _SZ, _P, _SZ, _P, _P]),
    "csw_sparse_decompress": (_I, [_P, _SZ, _P, _P]),
    "csw_mgr_create": (_I, [C.POINTER(MgrConfig), C.POINTER(_P)]),
    "csw_mgr_destroy": (_I, [_P]),
    "csw_mgr_set_zfp_maxbits": (_I, [_P, _U]),
    "csw_mgr_keep_staged": (_I, [_P, C.c_int]),
    "csw_swap_out_cancel": (_I, [_P, _P, C.POINTER(C.c_int)]),
    "csw_mgr_get_streams": (_I, [_P, C.POINTER(_P), C.POINTER(_P), C.POINTER(_P)]),
    "csw_swap_out": (_I, [_P, _P, _SZ, _I, _P, C.POINTER(_P)]),
    "csw_swap_out_done": (_I, [_P, _P, C.POINTER(_I)]),
    "csw_swap_out_sync": (_I, [_P, _P]),
    "csw_swap_out_wait": (_I, [_P, _P, _P]),
    "csw_prefetch": (_I, [_P, _P]),
    "csw_swap_in": (_I, [_P, _P, _P, _P]),
    "csw_swap_in_start": (_I, [_P, _P, _P, _P]),
    "csw_swap_in_wait": (_I, [_P, _P, _P]),
    "csw_ticket_release": (_I, [_P, _P]),
    "csw_ticket_query": (_I, [_P, _P, C.POINTER(TicketInfo)]),
    "csw_ticket_export": (_I, [_P, _P, _P, _SZ, C.POINTER(_SZ)]),
    "csw_blob_info": (_I, [_P, _SZ, C.POINTER(BlobHeader)]),
    "csw_blob_import": (_I, [_P, _P, _SZ, C.POINTER(_P)]),
    "csw_mgr_get_stats": (_I, [_P, C.POINTER(MgrStats)]),
    "csw_mgr_reset_stats": (_I, [_P]),
    "csw_mgr_sync": (_I, [_P]),
    "csw_cost_fit": (_I, [_P, C.POINTER(CostModelStruct)]),
    "csw_cost_decide": (_I, [C.POINTER(CostModelStruct), C.POINTER(TensorDescStruct), _SZ, C.c_double, C.POINTER(_I),
                             C.POINTER(C.c_double)]),
    "csw_cost_simulate": (_I, [C.POINTER(CostModelStruct), C.POINTER(TensorDescStruct), _SZ, C.c_double, C.POINTER(_I),
                               C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "csw_host_alloc": (_I, [_SZ, C.POINTER(_P)]),
    "csw_host_free": (_I, [_P]),
    # reference-named entry points
    "PreGPUcompression": (None, [_I, _I, _P, _P, _I, _I, _P]),
    "PreAcc": (None, [_P, _I, _P, _I, _I, _P]),
    "GPUcompression": (None, [_I, _I, _P, _P, _P, _P, _I, _I, _P]),
    "GPUdecompression": (None, [_P, _P, _I, _I, _P, _P, _I, _I]),
    "cuda_compress": (_SZ, [C.POINTER(ZfpStream), C.POINTER(ZfpField)]),
    "cuda_decompress": (None, [C.POINTER(ZfpStream), C.POINTER(ZfpField)]),
    "csw_set_device_allocator": (None, [_P, _P]),
}

# entry points with C++ linkage (the wrappers the reference's Execution calls,
# CSWAP+/Execution.h:63,113): declared name -> (exported symbol, restype, argtypes)
CXX_SIGNATURES = {
    "setRatio": ("_Z8setRatioi", None, [_I]),
    "compress": ("_Z8compressPvmRm", _P, [_P, _SZ, C.POINTER(_SZ)]),
    "decompress": ("_Z10decompressPvmS_m", None, [_P, _SZ, _P, _SZ]),
}

_lib = None


def lib():
    """The loaded library; raises LibraryMissing when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m cswap_b200.build` (nvcc, sm_100a). "
                "There is no CPU implementation of this path.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        for name, (symbol, res, args) in CXX_SIGNATURES.items():
            fn = getattr(L, symbol)
            fn.restype = res
            fn.argtypes = args
            setattr(L, "cxx_" + name, fn)
        _lib = L
    return _lib


def check(status: int, what: str = "") -> None:
    if status != 0:
        L = lib()
        msg = L.csw_status_string(status).decode()
        if status == 3:
            msg += f" (cudaError {L.csw_last_cuda_error()})"
        raise CswapError(status, f"{what}: {msg}" if what else msg)
