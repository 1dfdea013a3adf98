"""Tensor-level front end of the codecs.

Each function takes CUDA float32 tensors, passes raw device pointers and the
current CUDA stream through the C ABI (include/cswap_b200.h) and returns
tensors.  Nothing here computes: without the CUDA library the calls raise.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from ._lib import SparseLayout, check, lib

# policy codes (CSWAP+/Execution.h:70,86,107,243)
POLICY_KEEP, POLICY_DROP, POLICY_RAW, POLICY_SPARSE, POLICY_ZFP = 0, 1, 2, 3, 6


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(device) -> int:
    """cudaStream_t of torch's current stream on `device` (the raw accessor
    skips building a Stream object, which matters at one call per swapped tensor)."""
    if _raw_stream is not None:
        dev = torch.device(device) if not isinstance(device, torch.device) else device
        return _raw_stream(dev.index if dev.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda_f32(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this path has no CPU implementation)")
    if t.dtype != torch.float32:
        raise ValueError(f"{name} must be float32")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


# ---------------------------------------------------------------------------
# ZFP
# ---------------------------------------------------------------------------

def zfp_view(numel: int) -> Tuple[int, int, int]:
    """(nx, ny, nz) of the swap path's 3-D view of a flat tensor."""
    nx, ny, nz = C.c_size_t(), C.c_size_t(), C.c_size_t()
    check(lib().csw_zfp_view(numel, C.byref(nx), C.byref(ny), C.byref(nz)), "csw_zfp_view")
    return nx.value, ny.value, nz.value


def zfp_max_bytes(nx: int, ny: int, nz: int, maxbits: int) -> int:
    out = C.c_size_t()
    check(lib().csw_zfp_max_bytes(nx, ny, nz, maxbits, C.byref(out)), "csw_zfp_max_bytes")
    return out.value


def _dims(t: torch.Tensor, dims: Optional[Tuple[int, int, int]]) -> Tuple[int, int, int]:
    if dims is not None:
        nx, ny, nz = dims
        if nx * max(ny, 1) * max(nz, 1) != t.numel():
            raise ValueError("dims do not match the tensor's element count")
        return nx, ny, nz
    return zfp_view(t.numel())


def zfp_compress(t: torch.Tensor, maxbits: int = 512, dims: Optional[Tuple[int, int, int]] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fixed-rate ZFP stream (uint8 tensor) of `t` at `maxbits` bits per block.

    `dims` = (nx, ny, nz), x fastest, 0 for unused axes; default is the swap
    path's 32 x 32 x numel/1024 view."""
    _require_cuda_f32(t, "t")
    nx, ny, nz = _dims(t, dims)
    need = zfp_max_bytes(nx, ny, nz, maxbits)
    if out is None:
        out = torch.empty(need, dtype=torch.uint8, device=t.device)
    elif out.numel() * out.element_size() < need or not out.is_cuda:
        raise ValueError("out is too small or not on the device")
    with torch.cuda.device(t.device):
        check(lib().csw_zfp_compress(t.data_ptr(), nx, ny, nz, maxbits, out.data_ptr(),
                                     out.numel() * out.element_size(), None, _stream_ptr(t.device)),
              "csw_zfp_compress")
    return out


def zfp_decompress(stream: torch.Tensor, numel: int, maxbits: int = 512,
                   dims: Optional[Tuple[int, int, int]] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not stream.is_cuda:
        raise ValueError("stream must be a CUDA tensor")
    if out is None:
        out = torch.empty(numel, dtype=torch.float32, device=stream.device)
    _require_cuda_f32(out, "out")
    nx, ny, nz = _dims(out, dims)
    with torch.cuda.device(stream.device):
        check(lib().csw_zfp_decompress(stream.data_ptr(), stream.numel() * stream.element_size(), nx, ny, nz, maxbits,
                                       out.data_ptr(), _stream_ptr(stream.device)), "csw_zfp_decompress")
    return out


# ---------------------------------------------------------------------------
# sparse, native layout
# ---------------------------------------------------------------------------

def sparse_layout(n: int) -> SparseLayout:
    L = SparseLayout()
    check(lib().csw_sparse_layout_of(n, C.byref(L)), "csw_sparse_layout_of")
    return L


def sparse_packed_bytes(n: int, nnz: int) -> int:
    """Bytes of a packed buffer that have to move for n elements, nnz kept."""
    return sparse_layout(n).values + 4 * nnz


def sparse_compress(t: torch.Tensor, out: Optional[torch.Tensor] = None,
                    nnz_out: Optional[torch.Tensor] = None, onepass: bool = False
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """(packed uint8 buffer, one-element int32 device tensor holding nnz).

    onepass=True reads the tensor once (csw_sparse_compress_onepass): same bitmap,
    count and per-tile contents, tile segments in schedule order."""
    _require_cuda_f32(t, "t")
    n = t.numel()
    L = sparse_layout(n)
    if out is None:
        out = torch.empty(L.bound, dtype=torch.uint8, device=t.device)
    if nnz_out is None:
        nnz_out = torch.zeros(1, dtype=torch.int32, device=t.device)
    with torch.cuda.device(t.device):
        fn = lib().csw_sparse_compress_onepass if onepass else lib().csw_sparse_compress
        check(fn(t.data_ptr(), n, out.data_ptr(), out.numel(), nnz_out.data_ptr(), _stream_ptr(t.device)),
              "csw_sparse_compress")
    return out, nnz_out


def sparse_decompress(packed: torch.Tensor, n: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not packed.is_cuda:
        raise ValueError("packed must be a CUDA tensor")
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=packed.device)
    _require_cuda_f32(out, "out")
    with torch.cuda.device(packed.device):
        check(lib().csw_sparse_decompress(packed.data_ptr(), n, out.data_ptr(), _stream_ptr(packed.device)),
              "csw_sparse_decompress")
    return out


# ---------------------------------------------------------------------------
# sparse, reference layout through the reference-named entry points
# ---------------------------------------------------------------------------

def legacy_sizes(n: int, workers: int):
    chunk = -(-n // workers)
    words_per = -(-chunk // 32)
    return chunk, words_per, words_per * workers


def legacy_sparse_compress(t: torch.Tensor, dimsize: int = 512, blocksize: int = 32):
    """The call sequence of CSWAP+/Execution.h:88-95.  Returns
    (begin int32[P], bitmap int32-as-uint32[P*ceil(chunk/32)], values f32[nnz], nnz).
    Reads the count back to size `values`, as the reference does."""
    import math

    _require_cuda_f32(t, "t")
    n = t.numel()
    P = dimsize * blocksize
    _, _, bw = legacy_sizes(n, P)
    L = lib()
    s = _stream_ptr(t.device)
    begin = torch.zeros(P, dtype=torch.int32, device=t.device)
    num = torch.zeros(1, dtype=torch.int32, device=t.device)
    bitmap = torch.zeros(bw, dtype=torch.int32, device=t.device)
    with torch.cuda.device(t.device):
        L.PreGPUcompression(n, P, t.data_ptr(), begin.data_ptr(), dimsize, blocksize, s)
        kernel_size = int(math.ceil(float(n) / math.ceil(float(n) / P)))
        L.PreAcc(begin.data_ptr(), kernel_size, num.data_ptr(), 1, 1, s)
        nnz = int(num.item())
        values = torch.empty(max(nnz, 1), dtype=torch.float32, device=t.device)
        L.GPUcompression(n, P, t.data_ptr(), values.data_ptr(), begin.data_ptr(), bitmap.data_ptr(), dimsize,
                         blocksize, s)
    return begin, bitmap, values[:nnz], nnz


def legacy_sparse_decompress(values: torch.Tensor, n: int, bitmap: torch.Tensor, begin: torch.Tensor,
                             dimsize: int = 512, blocksize: int = 32, out: Optional[torch.Tensor] = None):
    """GPUdecompression (runs on the legacy default stream like the reference)."""
    if out is None:
        out = torch.zeros(n, dtype=torch.float32, device=bitmap.device)
    v = values if values.numel() else torch.zeros(1, dtype=torch.float32, device=bitmap.device)
    with torch.cuda.device(bitmap.device):
        torch.cuda.current_stream(bitmap.device).synchronize()
        lib().GPUdecompression(v.data_ptr(), out.data_ptr(), n, dimsize * blocksize, bitmap.data_ptr(),
                               begin.data_ptr(), dimsize, blocksize)
        torch.cuda.synchronize(bitmap.device)
    return out
