/*
 * Entry points with the reference's own names and signatures, so that code
 * written against CSWAP+ links against libcswap_b200.so unchanged:
 *
 *   PreGPUcompression / PreAcc / GPUcompression / GPUdecompression
 *       CSWAP+/zfp/compression.cuh:4-8, declared again at CSWAP+/Execution.h:23-27
 *   cuda_compress / cuda_decompress
 *       CSWAP+/zfp/cuZFP.h:10-12
 *
 * The structs below mirror the memory layout of zfp_stream, zfp_field and
 * bitstream (CSWAP+/zfp/zfp.h:95-102,140-145, CSWAP+/zfp/bitstream.c:131-141,
 * 64-bit stream words) so that objects built by the reference's zfp.c can be
 * passed straight in.
 */
#ifndef CSWAP_COMPAT_H
#define CSWAP_COMPAT_H

#include <stddef.h>
#include <stdint.h>

#include "cswap_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- sparse codec, reference layout -------------------------------------- */
/* P = kernelSize workers, chunk = ceil(arraySize / P).  Buffers:
 *   valueIndex[P] int32, bitmap[P * ceil(chunk/32)] uint32, values[nnz] float.
 * dimsize/blocksize are accepted for signature compatibility; the launch
 * shape is chosen by the library. */

/* per-worker non-zero counts (compression.cu:134-165) */
void PreGPUcompression(int arraySize, int kernelSize, float* arrayGPU, int* valueIndex, int dimsize, int blocksize,
                       csw_stream_t stream);
/* in-place exclusive scan of the first KernelSize counts; total to num[0]
 * (compression.cu:9-19) */
void PreAcc(int* valueIndex, int KernelSize, int* num, int dimsize, int blocksize, csw_stream_t stream);
/* occupancy words + packed non-zeros (compression.cu:168-239) */
void GPUcompression(int arraySize, int kernelSize, float* arrayGPU, float* compressedList, int* compressedValueIndex,
                    uint32_t* compressedBinIndex, int dimsize, int blocksize, csw_stream_t stream);
/* scatter back on the default stream; positions after the last set bit of
 * each bitmap word are not written (compression.cu:241-318,367-374) */
void GPUdecompression(float* arrayGPU, float* destiGPU, int arraySize, int kernelSize, uint32_t* gpuDataindex,
                      int* beginIndex, int dimsize, int blocksize);

/* ---- zfp objects ----------------------------------------------------------- */
typedef struct {
  unsigned bits;    /* buffered bits */
  uint64_t buffer;
  uint64_t* ptr;    /* next word */
  uint64_t* begin;  /* start of stream (host or device memory) */
  uint64_t* end;
} csw_bitstream;

typedef struct {
  unsigned minbits, maxbits, maxprec;
  int minexp;
  csw_bitstream* stream;
  struct {
    int policy;
    struct { unsigned threads, chunk_size; } omp;
  } exec;
} csw_zfp_stream;

typedef struct {
  int type;               /* 3 = float32 (zfp_type_float); other types are rejected */
  size_t nx, ny, nz, nw;
  ptrdiff_t sx, sy, sz, sw;
  void* data;             /* host or device memory */
} csw_zfp_field;

/* Fixed-rate compress at stream->maxbits bits per block; field data and the
 * stream buffer may each be host or device memory.  Blocks until done,
 * returns the stream bytes (0 on failure) and advances stream->stream->ptr
 * (cuZFP.cu:364-436). */
size_t cuda_compress(csw_zfp_stream* stream, const csw_zfp_field* field);
/* Inverse (cuZFP.cu:440-532). */
void cuda_decompress(csw_zfp_stream* stream, csw_zfp_field* field);

/* ---- the wrappers the reference's Execution calls -------------------------- */
/* Device memory for buffers the library hands to its caller (compress below).
 * Defaults to cudaMalloc / cudaFree; a libtorch program passes the caching
 * allocator's raw_alloc / raw_delete so that the caller can free the buffer
 * the way the reference does (Execution.h:296).  NULL restores the default. */
typedef void* (*csw_alloc_fn)(size_t bytes);
typedef void (*csw_free_fn)(void* p);
void csw_set_device_allocator(csw_alloc_fn alloc, csw_free_fn release);

#ifdef __cplusplus
}

/* C++ linkage, as in the reference's modified PyTorch (the definitions are not
 * part of the reference tree; only the call sites are):
 *   setRatio(int)            CSWAP+/Execution.h:63   bits per zfp block for later compress() calls
 *   compress(ptr, n, bytes)  CSWAP+/Execution.h:113  ZFP-compress n floats at dev_ptr on the legacy
 *                            default stream into a new device buffer (allocated through the
 *                            allocator set above, freed by the caller); out_bytes receives its
 *                            size.  The tensor is viewed 32 x 32 x n/1024; values past the last
 *                            whole slab follow the stream as they are.  NULL (out_bytes 0) on failure.
 *   decompress(buf, bytes, dst, n)  the inverse, for the swap-in half the reference keeps in its
 *                            engine: rebuilds n floats at dev_dst from a buffer made by compress()
 *                            at the current ratio. */
void setRatio(int maxbits);
void* compress(void* dev_ptr, size_t numel, size_t& out_bytes);
void decompress(void* dev_buf, size_t bytes, void* dev_dst, size_t numel);

extern "C" {
#endif

#ifdef __cplusplus
}
#endif
#endif /* CSWAP_COMPAT_H */
