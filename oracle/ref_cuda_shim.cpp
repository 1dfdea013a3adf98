// Thin C entry points around the reference's own CUDA codec (cuZFP.cu and
// compression.cu of CSWAP+/zfp, compiled where they lie by build_ref_cuda.sh
// into _ref/libcswap_ref_cuda.so).  TEST INFRASTRUCTURE ONLY: the tests use it
// to compare the product's streams with what the reference's kernels emit on
// the same GPU, and bench.py times it as the reference arm.  Nothing of the
// reference is copied here; its headers are included by path.
//
// The reference prints timing lines from inside cuda_compress /
// cuda_decompress (cuZFP.cu:392-399,469-476, encode3.cuh:151); they are sent
// to /dev/null for the duration of each call so that callers keep a clean
// standard output.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

extern "C" {
#include "zfp.h"
}
#include "cuZFP.h"
#include "compression.cuh"

namespace {
struct Quiet {
  int saved;
  Quiet() {
    fflush(stdout);
    saved = dup(1);
    int nul = open("/dev/null", O_WRONLY);
    if (nul >= 0) {
      dup2(nul, 1);
      close(nul);
    }
  }
  ~Quiet() {
    fflush(stdout);
    if (saved >= 0) {
      dup2(saved, 1);
      close(saved);
    }
  }
};

void fill_field(zfp_field* f, void* data, size_t nx, size_t ny, size_t nz) {
  memset(f, 0, sizeof(*f));
  f->type = zfp_type_float;
  f->nx = nx;
  f->ny = ny;
  f->nz = nz;
  f->data = data;
}
}  // namespace

extern "C" {

// sizeof / offsetof of the reference's structs, for layout checks of the
// product's mirrors (include/cswap_compat.h)
size_t refcuda_sizeof_zfp_stream() { return sizeof(zfp_stream); }
size_t refcuda_sizeof_zfp_field() { return sizeof(zfp_field); }

// Compress the device array d_field (nx*ny*nz floats, contiguous; ny = nz = 0
// for lower-dimensional fields) at maxbits bits per block into the device
// buffer d_stream of cap bytes.  Returns the stream bytes the reference reports.
size_t refcuda_zfp_compress(float* d_field, size_t nx, size_t ny, size_t nz, unsigned maxbits, void* d_stream,
                            size_t cap) {
  Quiet q;
  zfp_field field;
  fill_field(&field, d_field, nx, ny, nz);
  zfp_stream* zfp = zfp_stream_open(NULL);
  zfp->minbits = maxbits;
  zfp->maxbits = maxbits;
  bitstream* bs = stream_open(d_stream, cap);
  zfp_stream_set_bit_stream(zfp, bs);
  zfp_stream_rewind(zfp);
  const size_t bytes = cuda_compress(zfp, &field);
  zfp_stream_close(zfp);
  stream_close(bs);
  return bytes;
}

void refcuda_zfp_decompress(void* d_stream, size_t cap, size_t nx, size_t ny, size_t nz, unsigned maxbits,
                            float* d_field) {
  Quiet q;
  zfp_field field;
  fill_field(&field, d_field, nx, ny, nz);
  zfp_stream* zfp = zfp_stream_open(NULL);
  zfp->minbits = maxbits;
  zfp->maxbits = maxbits;
  bitstream* bs = stream_open(d_stream, cap);
  zfp_stream_set_bit_stream(zfp, bs);
  zfp_stream_rewind(zfp);
  cuda_decompress(zfp, &field);
  zfp_stream_close(zfp);
  stream_close(bs);
}

// The sparse call sequence of Execution::pre, policy 3 (Execution.h:88-95),
// on the legacy default stream: count, scan, read the total back (the
// reference blocks on this copy), pack.  Returns the number of non-zeros.
int refcuda_sparse_compress(float* d_in, int n, int dimsize, int blocksize, int* d_begin, int* d_num,
                            uint32_t* d_bitmap, float* d_values) {
  const int P = dimsize * blocksize;
  PreGPUcompression(n, P, d_in, d_begin, dimsize, blocksize, 0);
  const int active = (int)ceilf((float)n / ceilf((float)n / (float)P));  // Execution.h:90
  PreAcc(d_begin, active, d_num, 1, 1, 0);
  int nnz = 0;
  cudaMemcpy(&nnz, d_num, sizeof(int), cudaMemcpyDeviceToHost);
  GPUcompression(n, P, d_in, d_values, d_begin, d_bitmap, dimsize, blocksize, 0);
  return nnz;
}

// GPUdecompression as Execution's backward hook calls it (default stream).
void refcuda_sparse_decompress(float* d_values, float* d_out, int n, int dimsize, int blocksize, uint32_t* d_bitmap,
                               int* d_begin) {
  GPUdecompression(d_values, d_out, n, dimsize * blocksize, d_bitmap, d_begin, dimsize, blocksize);
}

}  // extern "C"
