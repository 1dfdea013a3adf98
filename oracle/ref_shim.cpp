/*
 * Host build of the reference's own codec code.  TEST INFRASTRUCTURE ONLY.
 *
 * This file holds no reference source: it includes the reference's headers
 * from where they lie (-I <reference>/CSWAP+/zfp) and wraps them in a C ABI so
 * the CPU restatement (cswap_oracle.c) can be checked against them.  The
 * build recipe is oracle/build_ref.sh; the output goes to oracle/_ref/ only.
 *
 * Three flavours are exported:
 *   ref_asis_*   the reference's zfp_encode_block / zfp_decode exactly as
 *                written, BlockWriter/BlockReader included.  On x86 their
 *                64-bit shifts by 64 differ from the GPU (which yields 0), so
 *                these are only valid for blocks whose plane coder never
 *                writes a full 64-bit verbatim plane.
 *   ref_bs_*     the reference's arithmetic (max_exponent, fwd_cast,
 *                fwd_xform, fwd_order, uint2int, inv_xform, dequantize) with
 *                bit I/O through the reference's bitstream.c and a plane loop
 *                that follows encode.cuh:331-344 / decode.cuh:141-173.
 *   ref_sparse_* the reference's four sparse kernels run as host loops over
 *                (blockIdx, threadIdx); their bodies are cut out of
 *                compression.cu at build time into a temporary include.
 */
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstring>

typedef unsigned int uint;
using std::fabs;
using std::frexp;
using std::ldexp;
using std::max;
using std::min;
using std::modf;
using std::pow;
using std::sqrt;
static inline int min(unsigned a, int b) { return (int)a < b ? (int)a : b; }
static inline int min(int a, unsigned b) { return a < (int)b ? a : (int)b; }
static inline unsigned long long atomicAdd(unsigned long long* p, unsigned long long v) {
  unsigned long long o = *p;
  *p += v;
  return o;
}

#include "encode.cuh"
#include "decode.cuh"

/* bit I/O of the reference's bitstream.c is declared by bitstream.h (pulled in
 * through zfp.h); the recipe compiles bitstream.c as C and links it. */

template <int BS>
static void asis_encode(float* fblock, int maxbits, unsigned block_idx, unsigned long long* stream) {
  cuZFP::zfp_encode_block<float, BS>(fblock, maxbits, block_idx, stream);
}

template <int BS>
static void asis_decode(unsigned long long* stream, int maxbits, unsigned block_idx, float* fblock) {
  cuZFP::BlockReader<BS> reader(stream, maxbits, block_idx, INT_MAX);
  memset(fblock, 0, sizeof(float) * BS);
  cuZFP::zfp_decode<float, BS>(reader, fblock, maxbits);
}

/* plane loops over the reference's bitstream (same control flow as
 * encode.cuh:331-344 and decode.cuh:141-173) */
template <int BS>
static void bs_encode(float* fblock, int maxbits, size_t block_idx, void* buf, size_t bytes) {
  using namespace cuZFP;
  bitstream* s = stream_open(buf, bytes);
  /* blocks are written strictly in order by the caller; seek is only legal on
   * word boundaries for writes, so the caller guarantees ordered calls when
   * maxbits % 64 != 0 by passing block_idx == next block. */
  size_t start = block_idx * (size_t)maxbits;
  if (start % 64 == 0) {
    stream_wseek(s, start);
  } else {
    /* re-read the partial word already written and continue from it */
    stream_rseek(s, start - start % 64);
    uint64_t head = stream_read_bits(s, (uint)(start % 64));
    stream_wseek(s, start - start % 64);
    stream_write_bits(s, head, (uint)(start % 64));
  }
  int emax = max_exponent<float, BS>(fblock);
  int maxprec = precision(emax, get_precision<float>(), get_min_exp<float>());
  uint e = maxprec ? emax + get_ebias<float>() : 0;
  if (e) {
    stream_write_bits(s, 2 * e + 1, 9);
    int iblock[BS];
    fwd_cast<float, int, BS>(iblock, fblock, emax);
    transform<BS> t;
    t.fwd_xform(iblock);
    unsigned ublock[BS];
    fwd_order<int, unsigned, BS>(ublock, iblock);
    uint bits = maxbits - 9;
    for (uint k = 32, n = 0; bits && k-- > 0;) {
      uint64 x = 0;
      for (uint i = 0; i < BS; i++) x += (uint64)((ublock[i] >> k) & 1u) << i;
      uint m = n < bits ? n : bits;
      bits -= m;
      x = stream_write_bits(s, x, m);
      for (; n < BS && bits && (bits--, stream_write_bit(s, !!x)); x >>= 1, n++)
        for (; n < BS - 1 && bits && (bits--, !stream_write_bit(s, x & 1u)); x >>= 1, n++)
          ;
    }
  }
  size_t used = stream_wtell(s) - start;
  stream_pad(s, (uint)(maxbits - used));
  stream_flush(s);
  stream_close(s);
}

template <int BS>
static void bs_decode(void* buf, size_t bytes, int maxbits, size_t block_idx, float* fblock) {
  using namespace cuZFP;
  bitstream* s = stream_open(buf, bytes);
  stream_rseek(s, block_idx * (size_t)maxbits);
  memset(fblock, 0, sizeof(float) * BS);
  if (stream_read_bit(s)) {
    uint emax = (uint)stream_read_bits(s, 8) - get_ebias<float>();
    unsigned ublock[BS];
    memset(ublock, 0, sizeof(ublock));
    uint bits = maxbits - 9, k, m, n;
    for (k = 32, m = n = 0; bits && (m = 0, k-- > 0);) {
      m = n < bits ? n : bits;
      bits -= m;
      uint64 x = stream_read_bits(s, m);
      for (; bits && n < BS; n++, m = n) {
        bits--;
        if (stream_read_bit(s)) {
          for (; bits && n < BS - 1; n++) {
            bits--;
            if (stream_read_bit(s)) break;
          }
          x += (uint64)1 << n;
        } else {
          m = BS;
          break;
        }
      }
      for (uint i = 0; i < BS; i++, x >>= 1) ublock[i] += (unsigned)(x & 1u) << k;
    }
    int iblock[BS];
    const unsigned char* perm = get_perm<BS>();
    for (int i = 0; i < BS; ++i) iblock[perm[i]] = uint2int(ublock[i]);
    inv_transform<BS> t;
    t.inv_xform(iblock);
    float inv_w = dequantize<int, float>(1, emax);
    for (int i = 0; i < BS; ++i) fblock[i] = inv_w * (float)iblock[i];
  }
  stream_close(s);
}

/* ---- sparse kernels as host loops --------------------------------------- */
namespace refsparse {
struct idx3 {
  unsigned x, y, z;
};
static thread_local idx3 blockDim_, blockIdx_, threadIdx_;
#define blockDim refsparse::blockDim_
#define blockIdx refsparse::blockIdx_
#define threadIdx refsparse::threadIdx_
#undef __global__
#define __global__ static
#undef __shared__
#define __shared__ static thread_local
#include "ref_sparse_kernels.inc" /* generated by build_ref.sh from compression.cu */
#undef blockDim
#undef blockIdx
#undef threadIdx
template <class F>
static void launch(int grid, int block, F body) {
  blockDim_ = {(unsigned)block, 1, 1};
  for (int b = 0; b < grid; b++)
    for (int t = 0; t < block; t++) {
      blockIdx_ = {(unsigned)b, 0, 0};
      threadIdx_ = {(unsigned)t, 0, 0};
      body();
    }
}
}  // namespace refsparse

extern "C" {

void ref_asis_encode_block(float* fblock, int dims, int maxbits, unsigned block_idx, unsigned long long* stream) {
  if (dims == 3) asis_encode<64>(fblock, maxbits, block_idx, stream);
  else if (dims == 2) asis_encode<16>(fblock, maxbits, block_idx, stream);
  else asis_encode<4>(fblock, maxbits, block_idx, stream);
}
void ref_asis_decode_block(unsigned long long* stream, int dims, int maxbits, unsigned block_idx, float* fblock) {
  if (dims == 3) asis_decode<64>(stream, maxbits, block_idx, fblock);
  else if (dims == 2) asis_decode<16>(stream, maxbits, block_idx, fblock);
  else asis_decode<4>(stream, maxbits, block_idx, fblock);
}
void ref_bs_encode_block(float* fblock, int dims, int maxbits, size_t block_idx, void* buf, size_t bytes) {
  if (dims == 3) bs_encode<64>(fblock, maxbits, block_idx, buf, bytes);
  else if (dims == 2) bs_encode<16>(fblock, maxbits, block_idx, buf, bytes);
  else bs_encode<4>(fblock, maxbits, block_idx, buf, bytes);
}
void ref_bs_decode_block(void* buf, size_t bytes, int dims, int maxbits, size_t block_idx, float* fblock) {
  if (dims == 3) bs_decode<64>(buf, bytes, maxbits, block_idx, fblock);
  else if (dims == 2) bs_decode<16>(buf, bytes, maxbits, block_idx, fblock);
  else bs_decode<4>(buf, bytes, maxbits, block_idx, fblock);
}
const unsigned char* ref_perm3(void) { return cuZFP::perm_3d; }
const unsigned char* ref_perm2(void) { return cuZFP::perm_2; }

void ref_fwd_lift(int* p, int stride) {
  if (stride == 1) cuZFP::fwd_lift<int, 1>(p);
  else if (stride == 4) cuZFP::fwd_lift<int, 4>(p);
  else cuZFP::fwd_lift<int, 16>(p);
}
void ref_inv_lift(int* p, int stride) {
  if (stride == 1) cuZFP::inv_lift<int, 1>(p);
  else if (stride == 4) cuZFP::inv_lift<int, 4>(p);
  else cuZFP::inv_lift<int, 16>(p);
}

/* the call sequence of Execution.h:88-95 and the (absent) swap-in caller */
int ref_sparse_compress(float* in, int n, int dimsize, int blocksize, int* begin, uint32_t* bitmap, float* values) {
  int P = dimsize * blocksize;
  refsparse::launch(dimsize, blocksize, [&] { refsparse::PreGPUcompression(n, P, in, begin); });
  int kernel_size = (int)ceil(float(n) / ceil(float(n) / P));
  int num = 0;
  refsparse::launch(1, 1, [&] { refsparse::PreAcc(begin, kernel_size, &num); });
  refsparse::launch(dimsize, blocksize, [&] { refsparse::GPUcompression(n, P, in, values, begin, bitmap); });
  return num;
}
void ref_sparse_decompress(float* values, float* out, int n, int dimsize, int blocksize, uint32_t* bitmap, int* begin) {
  int P = dimsize * blocksize;
  refsparse::launch(dimsize, blocksize, [&] { refsparse::GPUdecompression(values, out, n, P, bitmap, begin); });
}
}
