// CUDA kernels of the zero-value ("ZVC") sparse codec for sm_100a.
//
// Replaces PreGPUcompression / PreAcc / GPUcompression / GPUdecompression of
// CSWAP+/zfp/compression.cu:9-19,134-318.  The reference gives each of 16384
// threads a contiguous chunk (stride-`chunk` loads, a one-thread serial scan
// and a blocking 4-byte copy to size the output).  Here:
//
//  native format  - bitmap[ceil(n/32)] in element order built by warp ballots
//                   from coalesced loads, values[nnz] in element order, and an
//                   exclusive per-tile (4096 elements) offset table so that
//                   decompression is independent per tile.  A value is kept
//                   when its BIT PATTERN is non-zero, so -0.0 and NaN payloads
//                   round-trip exactly.
//  count -> scan -> pack, three launches, no inter-CTA waiting; the total is
//                   written to a caller-supplied word (device or mapped host).
//  single pass    - same bitmap and per-tile contents from one read of the
//                   tensor; tiles claim their segments with an atomic add, so
//                   segment order follows the schedule, not the element order.
//  legacy format  - the reference's `begin | bitmap | values` layout with its
//                   P-worker chunking, one warp per worker, behind the
//                   reference's own entry-point names.
#include <cuda_runtime.h>

#include <cstdint>

#include "sparse_kernels.h"

namespace csw {

namespace {

constexpr int kTile = SPARSE_TILE;        // elements per tile
constexpr int kThreads = 256;             // 8 warps, 512 elements (16 bitmap words) each
constexpr int kWordsPerWarp = kTile / 32 / (kThreads / 32);  // 16

__device__ __forceinline__ uint32_t lanemask_lt() {
  uint32_t m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// ---- pass 1: bitmap + per-tile counts ---------------------------------------------
__global__ void __launch_bounds__(kThreads)
sparse_count_kernel(const uint32_t* __restrict__ in, uint64_t n, uint32_t* __restrict__ bitmap,
                    uint32_t* __restrict__ tile_cnt) {
  __shared__ uint32_t warp_cnt[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint64_t base = (uint64_t)blockIdx.x * kTile + (uint64_t)warp * (kWordsPerWarp * 32);
  uint32_t v[kWordsPerWarp];
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    const uint64_t i = base + j * 32 + lane;
    v[j] = i < n ? __ldg(in + i) : 0u;
  }
  uint32_t mine = 0, cnt = 0;
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    const uint32_t w = __ballot_sync(0xffffffffu, v[j] != 0u);
    cnt += __popc(w);
    if (lane == j) mine = w;
  }
  const uint64_t word0 = base >> 5, nwords = (n + 31) >> 5;
  if (lane < kWordsPerWarp && word0 + lane < nwords) bitmap[word0 + lane] = mine;
  if (lane == 0) warp_cnt[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t s = 0;
#pragma unroll
    for (int i = 0; i < kThreads / 32; i++) s += warp_cnt[i];
    tile_cnt[blockIdx.x] = s;
  }
}

// ---- pass 2: exclusive scan of the tile counts (one CTA) --------------------------
// One CTA of 1024 threads scans `len` counts: off[i] = sum of cnt[0 .. i-1], the
// total to *total.  cnt and off may be the same array (each thread reads its own
// element before it writes it), which is how the in-place callers use it.
template <class T>
__global__ void __launch_bounds__(1024)
block_exclusive_scan_kernel(const T* cnt, T* off, uint32_t len, T* __restrict__ total) {
  __shared__ T warp_sum[32];
  __shared__ T carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (uint32_t base = 0; base < len; base += 1024) {
    const uint32_t i = base + threadIdx.x;
    const T c = i < len ? cnt[i] : T(0);
    T x = c;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const T y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) warp_sum[warp] = x;
    __syncthreads();
    if (warp == 0) {
      T s = warp_sum[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const T y = __shfl_up_sync(0xffffffffu, s, d);
        if (lane >= d) s += y;
      }
      warp_sum[lane] = s;  // inclusive
    }
    __syncthreads();
    const T carry = carry_s;
    if (i < len) off[i] = carry + (warp ? warp_sum[warp - 1] : T(0)) + x - c;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + warp_sum[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) *total = carry_s;
}

// ---- pass 3: pack the non-zeros ----------------------------------------------------
__global__ void __launch_bounds__(kThreads)
sparse_pack_kernel(const uint32_t* __restrict__ in, uint64_t n, const uint32_t* __restrict__ tile_off,
                   uint32_t* __restrict__ values) {
  __shared__ uint32_t warp_cnt[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint64_t base = (uint64_t)blockIdx.x * kTile + (uint64_t)warp * (kWordsPerWarp * 32);
  uint32_t v[kWordsPerWarp], w[kWordsPerWarp];
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    const uint64_t i = base + j * 32 + lane;
    v[j] = i < n ? __ldg(in + i) : 0u;
  }
  uint32_t cnt = 0;
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    w[j] = __ballot_sync(0xffffffffu, v[j] != 0u);
    cnt += __popc(w[j]);
  }
  if (lane == 0) warp_cnt[warp] = cnt;
  __syncthreads();
  uint32_t off = tile_off[blockIdx.x];
  for (int i = 0; i < warp; i++) off += warp_cnt[i];
  const uint32_t lt = lanemask_lt();
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    if (v[j] != 0u) values[off + __popc(w[j] & lt)] = v[j];
    off += __popc(w[j]);
  }
}

// ---- single pass: tiles claim their value segments from a cursor ---------------------
// Reads the tensor once.  A tile counts its non-zeros, claims that many slots
// with one atomic add on `cursor` (which must be zero at launch and holds the
// total afterwards) and records where its segment starts in tile_off; bitmap
// and per-tile contents are the same as the three-pass result, but segments
// sit in the order the tiles claimed them, so the values array (not what
// decompression returns) can differ from run to run.  No CTA waits for another.
__global__ void __launch_bounds__(kThreads)
sparse_onepass_kernel(const uint32_t* __restrict__ in, uint64_t n, uint32_t* __restrict__ bitmap,
                      uint32_t* __restrict__ tile_off, uint32_t* __restrict__ values, uint32_t* __restrict__ cursor) {
  __shared__ uint32_t warp_cnt[kThreads / 32];
  __shared__ uint32_t tile_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint64_t base = (uint64_t)blockIdx.x * kTile + (uint64_t)warp * (kWordsPerWarp * 32);
  uint32_t v[kWordsPerWarp], w[kWordsPerWarp];
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    const uint64_t i = base + j * 32 + lane;
    v[j] = i < n ? __ldg(in + i) : 0u;
  }
  uint32_t mine = 0, cnt = 0;
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    w[j] = __ballot_sync(0xffffffffu, v[j] != 0u);
    cnt += __popc(w[j]);
    if (lane == j) mine = w[j];
  }
  const uint64_t word0 = base >> 5, nwords = (n + 31) >> 5;
  if (lane < kWordsPerWarp && word0 + lane < nwords) bitmap[word0 + lane] = mine;
  if (lane == 0) warp_cnt[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t total = 0;
#pragma unroll
    for (int i = 0; i < kThreads / 32; i++) total += warp_cnt[i];
    const uint32_t at = atomicAdd(cursor, total);
    tile_off[blockIdx.x] = at;
    tile_base = at;
  }
  __syncthreads();
  uint32_t off = tile_base;
  for (int i = 0; i < warp; i++) off += warp_cnt[i];
  const uint32_t lt = lanemask_lt();
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    if (v[j] != 0u) values[off + __popc(w[j] & lt)] = v[j];
    off += __popc(w[j]);
  }
}

// ---- decompression -----------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
sparse_unpack_kernel(const uint32_t* __restrict__ bitmap, const uint32_t* __restrict__ values,
                     const uint32_t* __restrict__ tile_off, uint64_t n, uint32_t* __restrict__ out) {
  __shared__ uint32_t warp_cnt[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint64_t base = (uint64_t)blockIdx.x * kTile + (uint64_t)warp * (kWordsPerWarp * 32);
  const uint64_t word0 = base >> 5, nwords = (n + 31) >> 5;
  const uint32_t mine = (lane < kWordsPerWarp && word0 + lane < nwords) ? __ldg(bitmap + word0 + lane) : 0u;
  // exclusive prefix of the popcounts of this warp's 16 words
  uint32_t x = __popc(mine);
  const uint32_t c = x;
#pragma unroll
  for (int d = 1; d < kWordsPerWarp; d <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  if (lane == kWordsPerWarp - 1) warp_cnt[warp] = x;
  __syncthreads();
  uint32_t off = tile_off[blockIdx.x];
  for (int i = 0; i < warp; i++) off += warp_cnt[i];
  const uint32_t my_off = off + x - c;
  const uint32_t lt = lanemask_lt();
  // three separate sweeps so that all sixteen gathers of a thread are in flight
  // together (the warp shuffles would otherwise pin each load to its store)
  uint32_t src[kWordsPerWarp];  // index of my value, or ~0 when my element is zero
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    const uint32_t w = __shfl_sync(0xffffffffu, mine, j);
    const uint32_t o = __shfl_sync(0xffffffffu, my_off, j);
    src[j] = ((w >> lane) & 1u) ? o + __popc(w & lt) : 0xffffffffu;
  }
  uint32_t val[kWordsPerWarp];
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) val[j] = src[j] != 0xffffffffu ? __ldg(values + src[j]) : 0u;
#pragma unroll
  for (int j = 0; j < kWordsPerWarp; j++) {
    const uint64_t i = base + j * 32 + lane;
    if (i < n) out[i] = val[j];
  }
}

// ---- reference layout: one warp per worker ------------------------------------------
// Worker i owns elements [i*chunk, min((i+1)*chunk, n)); non-zero test is the
// float comparison of compression.cu:158,220 (-0.0 dropped, NaN kept).
__device__ __forceinline__ bool legacy_nz(uint32_t bits) { return __uint_as_float(bits) != 0.0f; }

__global__ void __launch_bounds__(kThreads)
legacy_count_kernel(const uint32_t* __restrict__ in, int n, int chunk, int workers, int* __restrict__ count) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (i >= workers) return;
  const long long lo = (long long)chunk * i;
  if (lo >= n) return;  // compression.cu:149: such workers leave their slot untouched
  const long long hi = lo + chunk < n ? lo + chunk : n;
  int cnt = 0;
  for (long long p = lo; p < hi; p += 32) {
    const bool nz = p + lane < hi && legacy_nz(__ldg(in + p + lane));
    cnt += __popc(__ballot_sync(0xffffffffu, nz));
  }
  if (lane == 0) count[i] = cnt;
}

__global__ void __launch_bounds__(kThreads)
legacy_pack_kernel(const uint32_t* __restrict__ in, int n, int chunk, int workers, uint32_t* __restrict__ values,
                   const int* __restrict__ begin, uint32_t* __restrict__ bitmap) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (i >= workers) return;
  const long long lo = (long long)chunk * i;
  if (lo >= n) return;
  const long long hi = lo + chunk < n ? lo + chunk : n;
  const int words_per = (chunk + 31) / 32;
  int off = begin[i];
  uint32_t* bm = bitmap + (long long)i * words_per;
  const uint32_t lt = lanemask_lt();
  for (long long p = lo; p < hi; p += 32, bm++) {
    const uint32_t v = p + lane < hi ? __ldg(in + p + lane) : 0u;
    const bool nz = p + lane < hi && legacy_nz(v);
    const uint32_t w = __ballot_sync(0xffffffffu, nz);
    if (nz) values[off + __popc(w & lt)] = v;
    off += __popc(w);
    if (lane == 0) *bm = w;
  }
}

// compression.cu:241-318: positions after the last set bit of a bitmap word
// are left untouched.
__global__ void __launch_bounds__(kThreads)
legacy_unpack_kernel(const uint32_t* __restrict__ values, uint32_t* __restrict__ out, int n, int chunk, int workers,
                     const uint32_t* __restrict__ bitmap, const int* __restrict__ begin) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (i >= workers) return;
  const long long lo = (long long)chunk * i;
  if (lo >= n) return;
  const int words_per = (chunk + 31) / 32;
  const uint32_t* bm = bitmap + (long long)i * words_per;
  int off = begin[i];
  const uint32_t lt = lanemask_lt();
  for (int k = 0; k < words_per; k++) {
    const uint32_t w = __ldg(bm + k);
    const int written = 32 - __clz((int)w);  // 0 when the word is empty
    const long long p = lo + 32LL * k + lane;
    if (lane < written && p < n) out[p] = ((w >> lane) & 1u) ? __ldg(values + off + __popc(w & lt)) : 0u;
    off += __popc(w);
  }
}

}  // namespace

// =====================================================================================
// launchers
// =====================================================================================
cudaError_t sparse_compress_launch(const float* in, uint64_t n, uint32_t* bitmap, float* values, uint32_t* tile_off,
                                   uint32_t* nnz_out, cudaStream_t stream) {
  const uint32_t ntiles = (uint32_t)((n + kTile - 1) / kTile);
  if (ntiles) {
    sparse_count_kernel<<<ntiles, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(in), n, bitmap, tile_off);
  }
  block_exclusive_scan_kernel<uint32_t><<<1, 1024, 0, stream>>>(tile_off, tile_off, ntiles, nnz_out);
  if (ntiles) {
    sparse_pack_kernel<<<ntiles, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(in), n, tile_off,
                                                        reinterpret_cast<uint32_t*>(values));
  }
  return cudaGetLastError();
}

cudaError_t sparse_compress_scratch_launch(const float* in, uint64_t n, uint32_t* bitmap, float* values,
                                           uint32_t* tile_off, uint32_t* tile_cnt_scratch, uint32_t* nnz_out,
                                           cudaStream_t stream) {
  const uint32_t ntiles = (uint32_t)((n + kTile - 1) / kTile);
  if (ntiles) {
    sparse_count_kernel<<<ntiles, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(in), n, bitmap,
                                                         tile_cnt_scratch);
  }
  block_exclusive_scan_kernel<uint32_t><<<1, 1024, 0, stream>>>(tile_cnt_scratch, tile_off, ntiles, nnz_out);
  if (ntiles) {
    sparse_pack_kernel<<<ntiles, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(in), n, tile_off,
                                                        reinterpret_cast<uint32_t*>(values));
  }
  return cudaGetLastError();
}

cudaError_t sparse_compress_onepass_launch(const float* in, uint64_t n, uint32_t* bitmap, float* values,
                                           uint32_t* tile_off, uint32_t* nnz_out, cudaStream_t stream) {
  const uint32_t ntiles = (uint32_t)((n + kTile - 1) / kTile);
  cudaError_t e = cudaMemsetAsync(nnz_out, 0, sizeof(uint32_t), stream);  // the cursor, then the total
  if (e != cudaSuccess || !ntiles) return e;
  sparse_onepass_kernel<<<ntiles, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(in), n, bitmap, tile_off,
                                                         reinterpret_cast<uint32_t*>(values), nnz_out);
  return cudaGetLastError();
}

cudaError_t sparse_decompress_launch(const uint32_t* bitmap, const float* values, const uint32_t* tile_off, uint64_t n,
                                     float* out, cudaStream_t stream) {
  const uint32_t ntiles = (uint32_t)((n + kTile - 1) / kTile);
  if (!ntiles) return cudaSuccess;
  sparse_unpack_kernel<<<ntiles, kThreads, 0, stream>>>(bitmap, reinterpret_cast<const uint32_t*>(values), tile_off, n,
                                                        reinterpret_cast<uint32_t*>(out));
  return cudaGetLastError();
}

static int ceil_div_i(int a, int b) { return a % b == 0 ? a / b : a / b + 1; }

cudaError_t legacy_count_launch(int n, int workers, const float* in, int* count, cudaStream_t stream) {
  if (n <= 0 || workers <= 0) return cudaSuccess;
  const int chunk = ceil_div_i(n, workers);
  legacy_count_kernel<<<(workers + 7) / 8, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(in), n, chunk,
                                                                  workers, count);
  return cudaGetLastError();
}
cudaError_t legacy_scan_launch(int* idx, int len, int* num, cudaStream_t stream) {
  if (len <= 0) return cudaSuccess;
  // in-place scan of the first `len` counts, total to num[0] (compression.cu:9-19)
  block_exclusive_scan_kernel<int><<<1, 1024, 0, stream>>>(idx, idx, (uint32_t)len, num);
  return cudaGetLastError();
}
cudaError_t legacy_pack_launch(int n, int workers, const float* in, float* values, const int* begin, uint32_t* bitmap,
                               cudaStream_t stream) {
  if (n <= 0 || workers <= 0) return cudaSuccess;
  const int chunk = ceil_div_i(n, workers);
  legacy_pack_kernel<<<(workers + 7) / 8, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(in), n, chunk,
                                                                 workers, reinterpret_cast<uint32_t*>(values), begin,
                                                                 bitmap);
  return cudaGetLastError();
}
cudaError_t legacy_unpack_launch(const float* values, float* out, int n, int workers, const uint32_t* bitmap,
                                 const int* begin, cudaStream_t stream) {
  if (n <= 0 || workers <= 0) return cudaSuccess;
  const int chunk = ceil_div_i(n, workers);
  legacy_unpack_kernel<<<(workers + 7) / 8, kThreads, 0, stream>>>(reinterpret_cast<const uint32_t*>(values),
                                                                   reinterpret_cast<uint32_t*>(out), n, chunk, workers,
                                                                   bitmap, begin);
  return cudaGetLastError();
}

}  // namespace csw
