// CUDA kernels of the fixed-rate ZFP float32 codec for sm_100a.
//
// Replaces cuZFP::cudaEncode / cudaDecode3 and their launchers
// (CSWAP+/zfp/encode3.cuh:49-186, decode3.cuh:42-178, encode1/2.cuh,
// decode1/2.cuh).  Two families:
//
//  * slab kernels for the swap path's view (nx = ny = 32, contiguous, whole
//    32-bit words per block): persistent CTAs, lane = zfp block, a group of
//    16 z-slabs (64 KiB, 256 blocks) per iteration.  The encoder pulls the
//    group with one bulk async copy (TMA) that lands while the previous group
//    is still being coded out of registers; coded words are staged word-major
//    in shared memory (bank = lane, so diverged lanes never conflict) and
//    leave as 128-bit coalesced stores.  The decoder stages the compressed
//    words the same way, parses them by bit position and stores the rebuilt
//    values straight to global memory (a warp store covers four full lines).
//  * generic kernels, one thread per block straight from/to global memory, for
//    any 1-D/2-D/3-D extents, strides, partial blocks and bit budgets.
//
// Every wait is bounded; a kernel that gives up records CSW_ERR_TIMEOUT in the
// status word it was given and returns with no copy in flight.
#include <cuda_runtime.h>

#include <cstdint>

#include "zfp_field.cuh"
#include "zfp_kernels.h"

namespace csw {

namespace {

constexpr int kThreads = 256;                  // blocks per CTA iteration
constexpr int kSlabFloats = 1024;              // one 32x32 z-slab
constexpr int kGroupSlabs = 16;                // z-slabs per CTA iteration
constexpr int kGroupFloats = kSlabFloats * kGroupSlabs;
constexpr int kGroupBytes = kGroupFloats * 4;  // 64 KiB
constexpr uint32_t kSpinLimit = 1u << 22;

// ---- PTX wrappers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}
// global -> shared bulk async copy, completion counted on the mbarrier
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- word staging: word w of the block owned by thread t lives at [w * 256 + t] -----
struct StageSink {
  uint32_t* p;  // &stage[threadIdx.x]
  __device__ __forceinline__ void put(int w, uint32_t v) { p[w * kThreads] = v; }
};
// Staged stream words of the decoder: rows nwords and nwords + 1 are kept zero
// so that reads just past a block need no bounds test.
struct StageWords {
  const uint32_t* p;  // &stage[threadIdx.x]
  __device__ __forceinline__ uint32_t word(int w) const { return p[w * kThreads]; }
};

// Staged words and the per-lane expansion queue of the staged encoder, both
// word-major so that a warp's lanes always hit 32 different banks.
struct SmemStage {
  uint32_t* p;  // &stage[threadIdx.x]
  uint32_t* q;  // &queue[threadIdx.x]
  __device__ __forceinline__ void or_word(int w, uint32_t v) { atomicOr(p + w * kThreads, v); }
  __device__ __forceinline__ void q_put(int slot, int field, uint32_t v) {
    q[(slot * QUEUE_FIELDS + field) * kThreads] = v;
  }
  __device__ __forceinline__ uint32_t q_get(int slot, int field) const {
    return q[(slot * QUEUE_FIELDS + field) * kThreads];
  }
};

// z-slab that feeds row z of a block with vz valid slabs (encode.cuh:17-38
// applied along z: a,a,a,a / a,b,b,a / a,b,c,a)
__device__ __forceinline__ int pad_src_z(int z, int vz) { return z < vz ? z : (z == 3 ? 0 : vz - 1); }

}  // namespace

// =====================================================================================
// slab encoder
// =====================================================================================
// One CTA per group of 16 z-slabs (256 blocks, lane = block).  A lane reads its
// 4x4x4 block with sixteen 128-bit loads (eight neighbouring lanes cover one
// 128-byte row segment, so a warp load touches four full lines), codes it into
// its own column of the word-major staging area and writes its own words out:
// after the table is built no warp waits for another.
__global__ void __launch_bounds__(kThreads, 2)
zfp_encode_slab_kernel(const float* __restrict__ in, uint32_t* __restrict__ out, uint32_t nz, int maxbits,
                       const PipeConsts kc) {
  extern __shared__ __align__(16) uint32_t smem_words[];
  const int nwords = maxbits >> 5;
  uint32_t* stage = smem_words;
  uint32_t* queue = stage + (nwords + STAGE_SPARE_ROWS) * kThreads;
  uint32_t* lut = queue + QUEUE_SLOTS * QUEUE_FIELDS * kThreads;

  const int tid = threadIdx.x;
  // my block: tile t of the group (4 slabs), block (bx, by) of its 8x8 grid
  const int t = tid >> 6, bx = tid & 7, by = (tid >> 3) & 7;
  const uint32_t zt = (blockIdx.x * 4 + t) * 4;  // first slab of my tile
  const int vz = zt >= nz ? 0 : (nz - zt < 4 ? (int)(nz - zt) : 4);
  float f[64];
  if (vz > 0) {
    const float* my = in + (size_t)zt * kSlabFloats + by * 128 + bx * 4;
#pragma unroll
    for (int z = 0; z < 4; z++) {
      const float* row = my + pad_src_z(z, vz) * kSlabFloats;
#pragma unroll
      for (int y = 0; y < 4; y++) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(row + y * 32));
        f[16 * z + 4 * y + 0] = v.x;
        f[16 * z + 4 * y + 1] = v.y;
        f[16 * z + 4 * y + 2] = v.z;
        f[16 * z + 4 * y + 3] = v.w;
      }
    }
  }
  lut[tid] = enc_lut_entry((uint32_t)tid);
  for (int w = 0; w < nwords; w++) stage[w * kThreads + tid] = 0u;  // coded bits are OR-ed in
  __syncthreads();  // the table is complete
  if (vz == 0) return;

  SmemStage st{stage + tid, queue + tid};
  encode_block3_staged(f, maxbits, st, lut, kc);

  // a lane's words sit in its own column: no barrier before reading them back
  uint32_t* dst = out + ((size_t)blockIdx.x * kThreads + tid) * nwords;
  const uint32_t* col = stage + tid;
  if ((nwords & 3) == 0) {
    for (int w = 0; w < nwords; w += 4)
      *reinterpret_cast<uint4*>(dst + w) = make_uint4(col[w * kThreads], col[(w + 1) * kThreads],
                                                      col[(w + 2) * kThreads], col[(w + 3) * kThreads]);
  } else {
    for (int w = 0; w < nwords; w++) dst[w] = col[w * kThreads];
  }
}

// =====================================================================================
// slab decoder
// =====================================================================================
__global__ void __launch_bounds__(kThreads, 2)
zfp_decode_slab_kernel(const uint32_t* __restrict__ in, float* __restrict__ out, uint32_t nz, int maxbits,
                       int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  uint32_t* stage = reinterpret_cast<uint32_t*>(smem_raw);
  const int nwords = maxbits >> 5;
  uint32_t* lut = stage + (nwords + STAGE_SPARE_ROWS) * kThreads;
  (void)status;

  const int tid = threadIdx.x;
  for (int i = tid; i < DEC_LUT_SIZE; i += kThreads) lut[i] = dec_lut_entry(i);
  for (int w = nwords; w < nwords + STAGE_SPARE_ROWS; w++) stage[w * kThreads + tid] = 0u;

  const uint32_t ngroups = (nz + kGroupSlabs - 1) / kGroupSlabs;
  const int t = tid >> 6, bx = tid & 7, by = (tid >> 3) & 7;

  for (uint32_t g = blockIdx.x; g < ngroups; g += gridDim.x) {
    // stage the group's compressed words, word-major
    const uint32_t tiles = ((nz + 3) >> 2) - g * 4 < 4 ? ((nz + 3) >> 2) - g * 4 : 4;
    const uint32_t nblk = tiles * 64;
    const uint32_t* src = in + (size_t)g * kThreads * nwords;
    if ((nwords & 3) == 0) {
      const uint32_t per = nwords >> 2, chunks = nblk * per;
      for (uint32_t q = tid; q < chunks; q += kThreads) {
        const uint32_t b = q / per, c = q - b * per;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src) + q);
        uint32_t* s = stage + (4 * c) * kThreads + b;
        s[0] = v.x;
        s[kThreads] = v.y;
        s[2 * kThreads] = v.z;
        s[3 * kThreads] = v.w;
      }
    } else {
      const uint32_t words = nblk * nwords;
      for (uint32_t q = tid; q < words; q += kThreads) {
        const uint32_t b = q / nwords, w = q - b * nwords;
        stage[w * kThreads + b] = __ldg(src + q);
      }
    }
    __syncthreads();

    const uint32_t zt = g * kGroupSlabs + t * 4;
    if (zt < nz) {
      float f[64];
      StageWords source{stage + tid};
      decode_block3_pos(source, maxbits, f, lut);
      // eight neighbouring lanes cover one 128-byte row segment, so every store
      // instruction of a warp writes four full lines: no staging of the output
      const int vz = nz - zt < 4 ? (int)(nz - zt) : 4;
      float* dst = out + (size_t)zt * kSlabFloats + by * 128 + bx * 4;
#pragma unroll
      for (int z = 0; z < 4; z++)
        if (z < vz) {
#pragma unroll
          for (int y = 0; y < 4; y++)
            *reinterpret_cast<float4*>(dst + z * kSlabFloats + y * 32) =
                make_float4(f[16 * z + 4 * y], f[16 * z + 4 * y + 1], f[16 * z + 4 * y + 2], f[16 * z + 4 * y + 3]);
        }
    }
    __syncthreads();  // the staged words are free for the next group
  }
}

// =====================================================================================
// generic kernels: one thread per block
// =====================================================================================
namespace {

// Words of block b go to bit offset b * maxbits.  With whole words per block
// they are plain stores; otherwise neighbours share words, the stream is
// zeroed beforehand and words are OR-ed in.
struct GlobalSink {
  uint32_t* out;
  uint64_t bit0;    // first bit of the block
  int maxbits;
  bool aligned;
  __device__ __forceinline__ void put(int w, uint32_t v) {
    const int left = maxbits - 32 * w;
    if (left < 32) v &= (1u << left) - 1u;
    const uint64_t p = bit0 + 32u * (uint32_t)w;
    if (aligned) {
      out[p >> 5] = v;
    } else {
      const uint32_t s = (uint32_t)(p & 31);
      if (v << s) atomicOr(out + (p >> 5), v << s);
      if (s && (v >> (32 - s))) atomicOr(out + (p >> 5) + 1, v >> (32 - s));
    }
  }
};
struct GlobalSource {
  const uint32_t* in;
  uint64_t bit0;
  uint64_t total_words;
  int nwords;
  __device__ __forceinline__ uint32_t get(int w) const {
    if (w >= nwords) return 0u;
    const uint64_t p = bit0 + 32u * (uint32_t)w, i = p >> 5;
    const uint32_t s = (uint32_t)(p & 31);
    uint32_t lo = i < total_words ? in[i] : 0u;
    if (!s) return lo;
    uint32_t hi = i + 1 < total_words ? in[i + 1] : 0u;
    return (lo >> s) | (hi << (32 - s));
  }
};

template <int DIMS>
__global__ void __launch_bounds__(128)
zfp_encode_generic_kernel(FieldGeom g, const float* __restrict__ in, uint32_t* __restrict__ out, int maxbits,
                          uint64_t nblocks) {
  __shared__ uint32_t lut[ENC_LUT_SIZE];
  for (int i = threadIdx.x; i < ENC_LUT_SIZE; i += blockDim.x) lut[i] = enc_lut_entry((uint32_t)i);
  __syncthreads();
  const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  float f[1 << (2 * DIMS)];
  gather_block<DIMS>(g, in, b, f);
  GlobalSink sink{out, b * (uint64_t)maxbits, maxbits, (maxbits & 31) == 0};
  encode_block<DIMS>(f, maxbits, sink, lut);
}

template <int DIMS>
__global__ void __launch_bounds__(128)
zfp_decode_generic_kernel(FieldGeom g, const uint32_t* __restrict__ in, float* __restrict__ out, int maxbits,
                          uint64_t nblocks, uint64_t total_words) {
  __shared__ uint32_t lut[DEC_LUT_SIZE];
  for (int i = threadIdx.x; i < DEC_LUT_SIZE; i += blockDim.x) lut[i] = dec_lut_entry(i);
  __syncthreads();
  const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  float f[1 << (2 * DIMS)];
  GlobalSource source{in, b * (uint64_t)maxbits, total_words, (maxbits + 31) >> 5};
  decode_block<DIMS>(source, maxbits, f, lut);
  scatter_block<DIMS>(g, out, b, f);
}

}  // namespace

// =====================================================================================
// launchers
// =====================================================================================
static size_t slab_smem_bytes(int maxbits, bool decode) {
  if (decode)
    return (size_t)((maxbits >> 5) + STAGE_SPARE_ROWS) * kThreads * 4 + DEC_LUT_SIZE * 4;
  return (size_t)((maxbits >> 5) + STAGE_SPARE_ROWS + QUEUE_SLOTS * QUEUE_FIELDS) * kThreads * 4 + ENC_LUT_SIZE * 4;
}

bool zfp_slab_eligible(const FieldGeom& g, const void* field, const void* stream, int maxbits) {
  return g.dims == 3 && g.nx == 32 && g.ny == 32 && g.sx == 1 && g.sy == 32 && g.sz == 1024 && (maxbits & 31) == 0 &&
         maxbits >= 32 && maxbits <= 2048 && (reinterpret_cast<uintptr_t>(field) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(stream) & 15) == 0;
}

static int slab_grid(uint32_t nz, int ctas_per_sm_times_sms) {
  const uint32_t ngroups = (nz + kGroupSlabs - 1) / kGroupSlabs;
  return (int)(ngroups < (uint32_t)ctas_per_sm_times_sms ? ngroups : (uint32_t)ctas_per_sm_times_sms);
}

cudaError_t zfp_encode_launch(const FieldGeom& g, const float* in, void* out, int maxbits, int sm_count, int* d_status,
                              cudaStream_t stream) {
  const uint64_t nblocks = geom_blocks(g);
  if (nblocks == 0) return cudaSuccess;
  if (zfp_slab_eligible(g, in, out, maxbits)) {
    const size_t smem = slab_smem_bytes(maxbits, false);
    cudaError_t e = cudaFuncSetAttribute(zfp_encode_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)slab_smem_bytes(2048, false));
    if (e != cudaSuccess) return e;
    const uint32_t ngroups = (g.nz + kGroupSlabs - 1) / kGroupSlabs;
    zfp_encode_slab_kernel<<<ngroups, kThreads, smem, stream>>>(in, reinterpret_cast<uint32_t*>(out), g.nz, maxbits,
                                                               pipe_consts());
    return cudaGetLastError();
  }
  if (maxbits & 31) {
    cudaError_t e = cudaMemsetAsync(out, 0, stream_bytes(g, (unsigned)maxbits), stream);
    if (e != cudaSuccess) return e;
  }
  const unsigned grid = (unsigned)((nblocks + 127) / 128);
  uint32_t* o = reinterpret_cast<uint32_t*>(out);
  if (g.dims == 3) zfp_encode_generic_kernel<3><<<grid, 128, 0, stream>>>(g, in, o, maxbits, nblocks);
  else if (g.dims == 2) zfp_encode_generic_kernel<2><<<grid, 128, 0, stream>>>(g, in, o, maxbits, nblocks);
  else zfp_encode_generic_kernel<1><<<grid, 128, 0, stream>>>(g, in, o, maxbits, nblocks);
  return cudaGetLastError();
}

cudaError_t zfp_decode_launch(const FieldGeom& g, const void* in, float* out, int maxbits, int sm_count, int* d_status,
                              cudaStream_t stream) {
  const uint64_t nblocks = geom_blocks(g);
  if (nblocks == 0) return cudaSuccess;
  if (zfp_slab_eligible(g, out, in, maxbits)) {
    const size_t smem = slab_smem_bytes(maxbits, true);
    cudaError_t e = cudaFuncSetAttribute(zfp_decode_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)slab_smem_bytes(2048, true));
    if (e != cudaSuccess) return e;
    zfp_decode_slab_kernel<<<slab_grid(g.nz, 2 * sm_count), kThreads, smem, stream>>>(
        reinterpret_cast<const uint32_t*>(in), out, g.nz, maxbits, d_status);
    return cudaGetLastError();
  }
  const unsigned grid = (unsigned)((nblocks + 127) / 128);
  const uint32_t* i32 = reinterpret_cast<const uint32_t*>(in);
  const uint64_t total_words = stream_bytes(g, (unsigned)maxbits) / 4;
  if (g.dims == 3) zfp_decode_generic_kernel<3><<<grid, 128, 0, stream>>>(g, i32, out, maxbits, nblocks, total_words);
  else if (g.dims == 2) zfp_decode_generic_kernel<2><<<grid, 128, 0, stream>>>(g, i32, out, maxbits, nblocks, total_words);
  else zfp_decode_generic_kernel<1><<<grid, 128, 0, stream>>>(g, i32, out, maxbits, nblocks, total_words);
  return cudaGetLastError();
}

}  // namespace csw
