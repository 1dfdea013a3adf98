// CUDA kernels of the fixed-rate ZFP float32 codec for sm_100a.
//
// Replaces cuZFP::cudaEncode / cudaDecode3 and their launchers
// (CSWAP+/zfp/encode3.cuh:49-186, decode3.cuh:42-178, encode1/2.cuh,
// decode1/2.cuh).  Two families:
//
//  * slab kernels for the swap path's view (nx = ny = 32, contiguous, whole
//    32-bit words per block): one CTA per group of 8 z-slabs (32 KiB, 128
//    blocks), four (encoder) or five (decoder) CTAs per SM, lane = zfp block
//    held in registers.  A lane moves its block with sixteen 128-bit accesses
//    (eight neighbouring lanes cover one 128-byte row segment, so a warp
//    access touches four whole lines); stream words sit word-major in shared
//    memory (bank = lane, so diverged lanes never conflict) and each lane
//    reads or writes its own 128-bit pieces of the stream.  After the lookup
//    table is in place no warp waits for another.
//    Measured against a persistent variant that pulled each group with a bulk
//    async copy into a shared tile and wrote the stream through a transposing
//    copy-out: the extra shared-memory hop, its barriers and the registers of
//    the persistent loop cost 40 % at 256 MiB (177 against 125 us).  A second
//    persistent encoder, whose lanes fetched their next block with 16-byte
//    asynchronous copies into slots of their own while coding (no barrier),
//    took 168 us (32 KB more shared memory per CTA, 196 bytes of spills, and
//    the CTAs of an SM marching through the same phase together); asking L2
//    for the successor CTA's lines ahead of time cost 3 % in either kernel.
//  * generic kernels, one thread per block straight from/to global memory, for
//    any 1-D/2-D/3-D extents, strides, partial blocks and bit budgets.
//
// No kernel here waits on another CTA, a flag or a copy engine.
#include <cuda_runtime.h>

#include <cstdint>

#include "zfp_field.cuh"
#include "zfp_kernels.h"

namespace csw {

namespace {

constexpr int kThreads = 128;                  // zfp blocks (lanes) per CTA
constexpr int kSlabFloats = 1024;              // one 32x32 z-slab
constexpr int kGroupSlabs = kThreads / 16;      // z-slabs per CTA: kThreads / 64 tiles of four
constexpr int kEncCtasPerSm = 4;                // 128 registers per thread: the encoder needs 122
constexpr int kDecCtasPerSm = 5;                // 96 registers: the decoder fits without spills, and a fifth
                                                // CTA hides more of its dependent shared-memory reads

// ---- word staging: word w of the block owned by thread t lives at [w * kThreads + t] --
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

// The expansion table, evaluated at compile time: a CTA copies it to shared
// memory (two words per thread) instead of computing 256 entries per launch.
struct EncTable {
  uint32_t v[ENC_LUT_SIZE];
};
constexpr EncTable make_enc_table() {
  EncTable t{};
  for (int i = 0; i < ENC_LUT_SIZE; i++) t.v[i] = enc_lut_entry((uint32_t)i);
  return t;
}
__device__ const EncTable g_enc_table = make_enc_table();

// z-slab that feeds row z of a block with vz valid slabs (encode.cuh:17-38
// applied along z: a,a,a,a / a,b,b,a / a,b,c,a)
__device__ __forceinline__ int pad_src_z(int z, int vz) { return z < vz ? z : (z == 3 ? 0 : vz - 1); }

}  // namespace

// =====================================================================================
// slab encoder
// =====================================================================================
// One CTA per group of 8 z-slabs (128 blocks, lane = block).  A lane reads its
// 4x4x4 block with sixteen 128-bit loads (eight neighbouring lanes cover one
// 128-byte row segment, so a warp load touches four full lines), codes it into
// its own column of the word-major staging area and writes its own words out:
// after the table is built no warp waits for another.
__global__ void __launch_bounds__(kThreads, kEncCtasPerSm)
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
  const uint32_t zt = (blockIdx.x * (kThreads / 64) + t) * 4;  // first slab of my tile
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
  for (int i = tid; i < ENC_LUT_SIZE; i += kThreads) lut[i] = __ldg(g_enc_table.v + i);
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
namespace {
// The parser table, evaluated at compile time: a CTA copies it to shared memory
// with four 128-bit loads per thread instead of rebuilding 4096 entries.
struct DecTable {
  uint32_t v[DEC_LUT_SIZE];
};
constexpr DecTable make_dec_table() {
  DecTable t{};
  for (int i = 0; i < DEC_LUT_SIZE; i++) t.v[i] = dec_lut_entry(i);
  return t;
}
__device__ const DecTable g_dec_table = make_dec_table();
static_assert(DEC_LUT_SIZE % (4 * kThreads) == 0, "table copy assumes whole 128-bit rounds");
}  // namespace

// One CTA per group of 8 z-slabs, lane = block, mirror image of the encoder: a
// lane pulls its own compressed words into its column of the word-major staging
// area, parses them by bit position and stores the rebuilt 4x4x4 block with
// sixteen 128-bit stores.  The only barrier is the one after the table copy.
__global__ void __launch_bounds__(kThreads, kDecCtasPerSm)
zfp_decode_slab_kernel(const uint32_t* __restrict__ in, float* __restrict__ out, uint32_t nz, int maxbits,
                       const PipeConsts kc) {
  extern __shared__ __align__(16) uint32_t smem_words[];
  const int nwords = maxbits >> 5;
  uint32_t* stage = smem_words;
  uint32_t* lut = stage + (nwords + STAGE_SPARE_ROWS) * kThreads;

  const int tid = threadIdx.x;
  const int t = tid >> 6, bx = tid & 7, by = (tid >> 3) & 7;
  const uint32_t zt = (blockIdx.x * (kThreads / 64) + t) * 4;  // first slab of my tile
  uint32_t* col = stage + tid;
  if (zt < nz) {
    const uint32_t* src = in + ((size_t)blockIdx.x * kThreads + tid) * nwords;
    if ((nwords & 3) == 0) {
      for (int w = 0; w < nwords; w += 4) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + w));
        col[w * kThreads] = v.x;
        col[(w + 1) * kThreads] = v.y;
        col[(w + 2) * kThreads] = v.z;
        col[(w + 3) * kThreads] = v.w;
      }
    } else {
      for (int w = 0; w < nwords; w++) col[w * kThreads] = __ldg(src + w);
    }
  }
  // reads just past a block find zeros and need no bounds test
  for (int w = nwords; w < nwords + STAGE_SPARE_ROWS; w++) col[w * kThreads] = 0u;
#pragma unroll
  for (int i = 0; i < DEC_LUT_SIZE / (4 * kThreads); i++)
    reinterpret_cast<uint4*>(lut)[i * kThreads + tid] =
        __ldg(reinterpret_cast<const uint4*>(g_dec_table.v) + i * kThreads + tid);
  __syncthreads();  // the table is complete
  if (zt >= nz) return;

  float f[64];
  StageWords source{col};
  decode_block3_pos(source, maxbits, f, lut, kc);
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
  for (int i = threadIdx.x; i < ENC_LUT_SIZE; i += blockDim.x) lut[i] = __ldg(g_enc_table.v + i);
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
  for (int i = threadIdx.x; i < DEC_LUT_SIZE; i += blockDim.x) lut[i] = __ldg(g_dec_table.v + i);
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
constexpr size_t kDefaultDynamicSmem = 48 * 1024;  // what a kernel may ask for without opting in
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

cudaError_t zfp_encode_launch(const FieldGeom& g, const float* in, void* out, int maxbits, cudaStream_t stream) {
  const uint64_t nblocks = geom_blocks(g);
  if (nblocks == 0) return cudaSuccess;
  if (zfp_slab_eligible(g, in, out, maxbits)) {
    const size_t smem = slab_smem_bytes(maxbits, false);
    if (smem > kDefaultDynamicSmem) {  // only the largest budgets: the call costs host time on every launch
      cudaError_t e = cudaFuncSetAttribute(zfp_encode_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)slab_smem_bytes(2048, false));
      if (e != cudaSuccess) return e;
    }
    const uint32_t ngroups = (g.nz + kGroupSlabs - 1) / kGroupSlabs;
    zfp_encode_slab_kernel<<<ngroups, kThreads, smem, stream>>>(in, reinterpret_cast<uint32_t*>(out), g.nz, maxbits,
                                                               pipe_consts());
    return cudaGetLastError();
  }
  if (maxbits & 31) {
    cudaError_t e = cudaMemsetAsync(out, 0, stream_bytes(g, (unsigned)maxbits), stream);
    if (e != cudaSuccess) return e;
  } else if ((nblocks * (uint64_t)maxbits) & 63) {
    // whole 32-bit words per block but an odd number of them in total: the
    // stream is sized in 64-bit words, so its last 32 bits belong to no block
    const size_t nbytes = stream_bytes(g, (unsigned)maxbits);
    cudaError_t e = cudaMemsetAsync(static_cast<char*>(out) + nbytes - 8, 0, 8, stream);
    if (e != cudaSuccess) return e;
  }
  const unsigned grid = (unsigned)((nblocks + 127) / 128);
  uint32_t* o = reinterpret_cast<uint32_t*>(out);
  if (g.dims == 3) zfp_encode_generic_kernel<3><<<grid, 128, 0, stream>>>(g, in, o, maxbits, nblocks);
  else if (g.dims == 2) zfp_encode_generic_kernel<2><<<grid, 128, 0, stream>>>(g, in, o, maxbits, nblocks);
  else zfp_encode_generic_kernel<1><<<grid, 128, 0, stream>>>(g, in, o, maxbits, nblocks);
  return cudaGetLastError();
}

cudaError_t zfp_decode_launch(const FieldGeom& g, const void* in, float* out, int maxbits, cudaStream_t stream) {
  const uint64_t nblocks = geom_blocks(g);
  if (nblocks == 0) return cudaSuccess;
  if (zfp_slab_eligible(g, out, in, maxbits)) {
    const size_t smem = slab_smem_bytes(maxbits, true);
    if (smem > kDefaultDynamicSmem) {
      cudaError_t e = cudaFuncSetAttribute(zfp_decode_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)slab_smem_bytes(2048, true));
      if (e != cudaSuccess) return e;
    }
    const uint32_t ngroups = (g.nz + kGroupSlabs - 1) / kGroupSlabs;
    zfp_decode_slab_kernel<<<ngroups, kThreads, smem, stream>>>(reinterpret_cast<const uint32_t*>(in), out, g.nz,
                                                               maxbits, pipe_consts());
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
