// C ABI of the codecs: argument checking, geometry, launches.
// Declarations and the reference interfaces they replace: include/cswap_b200.h,
// include/cswap_compat.h.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/cswap_b200.h"
#include "../../include/cswap_compat.h"
#include "internal.h"
#include "sparse_kernels.h"
#include "zfp_kernels.h"

namespace csw {

thread_local int tl_cuda_error = 0;

csw_status cuda_fail(cudaError_t e) {
  tl_cuda_error = (int)e;
  return CSW_ERR_CUDA;
}

// ---- per-device state: SM count and the device status word ----------------------
namespace {
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int* d_status = nullptr;  // one int, zero when healthy
};
constexpr int kMaxDevices = 64;
DeviceState g_dev[kMaxDevices];
std::mutex g_dev_mu;
}  // namespace

csw_status device_state(int* sm_count, int** d_status) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DeviceState& s = g_dev[dev];
  if (!s.ready) {
    e = cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaMalloc(&s.d_status, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaMemset(s.d_status, 0, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e);
    s.ready = true;
  }
  if (sm_count) *sm_count = s.sm_count;
  if (d_status) *d_status = s.d_status;
  return CSW_OK;
}

static bool valid_maxbits(unsigned maxbits) {
  // 9 header bits must fit (below that the reference overruns the block,
  // encode.cuh:360-366); 64 planes of 64 bits plus group tests bound the top
  return maxbits >= 9 && maxbits <= 4096;
}

}  // namespace csw

using namespace csw;

extern "C" {

const char* csw_status_string(csw_status s) {
  switch (s) {
    case CSW_OK: return "ok";
    case CSW_ERR_ARG: return "bad argument";
    case CSW_ERR_SIZE: return "output capacity too small";
    case CSW_ERR_CUDA: return "CUDA runtime error";
    case CSW_ERR_NOMEM: return "out of pool memory";
    case CSW_ERR_STATE: return "invalid state for this call";
    case CSW_ERR_TIMEOUT: return "bounded device wait ran out";
    case CSW_ERR_UNSUPPORTED: return "unsupported";
    case CSW_ERR_LIMIT: return "input exceeds the fixed limit of this entry point";
    default: return "unknown status";
  }
}

int csw_last_cuda_error(void) { return tl_cuda_error; }
const char* csw_version(void) { return "0.1.0"; }

csw_status csw_device_status(csw_stream_t stream) {
  int* d_status = nullptr;
  csw_status st = device_state(nullptr, &d_status);
  if (st != CSW_OK) return st;
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_fail(e);
  int h = 0;
  e = cudaMemcpy(&h, d_status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e);
  if (h != 0) {
    e = cudaMemset(d_status, 0, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e);
    return CSW_ERR_TIMEOUT;
  }
  return CSW_OK;
}

// ---- ZFP --------------------------------------------------------------------------
csw_status csw_zfp_max_bytes(size_t nx, size_t ny, size_t nz, unsigned maxbits, size_t* bytes) {
  if (!bytes || !valid_maxbits(maxbits)) return CSW_ERR_ARG;
  if (nx == 0 || (ny == 0 && nz != 0)) return CSW_ERR_ARG;
  if (nx > 0xfffffffcu || ny > 0xfffffffcu || nz > 0xfffffffcu) return CSW_ERR_ARG;  // extents are 32-bit inside
  const FieldGeom g = make_geom(nx, ny, nz, 0, 0, 0);
  // blocks * maxbits must not wrap a 64-bit count of bits
  const unsigned __int128 bits = (unsigned __int128)g.bx * g.by * g.bz * maxbits;
  if (bits > ((unsigned __int128)1 << 62)) return CSW_ERR_ARG;
  *bytes = stream_bytes(g, maxbits);
  return CSW_OK;
}

csw_status csw_zfp_view(size_t numel, size_t* nx, size_t* ny, size_t* nz) {
  if (!nx || !ny || !nz) return CSW_ERR_ARG;
  if (numel == 0 || numel % 1024) return CSW_ERR_UNSUPPORTED;
  *nx = 32;
  *ny = 32;
  *nz = numel / 1024;
  return CSW_OK;
}

static csw_status check_field(size_t nx, size_t ny, size_t nz, unsigned maxbits) {
  if (!valid_maxbits(maxbits)) return CSW_ERR_ARG;
  if (nx == 0 || (ny == 0 && nz != 0)) return CSW_ERR_ARG;
  if (nx > 0xfffffffcu || ny > 0xfffffffcu || nz > 0xfffffffcu) return CSW_ERR_ARG;
  return CSW_OK;
}

csw_status csw_zfp_compress_strided(const float* d_in, size_t nx, size_t ny, size_t nz, ptrdiff_t sx, ptrdiff_t sy,
                                    ptrdiff_t sz, unsigned maxbits, void* d_out, size_t cap, size_t* bytes,
                                    csw_stream_t stream) {
  csw_status st = check_field(nx, ny, nz, maxbits);
  if (st != CSW_OK) return st;
  if (!d_in || !d_out) return CSW_ERR_ARG;
  const FieldGeom g = make_geom(nx, ny, nz, sx, sy, sz);
  const size_t need = stream_bytes(g, maxbits);
  if (bytes) *bytes = need;
  if (cap < need) return CSW_ERR_SIZE;
  cudaError_t e = zfp_encode_launch(g, d_in, d_out, (int)maxbits, stream);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

csw_status csw_zfp_compress(const float* d_in, size_t nx, size_t ny, size_t nz, unsigned maxbits, void* d_out,
                            size_t cap, size_t* bytes, csw_stream_t stream) {
  return csw_zfp_compress_strided(d_in, nx, ny, nz, 0, 0, 0, maxbits, d_out, cap, bytes, stream);
}

csw_status csw_zfp_decompress_strided(const void* d_in, size_t bytes, size_t nx, size_t ny, size_t nz, ptrdiff_t sx,
                                      ptrdiff_t sy, ptrdiff_t sz, unsigned maxbits, float* d_out,
                                      csw_stream_t stream) {
  csw_status st = check_field(nx, ny, nz, maxbits);
  if (st != CSW_OK) return st;
  if (!d_in || !d_out) return CSW_ERR_ARG;
  const FieldGeom g = make_geom(nx, ny, nz, sx, sy, sz);
  if (bytes < stream_bytes(g, maxbits)) return CSW_ERR_SIZE;
  cudaError_t e = zfp_decode_launch(g, d_in, d_out, (int)maxbits, stream);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

csw_status csw_zfp_decompress(const void* d_in, size_t bytes, size_t nx, size_t ny, size_t nz, unsigned maxbits,
                              float* d_out, csw_stream_t stream) {
  return csw_zfp_decompress_strided(d_in, bytes, nx, ny, nz, 0, 0, 0, maxbits, d_out, stream);
}

// ---- sparse -------------------------------------------------------------------------
static size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

csw_status csw_sparse_layout_of(size_t n, csw_sparse_layout* L) {
  if (!L) return CSW_ERR_ARG;
  if (n > 0xffffffffull) return CSW_ERR_ARG;  // value offsets are 32-bit
  const size_t tiles = (n + SPARSE_TILE - 1) / SPARSE_TILE, words = (n + 31) / 32;
  L->tile_off = 0;
  L->bitmap = align16(tiles * 4);
  L->values = L->bitmap + align16(words * 4);
  L->bound = L->values + align16(n * 4);
  return CSW_OK;
}

csw_status csw_sparse_compress(const float* d_in, size_t n, void* d_out, size_t cap, uint32_t* nnz_out,
                               csw_stream_t stream) {
  csw_sparse_layout L;
  csw_status st = csw_sparse_layout_of(n, &L);
  if (st != CSW_OK) return st;
  if ((!d_in && n) || !d_out || !nnz_out) return CSW_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(d_out) & 15) != 0) return CSW_ERR_ARG;
  if (cap < L.bound) return CSW_ERR_SIZE;
  char* base = static_cast<char*>(d_out);
  cudaError_t e = sparse_compress_launch(d_in, n, reinterpret_cast<uint32_t*>(base + L.bitmap),
                                         reinterpret_cast<float*>(base + L.values),
                                         reinterpret_cast<uint32_t*>(base + L.tile_off), nnz_out, stream);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

csw_status csw_sparse_compress_onepass(const float* d_in, size_t n, void* d_out, size_t cap, uint32_t* nnz_out,
                                       csw_stream_t stream) {
  csw_sparse_layout L;
  csw_status st = csw_sparse_layout_of(n, &L);
  if (st != CSW_OK) return st;
  if ((!d_in && n) || !d_out || !nnz_out) return CSW_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(d_out) & 15) != 0) return CSW_ERR_ARG;
  if (cap < L.bound) return CSW_ERR_SIZE;
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, nnz_out) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
    cudaGetLastError();
    return CSW_ERR_ARG;  // the cursor is updated with device atomics
  }
  char* base = static_cast<char*>(d_out);
  cudaError_t e = sparse_compress_onepass_launch(d_in, n, reinterpret_cast<uint32_t*>(base + L.bitmap),
                                                 reinterpret_cast<float*>(base + L.values),
                                                 reinterpret_cast<uint32_t*>(base + L.tile_off), nnz_out, stream);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

csw_status csw_sparse_decompress(const void* d_in, size_t n, float* d_out, csw_stream_t stream) {
  csw_sparse_layout L;
  csw_status st = csw_sparse_layout_of(n, &L);
  if (st != CSW_OK) return st;
  if (!d_in || (!d_out && n)) return CSW_ERR_ARG;
  const char* base = static_cast<const char*>(d_in);
  cudaError_t e = sparse_decompress_launch(reinterpret_cast<const uint32_t*>(base + L.bitmap),
                                           reinterpret_cast<const float*>(base + L.values),
                                           reinterpret_cast<const uint32_t*>(base + L.tile_off), n, d_out, stream);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

// ---- pinned host memory -------------------------------------------------------------
csw_status csw_host_alloc(size_t bytes, void** p) {
  if (!p) return CSW_ERR_ARG;
  cudaError_t e = cudaHostAlloc(p, bytes ? bytes : 1, cudaHostAllocDefault);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}
csw_status csw_host_free(void* p) {
  cudaError_t e = cudaFreeHost(p);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

// =====================================================================================
// entry points with the reference's names
// =====================================================================================
static void legacy_report(const char* where, cudaError_t e) {
  if (e != cudaSuccess) {
    tl_cuda_error = (int)e;
    std::fprintf(stderr, "cswap_b200: %s: %s\n", where, cudaGetErrorString(e));
  }
}

void PreGPUcompression(int arraySize, int kernelSize, float* arrayGPU, int* valueIndex, int, int,
                       csw_stream_t stream) {
  legacy_report("PreGPUcompression", legacy_count_launch(arraySize, kernelSize, arrayGPU, valueIndex, stream));
}
void PreAcc(int* valueIndex, int KernelSize, int* num, int, int, csw_stream_t stream) {
  legacy_report("PreAcc", legacy_scan_launch(valueIndex, KernelSize, num, stream));
}
void GPUcompression(int arraySize, int kernelSize, float* arrayGPU, float* compressedList, int* compressedValueIndex,
                    uint32_t* compressedBinIndex, int, int, csw_stream_t stream) {
  legacy_report("GPUcompression", legacy_pack_launch(arraySize, kernelSize, arrayGPU, compressedList,
                                                     compressedValueIndex, compressedBinIndex, stream));
}
void GPUdecompression(float* arrayGPU, float* destiGPU, int arraySize, int kernelSize, uint32_t* gpuDataindex,
                      int* beginIndex, int, int) {
  legacy_report("GPUdecompression",
                legacy_unpack_launch(arrayGPU, destiGPU, arraySize, kernelSize, gpuDataindex, beginIndex, nullptr));
}

// ---- cuda_compress / cuda_decompress ------------------------------------------------
namespace {

bool is_device_ptr(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// grow-only device staging for callers that hand in host memory (the
// reference cudaMallocs and frees per call, cuZFP.cu:205-304)
struct Staging {
  void* p = nullptr;
  size_t cap = 0;
  int dev = -1;
  cudaError_t reserve(size_t bytes) {
    int d = 0;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess) return e;
    if (p && (d != dev || cap < bytes)) {
      cudaFree(p);
      p = nullptr;
      cap = 0;
    }
    if (!p) {
      e = cudaMalloc(&p, bytes ? bytes : 16);
      if (e != cudaSuccess) return e;
      cap = bytes;
      dev = d;
    }
    return cudaSuccess;
  }
};
std::mutex g_legacy_mu;
Staging g_field_stage, g_stream_stage;

bool contiguous(const csw_zfp_field* f) {
  const ptrdiff_t sx = f->sx ? f->sx : 1, sy = f->sy ? f->sy : (ptrdiff_t)f->nx,
                  sz = f->sz ? f->sz : (ptrdiff_t)(f->nx * (f->ny ? f->ny : 1));
  return sx == 1 && (f->ny == 0 || sy == (ptrdiff_t)f->nx) && (f->nz == 0 || sz == (ptrdiff_t)(f->nx * f->ny));
}
size_t field_values(const csw_zfp_field* f) { return f->nx * (f->ny ? f->ny : 1) * (f->nz ? f->nz : 1); }

// Host-to-host calls on large 3-D fields are cut into z-chunks (zfp blocks are
// independent, so chunk streams concatenate exactly) and run as a three-stage
// pipeline - host->device copy, codec, device->host copy - on three streams, so
// that both directions of the host link are busy at once.
struct Pipeline {
  cudaStream_t in = nullptr, work = nullptr, out = nullptr;
  static constexpr int kMaxChunks = 64;
  cudaEvent_t loaded[kMaxChunks] = {}, coded[kMaxChunks] = {};
  int dev = -1;
  cudaError_t prepare() {
    int d = 0;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess || d == dev) return e;
    if (dev >= 0) return cudaErrorInvalidDevice;  // created for another device: use the plain path
    e = cudaStreamCreateWithFlags(&in, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&work, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&out, cudaStreamNonBlocking);
    for (int i = 0; i < kMaxChunks && e == cudaSuccess; i++) {
      e = cudaEventCreateWithFlags(&loaded[i], cudaEventDisableTiming);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&coded[i], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) dev = d;
    return e;
  }
};
Pipeline g_pipe;

// true when the call was handled here (ok tells how it went)
bool pipelined_host_call(bool compress, const csw_zfp_field* f, void* h_stream, unsigned maxbits, size_t bytes,
                         bool* ok) {
  const size_t slab = f->nx * f->ny;                      // values per z-slab
  const size_t blocks_per_4 = ((f->nx + 3) / 4) * ((f->ny + 3) / 4);
  if (f->nz < 64 || maxbits % 64 || !contiguous(f) || slab * f->nz * 4 < (size_t(64) << 20)) return false;
  // chunk: a multiple of 4 slabs close to 32 MiB of field
  size_t zc = (size_t(32) << 20) / (slab * 4);
  zc = zc < 4 ? 4 : zc / 4 * 4;
  const size_t nchunks = (f->nz + zc - 1) / zc;
  if (nchunks < 2 || nchunks > Pipeline::kMaxChunks) return false;
  if (g_pipe.prepare() != cudaSuccess) { cudaGetLastError(); return false; }
  const size_t fb = slab * f->nz * 4;
  if (g_field_stage.reserve(fb) != cudaSuccess || g_stream_stage.reserve(bytes) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  *ok = false;
  cudaError_t e = cudaStreamSynchronize(nullptr);  // earlier default-stream work (as the reference's device sync)
  char* h_field = static_cast<char*>(f->data);
  char* d_field = static_cast<char*>(g_field_stage.p);
  char* d_stream = static_cast<char*>(g_stream_stage.p);
  char* hs = static_cast<char*>(h_stream);
  for (size_t c = 0; c < nchunks && e == cudaSuccess; c++) {
    const size_t z0 = c * zc, nzc = f->nz - z0 < zc ? f->nz - z0 : zc;
    const size_t foff = z0 * slab * 4, flen = nzc * slab * 4;
    const size_t soff = (z0 / 4) * blocks_per_4 * maxbits / 8;
    size_t slen = 0;
    csw_zfp_max_bytes(f->nx, f->ny, nzc, maxbits, &slen);
    csw_status st;
    if (compress) {
      e = cudaMemcpyAsync(d_field + foff, h_field + foff, flen, cudaMemcpyHostToDevice, g_pipe.in);
      if (e == cudaSuccess) e = cudaEventRecord(g_pipe.loaded[c], g_pipe.in);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(g_pipe.work, g_pipe.loaded[c], 0);
      if (e != cudaSuccess) break;
      st = csw_zfp_compress(reinterpret_cast<const float*>(d_field + foff), f->nx, f->ny, nzc, maxbits,
                            d_stream + soff, slen, nullptr, g_pipe.work);
      if (st != CSW_OK) {
        // work of earlier chunks is still queued on the three streams and the staging buffers are shared
        cudaStreamSynchronize(g_pipe.in);
        cudaStreamSynchronize(g_pipe.work);
        cudaStreamSynchronize(g_pipe.out);
        return true;
      }
      e = cudaEventRecord(g_pipe.coded[c], g_pipe.work);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(g_pipe.out, g_pipe.coded[c], 0);
      if (e == cudaSuccess) e = cudaMemcpyAsync(hs + soff, d_stream + soff, slen, cudaMemcpyDeviceToHost, g_pipe.out);
    } else {
      e = cudaMemcpyAsync(d_stream + soff, hs + soff, slen, cudaMemcpyHostToDevice, g_pipe.in);
      if (e == cudaSuccess) e = cudaEventRecord(g_pipe.loaded[c], g_pipe.in);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(g_pipe.work, g_pipe.loaded[c], 0);
      if (e != cudaSuccess) break;
      st = csw_zfp_decompress(d_stream + soff, slen, f->nx, f->ny, nzc, maxbits,
                              reinterpret_cast<float*>(d_field + foff), g_pipe.work);
      if (st != CSW_OK) {
        // work of earlier chunks is still queued on the three streams and the staging buffers are shared
        cudaStreamSynchronize(g_pipe.in);
        cudaStreamSynchronize(g_pipe.work);
        cudaStreamSynchronize(g_pipe.out);
        return true;
      }
      e = cudaEventRecord(g_pipe.coded[c], g_pipe.work);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(g_pipe.out, g_pipe.coded[c], 0);
      if (e == cudaSuccess) e = cudaMemcpyAsync(h_field + foff, d_field + foff, flen, cudaMemcpyDeviceToHost, g_pipe.out);
    }
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(g_pipe.out);
  if (e != cudaSuccess) {
    legacy_report(compress ? "cuda_compress" : "cuda_decompress", e);
    cudaStreamSynchronize(g_pipe.in);
    cudaStreamSynchronize(g_pipe.work);
    cudaStreamSynchronize(g_pipe.out);
    return true;
  }
  *ok = true;
  return true;
}

}  // namespace

size_t cuda_compress(csw_zfp_stream* zs, const csw_zfp_field* f) {
  if (!zs || !zs->stream || !zs->stream->begin || !f || !f->data) return 0;
  if (f->type != 3 || f->nw != 0) {
    std::fprintf(stderr, "cswap_b200: cuda_compress: only float32 fields of up to 3 dimensions are supported\n");
    return 0;
  }
  std::lock_guard<std::mutex> lk(g_legacy_mu);
  const unsigned maxbits = zs->maxbits;
  size_t bytes = 0;
  if (csw_zfp_max_bytes(f->nx, f->ny, f->nz, maxbits, &bytes) != CSW_OK) return 0;
  const bool field_dev = is_device_ptr(f->data), stream_dev = is_device_ptr(zs->stream->begin);
  if (!field_dev && !stream_dev) {
    bool ok = false;
    if (pipelined_host_call(true, f, zs->stream->begin, maxbits, bytes, &ok)) {
      if (!ok) return 0;
      zs->stream->bits = 64;
      zs->stream->ptr = zs->stream->begin + bytes / 8;
      return bytes;
    }
  }
  const float* d_field = static_cast<const float*>(f->data);
  ptrdiff_t sx = f->sx, sy = f->sy, sz = f->sz;
  if (!field_dev) {
    if (!contiguous(f)) return 0;  // as the reference: strided host arrays are refused (cuZFP.cu:381-385)
    const size_t fb = field_values(f) * sizeof(float);
    cudaError_t e = g_field_stage.reserve(fb);
    if (e == cudaSuccess) e = cudaMemcpyAsync(g_field_stage.p, f->data, fb, cudaMemcpyHostToDevice, nullptr);
    if (e != cudaSuccess) { legacy_report("cuda_compress", e); return 0; }
    d_field = static_cast<const float*>(g_field_stage.p);
    sx = sy = sz = 0;
  }
  void* d_stream = zs->stream->begin;
  if (!stream_dev) {
    cudaError_t e = g_stream_stage.reserve(bytes);
    if (e != cudaSuccess) { legacy_report("cuda_compress", e); return 0; }
    d_stream = g_stream_stage.p;
  }
  csw_status st = csw_zfp_compress_strided(d_field, f->nx, f->ny, f->nz, sx, sy, sz, maxbits, d_stream, bytes, nullptr,
                                           nullptr);
  if (st != CSW_OK) return 0;
  cudaError_t e = cudaSuccess;
  if (!stream_dev) e = cudaMemcpyAsync(zs->stream->begin, d_stream, bytes, cudaMemcpyDeviceToHost, nullptr);
  if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
  if (e != cudaSuccess) { legacy_report("cuda_compress", e); return 0; }
  // what zfp expects after a flush (cuZFP.cu:428-433)
  zs->stream->bits = 64;
  zs->stream->ptr = zs->stream->begin + bytes / 8;
  return bytes;
}

void cuda_decompress(csw_zfp_stream* zs, csw_zfp_field* f) {
  if (!zs || !zs->stream || !zs->stream->begin || !f || !f->data) return;
  if (f->type != 3 || f->nw != 0) {
    std::fprintf(stderr, "cswap_b200: cuda_decompress: only float32 fields of up to 3 dimensions are supported\n");
    return;
  }
  std::lock_guard<std::mutex> lk(g_legacy_mu);
  const unsigned maxbits = zs->maxbits;
  size_t bytes = 0;
  if (csw_zfp_max_bytes(f->nx, f->ny, f->nz, maxbits, &bytes) != CSW_OK) return;
  const bool field_dev = is_device_ptr(f->data), stream_dev = is_device_ptr(zs->stream->begin);
  if (!field_dev && !stream_dev) {
    bool ok = false;
    if (pipelined_host_call(false, f, zs->stream->begin, maxbits, bytes, &ok)) {
      if (ok) {
        zs->stream->bits = 64;
        zs->stream->ptr = zs->stream->begin + bytes / 8;
      }
      return;
    }
  }
  float* d_field = static_cast<float*>(f->data);
  ptrdiff_t sx = f->sx, sy = f->sy, sz = f->sz;
  const size_t fb = field_values(f) * sizeof(float);
  if (!field_dev) {
    if (!contiguous(f)) return;
    cudaError_t e = g_field_stage.reserve(fb);
    if (e != cudaSuccess) { legacy_report("cuda_decompress", e); return; }
    d_field = static_cast<float*>(g_field_stage.p);
    sx = sy = sz = 0;
  }
  const void* d_stream = zs->stream->begin;
  if (!stream_dev) {
    cudaError_t e = g_stream_stage.reserve(bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(g_stream_stage.p, zs->stream->begin, bytes, cudaMemcpyHostToDevice, nullptr);
    if (e != cudaSuccess) { legacy_report("cuda_decompress", e); return; }
    d_stream = g_stream_stage.p;
  }
  csw_status st =
      csw_zfp_decompress_strided(d_stream, bytes, f->nx, f->ny, f->nz, sx, sy, sz, maxbits, d_field, nullptr);
  if (st != CSW_OK) return;
  cudaError_t e = cudaSuccess;
  if (!field_dev) e = cudaMemcpyAsync(f->data, d_field, fb, cudaMemcpyDeviceToHost, nullptr);
  if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
  if (e != cudaSuccess) { legacy_report("cuda_decompress", e); return; }
  zs->stream->bits = 64;
  zs->stream->ptr = zs->stream->begin + bytes / 8;
}

}  // extern "C"


// ---- the wrappers the reference's Execution calls (Execution.h:63,113,296) ----------
namespace {
std::mutex g_wrap_mu;
unsigned g_ratio_maxbits = 512;
csw_alloc_fn g_alloc = nullptr;
csw_free_fn g_free = nullptr;

void* wrap_alloc(size_t bytes) {
  if (g_alloc) return g_alloc(bytes);
  void* p = nullptr;
  return cudaMalloc(&p, bytes) == cudaSuccess ? p : nullptr;
}
void wrap_free(void* p) {
  if (!p) return;
  if (g_free) g_free(p);
  else cudaFree(p);
}
// stream bytes and total bytes (stream + the values past the last whole slab)
bool wrap_geometry(size_t numel, unsigned maxbits, size_t* nz, size_t* zbytes, size_t* bytes) {
  *nz = numel / 1024;
  *zbytes = 0;
  if (*nz && csw_zfp_max_bytes(32, 32, *nz, maxbits, zbytes) != CSW_OK) return false;
  *bytes = *zbytes + (numel % 1024) * sizeof(float);
  return true;
}
}  // namespace

extern "C" void csw_set_device_allocator(csw_alloc_fn alloc, csw_free_fn release) {
  std::lock_guard<std::mutex> lk(g_wrap_mu);
  g_alloc = alloc && release ? alloc : nullptr;
  g_free = alloc && release ? release : nullptr;
}

void setRatio(int maxbits) {
  size_t probe;
  std::lock_guard<std::mutex> lk(g_wrap_mu);
  if (maxbits > 0 && csw_zfp_max_bytes(32, 32, 4, (unsigned)maxbits, &probe) == CSW_OK) g_ratio_maxbits = (unsigned)maxbits;
  else legacy_report("setRatio", cudaErrorInvalidValue);
}

void* compress(void* dev_ptr, size_t numel, size_t& out_bytes) {
  out_bytes = 0;
  unsigned maxbits;
  {
    std::lock_guard<std::mutex> lk(g_wrap_mu);
    maxbits = g_ratio_maxbits;
  }
  size_t nz, zbytes, bytes;
  if (!dev_ptr || !numel || !wrap_geometry(numel, maxbits, &nz, &zbytes, &bytes)) return nullptr;
  void* buf = wrap_alloc(bytes);
  if (!buf) return nullptr;
  csw_status st = CSW_OK;
  if (nz) st = csw_zfp_compress(static_cast<const float*>(dev_ptr), 32, 32, nz, maxbits, buf, zbytes, nullptr, nullptr);
  cudaError_t e = cudaSuccess;
  if (st == CSW_OK && bytes > zbytes)
    e = cudaMemcpyAsync(static_cast<char*>(buf) + zbytes, static_cast<const float*>(dev_ptr) + nz * 1024, bytes - zbytes,
                        cudaMemcpyDeviceToDevice, nullptr);
  if (st != CSW_OK || e != cudaSuccess) {
    legacy_report("compress", e != cudaSuccess ? e : cudaErrorUnknown);
    wrap_free(buf);
    return nullptr;
  }
  out_bytes = bytes;
  return buf;
}

void decompress(void* dev_buf, size_t bytes, void* dev_dst, size_t numel) {
  unsigned maxbits;
  {
    std::lock_guard<std::mutex> lk(g_wrap_mu);
    maxbits = g_ratio_maxbits;
  }
  size_t nz, zbytes, need;
  if (!dev_buf || !dev_dst || !numel || !wrap_geometry(numel, maxbits, &nz, &zbytes, &need) || bytes < need) {
    legacy_report("decompress", cudaErrorInvalidValue);
    return;
  }
  csw_status st = CSW_OK;
  if (nz) st = csw_zfp_decompress(dev_buf, zbytes, 32, 32, nz, maxbits, static_cast<float*>(dev_dst), nullptr);
  cudaError_t e = cudaSuccess;
  if (st == CSW_OK && need > zbytes)
    e = cudaMemcpyAsync(static_cast<float*>(dev_dst) + nz * 1024, static_cast<const char*>(dev_buf) + zbytes,
                        need - zbytes, cudaMemcpyDeviceToDevice, nullptr);
  if (st != CSW_OK || e != cudaSuccess) legacy_report("decompress", e != cudaSuccess ? e : cudaErrorUnknown);
}
