// An allocation-free way into the sparse compressor.
//
// Some callers may not allocate device memory at the moment they need to
// compress: a swap hook that runs while the framework's caching allocator is
// locked or already out of memory (which is exactly when swapping is wanted),
// a callback on a path where cudaMalloc's implicit device synchronisation
// would stall other streams, or an embedding with a fixed memory budget handed
// over at start-up.  For them the per-tile counters of the compressor live in
// a fixed array inside the library image instead of anywhere that has to be
// obtained at run time.  (The driver places that array, and the kernels, on a
// device when the library's code is first used there; a warm-up call at
// start-up gets that over with while memory is still available.)
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../include/cswap_b200.h"
#include "internal.h"
#include "sparse_kernels.h"

namespace csw {
namespace {

// One counter per 4096-element tile.  65536 tiles cover 268 435 456 floats
// (1 GiB); the array costs 256 KiB of device memory on every GPU that loads
// the library, for the life of the process.
constexpr uint32_t kMaxTiles = CSW_SPARSE_STATIC_MAX_ELEMS / SPARSE_TILE;
static __device__ __align__(256) uint32_t g_tile_counts[kMaxTiles];

// In host code the array's name is only a handle; the address kernels can use
// has to be asked for, per device, with that device current.
constexpr int kMaxDevices = 64;
uint32_t* g_counts_addr[kMaxDevices];
bool g_counts_ready[kMaxDevices];
std::mutex g_counts_mu;

csw_status counts_address(uint32_t** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(g_counts_mu);
  if (!g_counts_ready[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_tile_counts);
    if (e != cudaSuccess) return cuda_fail(e);
    g_counts_addr[dev] = static_cast<uint32_t*>(p);
    g_counts_ready[dev] = true;
  }
  *out = g_counts_addr[dev];
  return CSW_OK;
}

}  // namespace
}  // namespace csw

using namespace csw;

extern "C" csw_status csw_sparse_compress_static(const float* d_in, size_t n, void* d_out, size_t cap,
                                                 uint32_t* nnz_out, csw_stream_t stream) {
  if (n > CSW_SPARSE_STATIC_MAX_ELEMS) return CSW_ERR_LIMIT;  // more tiles than the fixed counter array holds
  csw_sparse_layout L;
  csw_status st = csw_sparse_layout_of(n, &L);
  if (st != CSW_OK) return st;
  if ((!d_in && n) || !d_out || !nnz_out) return CSW_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(d_out) & 15) != 0) return CSW_ERR_ARG;
  if (cap < L.bound) return CSW_ERR_SIZE;
  uint32_t* counts = nullptr;
  st = counts_address(&counts);
  if (st != CSW_OK) return st;
  // Every counter the scan reads (tiles 0 .. ceil(n/4096)-1) is rewritten by
  // the counting pass of this same call, so nothing left over from an earlier
  // call has to be cleared.
  char* base = static_cast<char*>(d_out);
  cudaError_t e = sparse_compress_scratch_launch(d_in, n, reinterpret_cast<uint32_t*>(base + L.bitmap),
                                                 reinterpret_cast<float*>(base + L.values),
                                                 reinterpret_cast<uint32_t*>(base + L.tile_off), counts, nnz_out,
                                                 stream);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}
