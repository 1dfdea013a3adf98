// Launch interface of the sparse-codec kernels (internal to the library).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace csw {

constexpr int SPARSE_TILE = 4096;  // elements per independently decodable tile

// Native format.  tile_off must hold ceil(n/4096) words (it is used as the
// count buffer first), bitmap ceil(n/32) words, values up to n floats.
// *nnz_out (device or mapped host memory) receives the number of values.
cudaError_t sparse_compress_launch(const float* in, uint64_t n, uint32_t* bitmap, float* values, uint32_t* tile_off,
                                   uint32_t* nnz_out, cudaStream_t stream);
// Same result, with the per-tile counts kept in a scratch array the caller owns
// (ceil(n/4096) words) instead of passing through tile_off.
cudaError_t sparse_compress_scratch_launch(const float* in, uint64_t n, uint32_t* bitmap, float* values,
                                           uint32_t* tile_off, uint32_t* tile_cnt_scratch, uint32_t* nnz_out,
                                           cudaStream_t stream);
// Single pass over the tensor: same bitmap, same per-tile contents, but the
// tiles' value segments are laid out in the order the tiles claimed them
// (tile_off says where each one starts).  *nnz_out must be DEVICE memory: it is
// the allocation cursor during the kernel and holds the total afterwards.
cudaError_t sparse_compress_onepass_launch(const float* in, uint64_t n, uint32_t* bitmap, float* values,
                                           uint32_t* tile_off, uint32_t* nnz_out, cudaStream_t stream);
cudaError_t sparse_decompress_launch(const uint32_t* bitmap, const float* values, const uint32_t* tile_off, uint64_t n,
                                     float* out, cudaStream_t stream);

// Reference layout (P workers, chunk = ceil(n/P)); see the legacy entry points.
cudaError_t legacy_count_launch(int n, int workers, const float* in, int* count, cudaStream_t stream);
cudaError_t legacy_scan_launch(int* idx, int len, int* num, cudaStream_t stream);
cudaError_t legacy_pack_launch(int n, int workers, const float* in, float* values, const int* begin, uint32_t* bitmap,
                               cudaStream_t stream);
cudaError_t legacy_unpack_launch(const float* values, float* out, int n, int workers, const uint32_t* bitmap,
                                 const int* begin, cudaStream_t stream);

}  // namespace csw
