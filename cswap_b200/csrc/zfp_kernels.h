// Launch interface of the ZFP kernels (internal to the library).
#pragma once
#include <cuda_runtime.h>

#include "zfp_field.cuh"

namespace csw {

// True when the slab (nx = ny = 32, contiguous, whole words, 16-byte aligned)
// kernels apply; everything else goes through the generic kernels.
bool zfp_slab_eligible(const FieldGeom& g, const void* field, const void* stream, int maxbits);

// Enqueue encode/decode of a whole field on `stream`.  `out` of the encoder
// must hold stream_bytes(g, maxbits); every byte of it is written.
cudaError_t zfp_encode_launch(const FieldGeom& g, const float* in, void* out, int maxbits, cudaStream_t stream);
cudaError_t zfp_decode_launch(const FieldGeom& g, const void* in, float* out, int maxbits, cudaStream_t stream);

}  // namespace csw
