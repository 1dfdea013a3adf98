/*
 * CPU oracle for the compressed tensor-swap codecs.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference algorithms (ISCS-ZJU/CSWAP, directory
 * CSWAP+/zfp): the cuZFP fixed-rate float32 codec and the zero-value ("ZVC")
 * sparse codec.  It exists to check the CUDA library and to be timed as the
 * CPU baseline; nothing in the shipped library may link or call it.
 *
 * Parity pin: the reference ships no golden vectors for this path.  The
 * restatement is pinned against the reference's own headers compiled for the
 * host (oracle/ref_shim.cpp -> oracle/_ref/libcswap_ref.so) and against
 * fixtures generated from that build (tests/golden/).
 */
#ifndef CSWAP_ORACLE_H
#define CSWAP_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- ZFP fixed-rate float32, 1-D / 2-D / 3-D ---------------------------- */

/* Bytes of whole 64-bit words covering every (padded) block of the field.
 * Equals the reference's shared.h:39-84 counts when maxbits % 64 == 0 and no
 * block is partial.  ny==0 / nz==0 select lower dimensionality. */
size_t orc_zfp_stream_bytes(size_t nx, size_t ny, size_t nz, unsigned maxbits);

/* Encode a contiguous float32 array viewed as nx*ny*nz (x fastest) at
 * `maxbits` bits per 4^d block.  `out` must hold orc_zfp_stream_bytes()+8
 * bytes and is fully written (zero filled first, encode3.cuh:152).
 * threads<=1: serial; otherwise OpenMP over blocks (needs maxbits%64==0,
 * else falls back to serial).  Returns stream bytes. */
size_t orc_zfp_encode(const float* in, size_t nx, size_t ny, size_t nz,
                      unsigned maxbits, uint64_t* out, int threads);

/* Inverse.  `out` receives nx*ny*nz floats. */
void orc_zfp_decode(const uint64_t* in, size_t nx, size_t ny, size_t nz,
                    unsigned maxbits, float* out, int threads);

/* One block, exposed for unit tests.  dims = 1,2,3 -> 4,16,64 values.
 * Writes at bit offset block_idx*maxbits of `stream` (which must be zeroed).
 * Returns the largest count of significant coefficients (n) seen by the plane
 * coder so callers can tell whether a full 64-bit verbatim plane occurred. */
int orc_zfp_encode_block(const float* fblock, int dims, unsigned maxbits,
                         size_t block_idx, uint64_t* stream);
void orc_zfp_decode_block(const uint64_t* stream, int dims, unsigned maxbits,
                          size_t block_idx, float* fblock);

/* Pieces, for unit tests (encode.cuh:73-99, shared.h:221-250, :176-181,
 * decode.cuh:33-37). */
void orc_fwd_lift(int32_t* p, unsigned stride);
void orc_inv_lift(int32_t* p, unsigned stride);
uint32_t orc_int2uint(int32_t x);
int32_t orc_uint2int(uint32_t x);
const unsigned char* orc_perm3(void);

/* ---- sparse (zero-value) codec ------------------------------------------ */

/* Native format of the CUDA library: bitmap[ceil(n/32)] uint32 in element
 * order (bit j of word w <=> element 32w+j has a non-zero BIT PATTERN, so
 * -0.0 and NaN survive), values[nnz] in element order, tile_off[ceil(n/4096)]
 * = exclusive prefix of non-zeros per 4096-element tile.  Returns nnz. */
size_t orc_sparse_compress(const float* in, size_t n, uint32_t* bitmap,
                           float* values, uint32_t* tile_off, int threads);
void orc_sparse_decompress(const uint32_t* bitmap, const float* values,
                           size_t n, float* out, int threads);

/* Reference layout (compression.cu:9-19,134-318; Execution.h:88-90):
 * P workers (P = dimsize*blocksize), chunk c = ceil(n/P); begin[P] exclusive
 * scan of per-worker counts over the first `active` = ceil(n/c) workers;
 * bitmap words of worker i start at i*ceil(c/32); non-zero test is float
 * `!= 0` (so -0.0 is dropped, NaN kept).  Returns nnz. */
size_t orc_legacy_sparse_compress(const float* in, int n, int P, int32_t* begin,
                                  uint32_t* bitmap, float* values);
/* Reference decompression: zeros after the last set bit of each bitmap word
 * are NOT written (compression.cu:281-292); `out` is left untouched there. */
void orc_legacy_sparse_decompress(const float* values, float* out, int n, int P,
                                  const uint32_t* bitmap, const int32_t* begin);

int orc_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
