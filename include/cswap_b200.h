/*
 * cswap_b200 - C ABI of the B200-native compressed tensor-swap path.
 *
 * A drop-in for the GPU codec and swap-out/swap-in path of CSWAP+
 * (ISCS-ZJU/CSWAP).  Plain pointers and sizes only; every entry point returns a
 * csw_status (the reference returns void and never reports errors,
 * CSWAP+/zfp/ErrorCheck.h:17-25).  All device work is enqueued on the stream
 * the caller passes; nothing synchronises the device unless stated.
 *
 * Sections:
 *   1. status codes
 *   2. ZFP fixed-rate float32 codec      (replaces cuda_compress/cuda_decompress,
 *                                         CSWAP+/zfp/cuZFP.h:10-12, cuZFP.cu:364-532)
 *   3. sparse zero-value codec           (replaces the four kernels of
 *                                         CSWAP+/zfp/compression.cuh:4-8)
 *   4. swap manager                      (replaces the device/host side of
 *                                         Execution::pre/post, CSWAP+/Execution.h:65-412)
 *   5. cost model                        (replaces c10::GetPolicyMaker(), call
 *                                         sites CSWAP+/Execution.h:224-233,
 *                                         CSWAP+/resnet-cifar10.cpp:407-437)
 *   6. legacy entry points with the reference's own names (cswap_compat.h)
 */
#ifndef CSWAP_B200_H
#define CSWAP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A CUDA stream handle (cudaStream_t); NULL is the legacy default stream. */
typedef struct CUstream_st* csw_stream_t;

/* ---- 1. status ----------------------------------------------------------- */
typedef int csw_status;
enum {
  CSW_OK = 0,
  CSW_ERR_ARG = 1,      /* bad argument (null pointer, bad rate, bad geometry)   */
  CSW_ERR_SIZE = 2,     /* output capacity too small; nothing was launched       */
  CSW_ERR_CUDA = 3,     /* a CUDA runtime call failed; see csw_last_cuda_error() */
  CSW_ERR_NOMEM = 4,    /* a pool or allocation is exhausted                     */
  CSW_ERR_STATE = 5,    /* call not valid in the handle's current state          */
  CSW_ERR_TIMEOUT = 6,  /* a bounded device-side wait ran out                    */
  CSW_ERR_UNSUPPORTED = 7,
  CSW_ERR_LIMIT = 8     /* input exceeds a fixed limit of the entry point called  */
};
const char* csw_status_string(csw_status s);
/* cudaError_t of the most recent failing runtime call on this thread (0 if none). */
int csw_last_cuda_error(void);
/* Library version, "major.minor.patch". */
const char* csw_version(void);
/* Reads (and clears) the device-side status word of the current device:
 * CSW_OK, or CSW_ERR_TIMEOUT if a kernel gave up on a bounded wait.
 * Synchronises `stream` first.  The kernels of this version contain no
 * device-side wait (no kernel depends on another CTA, a flag or a copy in
 * flight), so the word stays zero; the call remains as the place where such a
 * failure would surface. */
csw_status csw_device_status(csw_stream_t stream);

/* ---- 2. ZFP fixed-rate float32 ------------------------------------------- */
/* A field is a float32 array viewed as nx * ny * nz values, x fastest
 * (ny = 0 and/or nz = 0 select 2-D / 1-D blocks of 16 / 4 values, as zfp_field
 * does, CSWAP+/zfp/zfp.h:140-145).  `maxbits` is the bit budget per 4^d block
 * (zfp_stream.maxbits as consumed by CSWAP+/zfp/cuZFP.cu:395); for a rate of r
 * bits per value in 3-D it is 64 * r.  Block b occupies stream bits
 * [b * maxbits, (b + 1) * maxbits), 64-bit words, LSB first
 * (CSWAP+/zfp/encode.cuh:229-230,259-272). */

/* Bytes of stream for the field: whole 64-bit words covering every block
 * (counterpart of calc_device_mem{1,2,3}d, CSWAP+/zfp/shared.h:39-84). */
csw_status csw_zfp_max_bytes(size_t nx, size_t ny, size_t nz, unsigned maxbits, size_t* bytes);

/* Compress device array d_in into device buffer d_out of capacity `cap`
 * bytes; *bytes (host, may be NULL) receives the stream size.  Every byte of
 * the stream is written: no pre-zeroing is needed (the reference memsets,
 * CSWAP+/zfp/encode3.cuh:152).  Replaces cuda_compress for device pointers
 * (CSWAP+/zfp/cuZFP.cu:364-436) and the fork's compress() wrapper
 * (CSWAP+/Execution.h:113).  Strides are in elements; 0 means contiguous. */
csw_status csw_zfp_compress(const float* d_in, size_t nx, size_t ny, size_t nz, unsigned maxbits, void* d_out,
                            size_t cap, size_t* bytes, csw_stream_t stream);
csw_status csw_zfp_compress_strided(const float* d_in, size_t nx, size_t ny, size_t nz, ptrdiff_t sx, ptrdiff_t sy,
                                    ptrdiff_t sz, unsigned maxbits, void* d_out, size_t cap, size_t* bytes,
                                    csw_stream_t stream);

/* Decompress `bytes` of stream into device array d_out (every element is
 * written).  Replaces cuda_decompress (CSWAP+/zfp/cuZFP.cu:440-532). */
csw_status csw_zfp_decompress(const void* d_in, size_t bytes, size_t nx, size_t ny, size_t nz, unsigned maxbits,
                              float* d_out, csw_stream_t stream);
csw_status csw_zfp_decompress_strided(const void* d_in, size_t bytes, size_t nx, size_t ny, size_t nz, ptrdiff_t sx,
                                      ptrdiff_t sy, ptrdiff_t sz, unsigned maxbits, float* d_out,
                                      csw_stream_t stream);

/* The swap path's view of a flat tensor (BASELINE: nx = ny = 32,
 * nz = numel / 1024).  Returns CSW_ERR_UNSUPPORTED when numel is not a
 * multiple of 1024 (the swap manager then codes the whole slabs and moves the
 * remaining numel % 1024 values as they are). */
csw_status csw_zfp_view(size_t numel, size_t* nx, size_t* ny, size_t* nz);

/* ---- 3. sparse zero-value codec ------------------------------------------ */
/* Native packed layout of a compressed tensor of n floats, all offsets in
 * bytes from the start of the buffer, each section 16-byte aligned:
 *   [tile_off: ceil(n/4096) u32][bitmap: ceil(n/32) u32][values: nnz f32]
 * bit j of bitmap word w is set iff element 32w + j has a non-zero bit
 * pattern; the non-zeros of tile t (elements 4096 t ...) sit in element order
 * at values[tile_off[t] ...].  csw_sparse_compress lays the tiles' segments
 * out in tile order (tile_off[t] = number of values before element 4096 t);
 * csw_sparse_compress_onepass in the order the tiles were scheduled. */
typedef struct {
  size_t tile_off; /* always 0 */
  size_t bitmap;
  size_t values;
  size_t bound;    /* bytes needed when every element is non-zero */
} csw_sparse_layout;
csw_status csw_sparse_layout_of(size_t n, csw_sparse_layout* layout);

/* Compress n floats at d_in into d_out (capacity cap >= layout.bound).
 * *nnz_out receives the number of packed values when the stream reaches that
 * point; it may live in device memory or in mapped pinned host memory.  The
 * bytes to move afterwards are layout.values + 4 * nnz.  Replaces the
 * PreGPUcompression -> PreAcc -> blocking copy -> GPUcompression sequence of
 * CSWAP+/Execution.h:88-95 without any host round trip. */
csw_status csw_sparse_compress(const float* d_in, size_t n, void* d_out, size_t cap, uint32_t* nnz_out,
                               csw_stream_t stream);
/* The same compression from ONE read of the tensor (one launch instead of
 * three; about 1.7x faster on large tensors).  Bitmap, count and every tile's
 * segment are those of csw_sparse_compress, but each tile claims its place in
 * `values` with an atomic add, so the segments' order - and with it the bytes
 * of tile_off and values - depends on the schedule and can differ between two
 * runs on the same input.  csw_sparse_decompress returns the identical tensor
 * either way.  nnz_out must be DEVICE memory (it is the allocation cursor
 * while the kernel runs).  Used by the swap manager, whose packed buffers never
 * leave the library. */
csw_status csw_sparse_compress_onepass(const float* d_in, size_t n, void* d_out, size_t cap, uint32_t* nnz_out,
                                       csw_stream_t stream);
/* csw_sparse_compress for callers that must not allocate.  (No counterpart in
 * the reference, whose swap-out allocates on every call.)
 *
 * Meant for code that runs where device allocation is off the table: a swap
 * hook invoked while the framework's allocator is locked or has just failed
 * (the moment swapping is most wanted), a callback where cudaMalloc's implicit
 * synchronisation would stall unrelated streams, or a host program that gets a
 * fixed memory budget at start-up.  The compressor's per-tile counters sit in
 * a fixed 256 KiB array inside the library image (present on every GPU that
 * loads the library until the process exits); the call performs no cudaMalloc,
 * cudaFree or other allocating call, and writes the same bytes to d_out and
 * the same count to *nnz_out as csw_sparse_compress.
 *
 *  - n may be at most CSW_SPARSE_STATIC_MAX_ELEMS; larger inputs return
 *    CSW_ERR_LIMIT and launch nothing.
 *  - The first call on each device looks up the array's device address.  With
 *    the CUDA runtime's default lazy loading that first lookup (or launch) is
 *    also when the driver loads the library's kernels and the array itself
 *    onto the device, which does take device memory and can fail when none is
 *    left.  So make one warm-up call per device (n = 0 is enough) at start-up,
 *    outside any stream capture and before memory is tight; later calls on
 *    that device touch no allocator of any kind.
 *  - All calls share the one array: two calls whose kernels may run at the same
 *    time on the same GPU (different streams, no ordering between them) race
 *    and corrupt each other's output.  Calls ordered on one stream, or by
 *    events, are fine; nothing needs clearing between them. */
#define CSW_SPARSE_STATIC_MAX_ELEMS 268435456u /* 65536 tiles of 4096 floats = 1 GiB of input */
csw_status csw_sparse_compress_static(const float* d_in, size_t n, void* d_out, size_t cap, uint32_t* nnz_out,
                                      csw_stream_t stream);
/* Rebuild n floats at d_out from a packed buffer; every element is written
 * (the reference leaves trailing zeros unwritten, compression.cu:281-292). */
csw_status csw_sparse_decompress(const void* d_in, size_t n, float* d_out, csw_stream_t stream);

/* ---- 4. swap manager ------------------------------------------------------ */
/* Policy codes, as in CSWAP+/Execution.h:70,86,107,243. */
enum {
  CSW_POLICY_KEEP = 0,   /* leave the tensor on the device            */
  CSW_POLICY_DROP = 1,   /* free it; the caller recomputes it         */
  CSW_POLICY_RAW = 2,    /* swap uncompressed (vDNN)                  */
  CSW_POLICY_SPARSE = 3, /* sparse codec + swap                       */
  CSW_POLICY_ZFP = 6     /* ZFP fixed rate + swap                     */
};

typedef struct csw_mgr csw_mgr;       /* one per device / replica      */
typedef struct csw_ticket csw_ticket; /* one swapped-out tensor        */

typedef struct {
  int device;               /* CUDA device ordinal                                   */
  size_t pinned_bytes;      /* pinned host pool (0: 1 GiB)                           */
  size_t staging_bytes;     /* device pool for compressed staging (0: 512 MiB); a
                               payload stays staged after its copy out until the
                               pool needs the room, and a swap-in that still finds
                               it there does not cross the link                      */
  unsigned zfp_maxbits;     /* bits per block for CSW_POLICY_ZFP (0: 512 = rate 8);
                               the reference's setRatio(), CSWAP+/Execution.h:63     */
} csw_mgr_config;

csw_status csw_mgr_create(const csw_mgr_config* cfg, csw_mgr** out);
csw_status csw_mgr_destroy(csw_mgr* m);
csw_status csw_mgr_set_zfp_maxbits(csw_mgr* m, unsigned maxbits);
/* keep = 0: a staged payload is released as soon as its copy out has finished, so every
 * swap-in of it crosses the link; keep != 0 (the default): it stays until the staging pool
 * needs the room. */
csw_status csw_mgr_keep_staged(csw_mgr* m, int keep);
/* The manager's own streams (the reference's stream1, CSWAP+/Execution.h:49,
 * split by role), e.g. to tell a caching allocator that a tensor handed to
 * csw_swap_out is still being read on them. */
csw_status csw_mgr_get_streams(csw_mgr* m, csw_stream_t* codec, csw_stream_t* d2h, csw_stream_t* h2d);

/* Swap-out (Execution::pre, CSWAP+/Execution.h:65-133).  Waits (on the device,
 * by event) for `compute` to reach this point, compresses per `policy` on the
 * manager's codec stream into device staging, and copies to pinned host memory
 * on the manager's D2H stream.  Returns immediately; *ticket identifies the
 * host copy.  The caller may release d_ptr once csw_swap_out_done() reports
 * completion or after making its own stream wait with csw_swap_out_wait().
 * Under CSW_POLICY_ZFP the first numel / 1024 slabs of 32x32 values are coded
 * and the rest (numel % 1024 values) travels uncoded behind the stream; a
 * tensor of fewer than 1024 values falls back to CSW_POLICY_RAW.  The ticket
 * records what was used. */
csw_status csw_swap_out(csw_mgr* m, const float* d_ptr, size_t numel, int policy, csw_stream_t compute,
                        csw_ticket** ticket);
/* 1 in *done when the tensor's device bytes are no longer needed. */
csw_status csw_swap_out_done(csw_mgr* m, csw_ticket* t, int* done);
/* Block the host until d_ptr is no longer read. */
csw_status csw_swap_out_sync(csw_mgr* m, csw_ticket* t);
/* Make `stream` wait (device side) until d_ptr is no longer read. */
csw_status csw_swap_out_wait(csw_mgr* m, csw_ticket* t, csw_stream_t stream);

/* Swap-in (the fork's engine-side counterpart, implied by
 * CSWAP+/Execution.h:244-246,260-262,278-282,297-299): host -> device on the
 * H2D stream, decompress into d_dst on the codec stream, then make `compute`
 * wait for the result.  csw_prefetch starts the host -> device copy early. */
csw_status csw_prefetch(csw_mgr* m, csw_ticket* t);
csw_status csw_swap_in(csw_mgr* m, csw_ticket* t, float* d_dst, csw_stream_t compute);
/* The same in two halves, for bringing a tensor back before it is asked for:
 * csw_swap_in_start enqueues copy and decode into d_dst behind the work already
 * on `compute` (d_dst may still be in use by it) but does not make `compute`
 * wait; csw_swap_in_wait, called when the tensor is needed, makes `compute` wait
 * for the result.  csw_swap_in is the two back to back.  (No counterpart in the
 * reference, whose engine brings a tensor back when its consumer runs.) */
csw_status csw_swap_in_start(csw_mgr* m, csw_ticket* t, float* d_dst, csw_stream_t compute);
csw_status csw_swap_in_wait(csw_mgr* m, csw_ticket* t, csw_stream_t compute);
/* Give the ticket up.  Never blocks: its host and staging memory return to the
 * pools at once if no copy is in flight, else when a later call on the manager
 * finds them finished.  The handle is invalid afterwards. */
csw_status csw_ticket_release(csw_mgr* m, csw_ticket* t);
/* Raw copies out are handed to the copy stream a few at a time.  If this ticket's copy has
 * not been handed over yet it never will be: the ticket is released (the handle is dead
 * afterwards), *cancelled is 1 and the tensor it would have read is free to go at once.
 * Otherwise nothing happens and *cancelled is 0. */
csw_status csw_swap_out_cancel(csw_mgr* m, csw_ticket* t, int* cancelled);

typedef struct {
  int policy;            /* policy actually applied                       */
  size_t numel;
  size_t raw_bytes;      /* 4 * numel                                     */
  size_t moved_bytes;    /* bytes that crossed (or will cross) the link;
                            for sparse this is known once the count lands */
  int complete;          /* 1 once moved_bytes is final                   */
} csw_ticket_info;
csw_status csw_ticket_query(csw_mgr* m, csw_ticket* t, csw_ticket_info* info);

/* Self-describing form of a swapped-out tensor: a 64-byte header followed by
 * the payload exactly as it crossed the host link (raw floats, a ZFP stream, or
 * the packed sparse buffer).  The reference keeps rate, sizes and the sparse
 * side buffers only in live C++ objects (CSWAP+/Execution.h:98-102,115), so a
 * swapped tensor cannot outlive its process; a blob can be written to disk,
 * handed to another process or replica, and swapped in there. */
#define CSW_BLOB_MAGIC 0x50575343u /* "CSWP" */
#define CSW_BLOB_VERSION 1u
typedef struct {
  uint32_t magic, version;
  uint32_t policy;        /* CSW_POLICY_RAW / _SPARSE / _ZFP */
  uint32_t zfp_maxbits;   /* bits per zfp block, 0 unless policy is ZFP */
  uint64_t numel;         /* float32 elements of the tensor */
  uint64_t payload_bytes; /* bytes that follow the header */
  uint64_t nnz;           /* sparse: packed values; otherwise 0 */
  uint64_t reserved[3];
} csw_blob_header;        /* 64 bytes */
/* Copy header + payload of a ticket to dst (any host memory).  Waits for the
 * ticket's copy out to finish.  *bytes receives the size; with dst == NULL
 * only the size is reported.  CSW_ERR_SIZE if cap is too small. */
csw_status csw_ticket_export(csw_mgr* m, csw_ticket* t, void* dst, size_t cap, size_t* bytes);
/* Check a blob (magic, version, policy, sizes; for sparse payloads also that
 * every tile's segment lies inside the packed values) and return its header.
 * Needs no GPU. */
csw_status csw_blob_info(const void* blob, size_t bytes, csw_blob_header* header);
/* Turn a blob back into a ticket that lives in the manager's pinned pool, as
 * if the tensor had just been swapped out; csw_swap_in / csw_prefetch /
 * csw_ticket_release then work as usual.  Rejects blobs csw_blob_info rejects. */
csw_status csw_blob_import(csw_mgr* m, const void* blob, size_t bytes, csw_ticket** ticket);

typedef struct {
  uint64_t swap_outs, swap_ins;
  uint64_t raw_bytes_out, moved_bytes_out; /* uncompressed vs. on-link, swap-out */
  uint64_t raw_bytes_in, moved_bytes_in;   /* moved: what really crossed the link coming back */
  size_t pinned_in_use, pinned_high_water, staging_in_use, staging_high_water;
} csw_mgr_stats;
csw_status csw_mgr_get_stats(csw_mgr* m, csw_mgr_stats* s);
csw_status csw_mgr_reset_stats(csw_mgr* m);
/* Block the host until every queued swap-out and swap-in has finished; staged
   payloads kept for a quick return are dropped (afterwards every tensor swapped
   out is on the host only). */
csw_status csw_mgr_sync(csw_mgr* m);

/* ---- 5. cost model --------------------------------------------------------- */
/* Linear time models t = a + b * bytes (seconds, bytes of UNCOMPRESSED data)
 * for each codec direction, and link bandwidths in bytes/second. */
typedef struct {
  double zfp_enc_a, zfp_enc_b, zfp_dec_a, zfp_dec_b;         /* at the manager's maxbits */
  double sparse_enc_a, sparse_enc_b, sparse_dec_a, sparse_dec_b; /* at 50 % zeros        */
  double d2h_a, d2h_bps, h2d_a, h2d_bps;                     /* latency + bandwidth      */
  unsigned zfp_maxbits;
  /* per-byte slopes of the sparse codec at 75 % and 90 % zeros (the intercepts
   * are shared with the 50 % fit); 0 means "not fitted": the 50 % slope is used.
   * The decision interpolates between the three by the tensor's zero fraction. */
  double sparse_enc_b75, sparse_enc_b90, sparse_dec_b75, sparse_dec_b90;
  /* host time of one csw_swap_out + csw_ticket_release pair, seconds (what a
   * swapped tensor costs the thread that drives the model, whatever the policy) */
  double host_swap_s;
} csw_cost_model;

/* Measure the codecs and the host link on the manager's device (a few
 * hundred milliseconds; blocks until done).  model->zfp_maxbits selects the
 * ZFP rate to fit at and must be set on entry (0 means 512 = rate 8), so
 * zero-initialise the struct before the first call. */
csw_status csw_cost_fit(csw_mgr* m, csw_cost_model* model);

/* One swap candidate of the profiled iteration, in forward order (the inputs
 * the reference feeds its PolicyMaker: add_tensor / add_comptime / add_stepdep,
 * CSWAP+/Execution.h:224-233). */
typedef struct {
  size_t numel;
  double zero_fraction;   /* measured sparsity in [0,1]; <0 if unknown              */
  int lossy_ok;           /* 1 if ZFP may be applied to this tensor                 */
  double ready_s;         /* forward time (from its start) at which the tensor's
                             consumer runs, i.e. when its swap-out may begin        */
  double need_s;          /* backward compute (from its start) that runs before the
                             tensor is needed again                                 */
} csw_tensor_desc;

/* Choose per tensor a policy in {RAW, SPARSE, ZFP} so that the simulated stall
 * of one step (serial D2H link in forward order, serial H2D link with one step
 * of prefetch in backward order, codec times from the model) is smallest;
 * `fwd_total_s` is the forward pass's compute time.  Writes n codes to `policy`
 * and, if non-NULL, each tensor's modelled stall in seconds to `exposed`. */
csw_status csw_cost_decide(const csw_cost_model* model, const csw_tensor_desc* tensors, size_t n, double fwd_total_s,
                           int* policy, double* exposed);
/* The same simulation for a policy vector the caller supplies (KEEP, RAW,
 * SPARSE or ZFP per tensor): each tensor's modelled stall to `exposed` (may be
 * NULL) and their sum to *total_stall_s.  A choice the tensor does not allow
 * (ZFP on fewer than 1024 values, SPARSE without a zero fraction) counts as RAW.
 * Unlike the decision, this prediction knows that a raw or sparse tensor whose
 * copy out is still under way when backward asks for it is handed back as it
 * is (no copy in, no stall - and no memory freed). */
csw_status csw_cost_simulate(const csw_cost_model* model, const csw_tensor_desc* tensors, size_t n, double fwd_total_s,
                             const int* policy, double* exposed, double* total_stall_s);

/* ---- pinned host memory helpers (for callers without a CUDA binding) ------ */
csw_status csw_host_alloc(size_t bytes, void** p);
csw_status csw_host_free(void* p);

#ifdef __cplusplus
}
#endif
#endif /* CSWAP_B200_H */
