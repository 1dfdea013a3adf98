/*
 * CPU oracle for the compressed tensor-swap codecs.  TEST INFRASTRUCTURE ONLY:
 * used by tests/, by the smoke check and by the bench's CPU-baseline leg.  The
 * shipped CUDA library never links or calls this file.
 *
 * Restates, in plain C, the algorithms of ISCS-ZJU/CSWAP (CSWAP+/zfp): each
 * function names the reference file:line it follows.  The reference computes
 * on the GPU, where a 64-bit shift by 64 yields 0; the same shift is undefined
 * in C and x86 masks the count, so every such shift is made explicit here.
 */
#include "cswap_oracle.h"

#include <math.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------- */
/* bit I/O at absolute bit positions (encode.cuh:214-304, decode.cuh:39-125)  */
/* ------------------------------------------------------------------------- */

typedef struct {
  uint64_t* words;
  size_t pos; /* absolute bit position */
} bitcur;

static uint64_t low_mask(unsigned n) { return n >= 64 ? ~(uint64_t)0 : (((uint64_t)1 << n) - 1); }

/* append the low n (0..64) bits of v; the target bits must be zero beforehand
 * (the reference adds into a zeroed stream, encode.cuh:268-281) */
static void put_bits(bitcur* c, uint64_t v, unsigned n) {
  if (!n) return;
  v &= low_mask(n);
  size_t w = c->pos >> 6;
  unsigned s = (unsigned)(c->pos & 63);
  c->words[w] |= v << s;
  if (s && s + n > 64) c->words[w + 1] |= v >> (64 - s);
  c->pos += n;
}

static uint64_t get_bits(bitcur* c, unsigned n) {
  if (!n) return 0;
  size_t w = c->pos >> 6;
  unsigned s = (unsigned)(c->pos & 63);
  uint64_t v = c->words[w] >> s;
  if (s && s + n > 64) v |= c->words[w + 1] << (64 - s);
  c->pos += n;
  return v & low_mask(n);
}

/* ------------------------------------------------------------------------- */
/* block arithmetic                                                           */
/* ------------------------------------------------------------------------- */

/* sequency orders (constants.h:8-93 perm_3d, :97-100 perm_1, :106-131 perm_2),
 * entries are x + 4*y + 16*z */
static const unsigned char PERM3[64] = {
    0,  1,  4,  16, 20, 17, 5,  2,  8,  32, 21, 6,  18, 24, 9,  33,
    36, 3,  12, 48, 22, 25, 37, 40, 34, 10, 7,  19, 28, 13, 49, 52,
    41, 38, 26, 23, 29, 53, 11, 35, 44, 14, 50, 56, 42, 27, 39, 45,
    30, 54, 57, 60, 51, 15, 43, 46, 58, 61, 55, 31, 62, 59, 47, 63};
static const unsigned char PERM2[16] = {0, 1, 4, 5, 2, 8, 6, 9, 3, 12, 10, 7, 13, 11, 14, 15};
static const unsigned char PERM1[4] = {0, 1, 2, 3};

const unsigned char* orc_perm3(void) { return PERM3; }

static const unsigned char* perm_for(int dims) { return dims == 3 ? PERM3 : dims == 2 ? PERM2 : PERM1; }

/* encode.cuh:73-99 — the order of the halvings is part of the format */
void orc_fwd_lift(int32_t* p, unsigned s) {
  int32_t x = p[0], y = p[s], z = p[2 * s], w = p[3 * s];
  x += w; x >>= 1; w -= x;
  z += y; z >>= 1; y -= z;
  x += z; x >>= 1; z -= x;
  w += y; w >>= 1; y -= w;
  w += y >> 1; y -= w >> 1;
  p[0] = x; p[s] = y; p[2 * s] = z; p[3 * s] = w;
}

/* shared.h:221-250.  Left shifts are done on the unsigned pattern: values can
 * wrap for garbage streams and the GPU simply wraps. */
static int32_t shl1(int32_t v) { return (int32_t)((uint32_t)v << 1); }
void orc_inv_lift(int32_t* p, unsigned s) {
  int32_t x = p[0], y = p[s], z = p[2 * s], w = p[3 * s];
  y += w >> 1; w -= y >> 1;
  y += w; w = shl1(w); w -= y;
  z += x; x = shl1(x); x -= z;
  y += z; z = shl1(z); z -= y;
  w += x; x = shl1(x); x -= w;
  p[0] = x; p[s] = y; p[2 * s] = z; p[3 * s] = w;
}

/* encode.cuh:154-201 */
static void fwd_xform(int32_t* p, int dims) {
  unsigned x, y, z;
  if (dims == 3) {
    for (z = 0; z < 4; z++) for (y = 0; y < 4; y++) orc_fwd_lift(p + 4 * y + 16 * z, 1);
    for (x = 0; x < 4; x++) for (z = 0; z < 4; z++) orc_fwd_lift(p + 16 * z + x, 4);
    for (y = 0; y < 4; y++) for (x = 0; x < 4; x++) orc_fwd_lift(p + x + 4 * y, 16);
  } else if (dims == 2) {
    for (y = 0; y < 4; y++) orc_fwd_lift(p + 4 * y, 1);
    for (x = 0; x < 4; x++) orc_fwd_lift(p + x, 4);
  } else {
    orc_fwd_lift(p, 1);
  }
}

/* decode.cuh:184-226 */
static void inv_xform(int32_t* p, int dims) {
  unsigned x, y, z;
  if (dims == 3) {
    for (y = 0; y < 4; y++) for (x = 0; x < 4; x++) orc_inv_lift(p + x + 4 * y, 16);
    for (x = 0; x < 4; x++) for (z = 0; z < 4; z++) orc_inv_lift(p + 16 * z + x, 4);
    for (z = 0; z < 4; z++) for (y = 0; y < 4; y++) orc_inv_lift(p + 4 * y + 16 * z, 1);
  } else if (dims == 2) {
    for (x = 0; x < 4; x++) orc_inv_lift(p + x, 4);
    for (y = 0; y < 4; y++) orc_inv_lift(p + 4 * y, 1);
  } else {
    orc_inv_lift(p, 1);
  }
}

/* shared.h:176-181, decode.cuh:33-37 */
uint32_t orc_int2uint(int32_t x) { return ((uint32_t)x + 0xaaaaaaaau) ^ 0xaaaaaaaau; }
int32_t orc_uint2int(uint32_t x) { return (int32_t)((x ^ 0xaaaaaaaau) - 0xaaaaaaaau); }

/* encode.cuh:40-71: frexp exponent of the largest magnitude, floored at -126;
 * -127 for an all-zero block */
static int max_exponent(const float* p, int n) {
  float m = 0;
  for (int i = 0; i < n; i++) {
    float f = fabsf(p[i]);
    if (f > m) m = f;
  }
  int e = -127;
  if (m > 0) {
    frexpf(m, &e);
    if (e < -126) e = -126;
  }
  return e;
}

/* (int32) conversion of encode.cuh:147 with the semantics the GPU gives it
 * (cvt.rzi.s32.f32): truncation, saturation, NaN -> 0.  Only blocks whose
 * largest magnitude is below 2^-97 (scale factor overflows, encode.cuh:53)
 * ever leave the range. */
static int32_t cast_rz(float p) {
  if (p != p) return 0;
  if (p >= 2147483648.0f) return INT32_MAX;
  if (p <= -2147483648.0f) return INT32_MIN;
  return (int32_t)p;
}

/* encode.cuh:306-345 after the transform: embedded group-tested plane coder */
static int encode_planes(bitcur* c, const uint32_t* u, int size, unsigned budget) {
  unsigned bits = budget, n = 0, k;
  int nmax = 0;
  for (k = 32; bits && k-- > 0;) {
    uint64_t x = 0;
    for (int i = 0; i < size; i++) x += (uint64_t)((u[i] >> k) & 1u) << i;
    unsigned m = n < bits ? n : bits;
    bits -= m;
    put_bits(c, x, m);
    x = m >= 64 ? 0 : x >> m; /* GPU: shift by 64 gives 0 (encode.cuh:281) */
    for (; n < (unsigned)size && bits; x >>= 1, n++) {
      bits--;
      put_bits(c, x != 0, 1);
      if (!x) break;
      for (; n < (unsigned)size - 1 && bits; x >>= 1, n++) {
        bits--;
        put_bits(c, x & 1u, 1);
        if (x & 1u) break;
      }
    }
    if ((int)n > nmax) nmax = (int)n;
  }
  return nmax;
}

/* decode.cuh:127-179 */
static void decode_planes(bitcur* c, uint32_t* u, int size, unsigned budget) {
  unsigned bits = budget, n = 0, k;
  memset(u, 0, (size_t)size * sizeof(uint32_t));
  for (k = 32; bits && k-- > 0;) {
    unsigned m = n < bits ? n : bits;
    bits -= m;
    uint64_t x = get_bits(c, m);
    for (; bits && n < (unsigned)size; n++) {
      bits--;
      if (get_bits(c, 1)) {
        for (; bits && n < (unsigned)size - 1; n++) {
          bits--;
          if (get_bits(c, 1)) break;
        }
        x += (uint64_t)1 << n;
      } else {
        break;
      }
    }
    for (int i = 0; i < size; i++, x >>= 1) u[i] += (uint32_t)(x & 1u) << k;
  }
}

/* encode.cuh:347-368 */
int orc_zfp_encode_block(const float* fblock, int dims, unsigned maxbits, size_t block_idx,
                         uint64_t* stream) {
  const int size = 1 << (2 * dims);
  bitcur c = {stream, block_idx * (size_t)maxbits};
  int emax = max_exponent(fblock, size);
  /* precision() (encode.cuh:10-15) is min(32, max(0, emax + 1074 + 8)) = 32 */
  unsigned e = (unsigned)(emax + 127);
  if (!e) return 0;
  put_bits(&c, 2 * e + 1, 9);
  int32_t iblock[64];
  uint32_t ublock[64];
  float s = ldexpf(1.0f, 30 - emax); /* encode.cuh:125-131 */
  for (int i = 0; i < size; i++) iblock[i] = cast_rz(s * fblock[i]);
  fwd_xform(iblock, dims);
  const unsigned char* perm = perm_for(dims);
  for (int i = 0; i < size; i++) ublock[i] = orc_int2uint(iblock[perm[i]]);
  return encode_planes(&c, ublock, size, maxbits - 9);
}

/* decode.cuh:228-288; the caller's block starts as zeros (decode3.cuh:72-73) */
void orc_zfp_decode_block(const uint64_t* stream, int dims, unsigned maxbits, size_t block_idx,
                          float* fblock) {
  const int size = 1 << (2 * dims);
  bitcur c = {(uint64_t*)stream, block_idx * (size_t)maxbits};
  memset(fblock, 0, (size_t)size * sizeof(float));
  if (!get_bits(&c, 1)) return;
  int emax = (int)get_bits(&c, 8) - 127;
  uint32_t ublock[64];
  int32_t iblock[64];
  decode_planes(&c, ublock, size, maxbits - 9);
  const unsigned char* perm = perm_for(dims);
  for (int i = 0; i < size; i++) iblock[perm[i]] = orc_uint2int(ublock[i]);
  inv_xform(iblock, dims);
  float w = ldexpf(1.0f, emax - 30); /* shared.h:197-203 */
  for (int i = 0; i < size; i++) fblock[i] = w * (float)iblock[i];
}

/* ------------------------------------------------------------------------- */
/* whole fields                                                               */
/* ------------------------------------------------------------------------- */

static int field_dims(size_t ny, size_t nz) { return nz ? 3 : ny ? 2 : 1; }

size_t orc_zfp_stream_bytes(size_t nx, size_t ny, size_t nz, unsigned maxbits) {
  int d = field_dims(ny, nz);
  size_t bx = (nx + 3) / 4, by = d >= 2 ? (ny + 3) / 4 : 1, bz = d >= 3 ? (nz + 3) / 4 : 1;
  /* Whole words covering every block.  The reference's own byte counts
   * (shared.h:39-84) truncate for 3-D and count unpadded values for 1-D/2-D;
   * they agree with this whenever maxbits % 64 == 0 and no block is partial. */
  return (bx * by * bz * maxbits + 63) / 64 * 8;
}

/* encode.cuh:17-38 */
static void pad_block(float* p, unsigned n, unsigned s) {
  switch (n) {
    case 0: p[0] = 0; /* fallthrough */
    case 1: p[s] = p[0]; /* fallthrough */
    case 2: p[2 * s] = p[s]; /* fallthrough */
    case 3: p[3 * s] = p[0]; /* fallthrough */
    default: break;
  }
}

typedef struct {
  size_t nx, ny, nz, bx, by, bz;
  int dims;
} geom;

static geom make_geom(size_t nx, size_t ny, size_t nz) {
  geom g;
  g.nx = nx; g.ny = ny; g.nz = nz;
  g.dims = field_dims(ny, nz);
  g.bx = (nx + 3) / 4;
  g.by = g.dims >= 2 ? (ny + 3) / 4 : 1;
  g.bz = g.dims >= 3 ? (nz + 3) / 4 : 1;
  return g;
}

/* block index -> origin (encode3.cuh:78-90, encode2.cuh, encode1.cuh) and
 * gather with replicate padding (encode3.cuh:12-47) */
static void gather(const geom* g, const float* in, size_t b, float* q) {
  size_t x0 = (b % g->bx) * 4, y0 = ((b / g->bx) % g->by) * 4, z0 = (b / (g->bx * g->by)) * 4;
  unsigned vx = g->nx - x0 < 4 ? (unsigned)(g->nx - x0) : 4;
  unsigned vy = g->dims >= 2 ? (g->ny - y0 < 4 ? (unsigned)(g->ny - y0) : 4) : 1;
  unsigned vz = g->dims >= 3 ? (g->nz - z0 < 4 ? (unsigned)(g->nz - z0) : 4) : 1;
  size_t sy = g->nx, sz = g->nx * (g->dims >= 2 ? g->ny : 1);
  for (unsigned z = 0; z < vz; z++) {
    for (unsigned y = 0; y < vy; y++) {
      for (unsigned x = 0; x < vx; x++)
        q[16 * z + 4 * y + x] = in[(z0 + z) * sz + (y0 + y) * sy + x0 + x];
      pad_block(q + 16 * z + 4 * y, vx, 1);
    }
    if (g->dims >= 2)
      for (unsigned x = 0; x < 4; x++) pad_block(q + 16 * z + x, vy, 4);
  }
  if (g->dims >= 3)
    for (unsigned y = 0; y < 4; y++)
      for (unsigned x = 0; x < 4; x++) pad_block(q + 4 * y + x, vz, 16);
}

/* decode3.cuh:10-39 */
static void scatter(const geom* g, float* out, size_t b, const float* q) {
  size_t x0 = (b % g->bx) * 4, y0 = ((b / g->bx) % g->by) * 4, z0 = (b / (g->bx * g->by)) * 4;
  unsigned vx = g->nx - x0 < 4 ? (unsigned)(g->nx - x0) : 4;
  unsigned vy = g->dims >= 2 ? (g->ny - y0 < 4 ? (unsigned)(g->ny - y0) : 4) : 1;
  unsigned vz = g->dims >= 3 ? (g->nz - z0 < 4 ? (unsigned)(g->nz - z0) : 4) : 1;
  size_t sy = g->nx, sz = g->nx * (g->dims >= 2 ? g->ny : 1);
  for (unsigned z = 0; z < vz; z++)
    for (unsigned y = 0; y < vy; y++)
      for (unsigned x = 0; x < vx; x++)
        out[(z0 + z) * sz + (y0 + y) * sy + x0 + x] = q[16 * z + 4 * y + x];
}

size_t orc_zfp_encode(const float* in, size_t nx, size_t ny, size_t nz, unsigned maxbits,
                      uint64_t* out, int threads) {
  geom g = make_geom(nx, ny, nz);
  size_t blocks = g.bx * g.by * g.bz;
  size_t bytes = orc_zfp_stream_bytes(nx, ny, nz, maxbits);
  memset(out, 0, bytes + 8);
  long long nb = (long long)blocks;
  if (maxbits % 64) threads = 1; /* neighbouring blocks share words */
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
  for (long long b = 0; b < nb; b++) {
    float q[64];
    gather(&g, in, (size_t)b, q);
    orc_zfp_encode_block(q, g.dims, maxbits, (size_t)b, out);
  }
  (void)threads;
  return bytes;
}

void orc_zfp_decode(const uint64_t* in, size_t nx, size_t ny, size_t nz, unsigned maxbits,
                    float* out, int threads) {
  geom g = make_geom(nx, ny, nz);
  long long nb = (long long)(g.bx * g.by * g.bz);
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
  for (long long b = 0; b < nb; b++) {
    float q[64];
    orc_zfp_decode_block(in, g.dims, maxbits, (size_t)b, q);
    scatter(&g, out, (size_t)b, q);
  }
  (void)threads;
}

/* ------------------------------------------------------------------------- */
/* sparse codec, native layout                                                */
/* ------------------------------------------------------------------------- */

#define ORC_TILE 4096

size_t orc_sparse_compress(const float* in, size_t n, uint32_t* bitmap, float* values,
                           uint32_t* tile_off, int threads) {
  const uint32_t* bits = (const uint32_t*)in;
  size_t tiles = (n + ORC_TILE - 1) / ORC_TILE;
  long long nt = (long long)tiles;
  /* pass 1: bitmap + per-tile counts */
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
  for (long long t = 0; t < nt; t++) {
    size_t lo = (size_t)t * ORC_TILE, hi = lo + ORC_TILE < n ? lo + ORC_TILE : n;
    uint32_t cnt = 0;
    for (size_t w = lo / 32; w * 32 < hi; w++) {
      uint32_t word = 0;
      for (unsigned j = 0; j < 32 && w * 32 + j < hi; j++)
        if (bits[w * 32 + j]) { word |= 1u << j; cnt++; }
      bitmap[w] = word;
    }
    tile_off[t] = cnt;
  }
  size_t total = 0;
  for (size_t t = 0; t < tiles; t++) { uint32_t c = tile_off[t]; tile_off[t] = (uint32_t)total; total += c; }
  /* pass 2: pack */
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#endif
  for (long long t = 0; t < nt; t++) {
    size_t lo = (size_t)t * ORC_TILE, hi = lo + ORC_TILE < n ? lo + ORC_TILE : n;
    size_t o = tile_off[t];
    for (size_t i = lo; i < hi; i++)
      if (bits[i]) values[o++] = in[i];
  }
  (void)threads;
  return total;
}

void orc_sparse_decompress(const uint32_t* bitmap, const float* values, size_t n, float* out,
                           int threads) {
  size_t tiles = (n + ORC_TILE - 1) / ORC_TILE;
  /* tile offsets are recomputed from the bitmap so the function is total */
  size_t o = 0;
  (void)threads;
  for (size_t t = 0; t < tiles; t++) {
    size_t lo = t * ORC_TILE, hi = lo + ORC_TILE < n ? lo + ORC_TILE : n;
    for (size_t i = lo; i < hi; i++) {
      if ((bitmap[i >> 5] >> (i & 31)) & 1u) out[i] = values[o++];
      else out[i] = 0.0f;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* sparse codec, reference layout                                             */
/* ------------------------------------------------------------------------- */

static int ceil_div(int a, int b) { return a % b == 0 ? a / b : a / b + 1; }

/* compression.cu:134-165 (count), :9-19 (serial scan over the first
 * ceil(n/chunk) workers, Execution.h:90), :168-239 (bitmap + pack) */
size_t orc_legacy_sparse_compress(const float* in, int n, int P, int32_t* begin, uint32_t* bitmap,
                                  float* values) {
  int chunk = ceil_div(n, P);
  /* Execution.h:90 computes the scan length in floating point */
  int active = (int)ceil((float)n / ceil((float)n / P));
  int words_per = ceil_div(chunk, 32);
  for (int i = 0; i < P; i++) {
    int lo = chunk * i, hi = lo + chunk;
    if (lo >= n) continue; /* the reference leaves begin[i] unwritten */
    if (hi > n) hi = n;
    int cnt = 0;
    for (int j = lo; j < hi; j++) if (in[j] != 0) cnt++;
    begin[i] = cnt;
  }
  for (int i = 1; i < active; i++) begin[i] += begin[i - 1];
  int total = begin[active - 1];
  for (int i = active - 1; i > 0; i--) begin[i] = begin[i - 1];
  begin[0] = 0;
  for (int i = 0; i < P; i++) {
    int lo = chunk * i, hi = lo + chunk;
    if (lo >= n) continue;
    if (hi > n) hi = n;
    int o = begin[i], cursor = 0, bw = i * words_per;
    uint32_t word = 0;
    for (int j = lo; j < hi; j++) {
      if (cursor == 32) { bitmap[bw++] = word; word = 0; cursor = 0; }
      if (in[j] != 0) { word |= 1u << cursor; values[o++] = in[j]; }
      cursor++;
    }
    bitmap[bw] = word; /* trailing (possibly full) word, compression.cu:229-236 */
  }
  return (size_t)total;
}

/* compression.cu:241-318 */
void orc_legacy_sparse_decompress(const float* values, float* out, int n, int P,
                                  const uint32_t* bitmap, const int32_t* begin) {
  int chunk = ceil_div(n, P);
  int words_per = ceil_div(chunk, 32);
  for (int i = 0; i < P; i++) {
    if ((long long)chunk * i >= n) continue;
    int w = words_per * i, wend = w + words_per;
    int rd = begin[i], k = 0, wr;
    for (; w < wend - 1; w++, k++) {
      uint32_t t = bitmap[w];
      wr = chunk * i + k * 32;
      while (t) {
        out[wr++] = (t & 1u) ? values[rd++] : 0.0f;
        t >>= 1;
      }
    }
    int end = (i + 1) * chunk;
    if (end < n) end = n; /* sic: compression.cu:296-298 widens instead of clamping */
    uint32_t t = bitmap[w];
    wr = chunk * i + k * 32;
    while (t) {
      if (wr == end) break;
      out[wr++] = (t & 1u) ? values[rd++] : 0.0f;
      t >>= 1;
    }
  }
}

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
