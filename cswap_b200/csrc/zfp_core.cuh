// Block-level arithmetic of the fixed-rate ZFP float32 codec, written for one
// thread holding one whole block in registers (lane = block).
//
// Format follows cuZFP as vendored by CSWAP+ (CSWAP+/zfp/encode.cuh:306-368,
// decode.cuh:127-288, shared.h:176-250, constants.h:8-131): 1 flag bit + 8-bit
// biased block exponent, block-floating-point cast to int32, passes of the
// 4-point lifting transform, sequency reorder + negabinary, then the embedded
// group-tested bit-plane coder cut at `maxbits` bits per block.
//
// What differs from the reference is only how the same bits are produced:
//  * bit planes come from 8x8 bit-matrix transposes of the coefficient bytes
//    (PRMT gathers + 3 masked swap stages), eight planes at a time, instead of
//    a 64-step gather per plane;
//  * the group-test phase of a plane is expanded (encoder) or parsed (decoder)
//    eight positions / stream bits per step through small tables held in
//    shared memory instead of one stream bit per step;
//  * coded bits are assembled in a 64-bit register window and leave as whole
//    32-bit words - no atomics and no pre-zeroed output.
//
// Everything here is plain scalar code per block, so the same header also
// compiles for the host (tests drive it lane by lane against the CPU oracle).
#pragma once
#include <cstdint>
#include <utility>

#if defined(__CUDACC__)
#define CSW_HD __host__ __device__ __forceinline__
#else
#define CSW_HD inline
#endif

namespace csw {

// ---- portable intrinsics ------------------------------------------------------
CSW_HD uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t s) {
#if defined(__CUDA_ARCH__)
  return __byte_perm(a, b, s);
#else
  uint64_t ab = ((uint64_t)b << 32) | a;
  uint32_t r = 0;
  for (int i = 0; i < 4; i++) r |= (uint32_t)((ab >> (8 * ((s >> (4 * i)) & 7))) & 0xff) << (8 * i);
  return r;
#endif
}
CSW_HD int clz64(uint64_t x) {
#if defined(__CUDA_ARCH__)
  return __clzll((long long)x);
#else
  return x ? __builtin_clzll(x) : 64;
#endif
}
CSW_HD int clz32(uint32_t x) {
#if defined(__CUDA_ARCH__)
  return __clz((int)x);
#else
  return x ? __builtin_clz(x) : 32;
#endif
}
CSW_HD int popc32(uint32_t x) {
#if defined(__CUDA_ARCH__)
  return __popc(x);
#else
  return __builtin_popcount(x);
#endif
}
CSW_HD uint32_t f2u(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  union { float f; uint32_t u; } c; c.f = f; return c.u;
#endif
}
CSW_HD float u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  union { float f; uint32_t u; } c; c.u = u; return c.f;
#endif
}
// float -> int32, round toward zero, saturating, NaN -> 0 (cvt.rzi.s32.f32)
CSW_HD int f2i_rz(float f) {
#if defined(__CUDA_ARCH__)
  return __float2int_rz(f);
#else
  if (f != f) return 0;
  if (f >= 2147483648.0f) return 2147483647;
  if (f <= -2147483648.0f) return (int)0x80000000;
  return (int)f;
#endif
}
// true when the predicate holds on every active lane of the warp (host: the one "lane")
CSW_HD bool warp_all(bool p) {
#if defined(__CUDA_ARCH__)
  return __all_sync(__activemask(), p);
#else
  return p;
#endif
}
// smallest value over the lanes of the warp, all of which must call (host: the one "lane")
CSW_HD int warp_min(int v) {
#if defined(__CUDA_ARCH__)
  return __reduce_min_sync(0xffffffffu, v);
#else
  return v;
#endif
}
CSW_HD int ctz32(uint32_t x) {  // x != 0
#if defined(__CUDA_ARCH__)
  return __ffs((int)x) - 1;
#else
  return __builtin_ctz(x);
#endif
}
CSW_HD uint32_t low_mask32(int n) {  // n in 0..32
  return n >= 32 ? 0xffffffffu : ((1u << n) - 1u);
}

// ---- sequency order (constants.h:8-131), entries are x + 4y + 16z ---------------
constexpr int perm3(int i) {
  constexpr unsigned char t[64] = {
      0,  1,  4,  16, 20, 17, 5,  2,  8,  32, 21, 6,  18, 24, 9,  33,
      36, 3,  12, 48, 22, 25, 37, 40, 34, 10, 7,  19, 28, 13, 49, 52,
      41, 38, 26, 23, 29, 53, 11, 35, 44, 14, 50, 56, 42, 27, 39, 45,
      30, 54, 57, 60, 51, 15, 43, 46, 58, 61, 55, 31, 62, 59, 47, 63};
  return t[i];
}
constexpr int perm2(int i) {
  constexpr unsigned char t[16] = {0, 1, 4, 5, 2, 8, 6, 9, 3, 12, 10, 7, 13, 11, 14, 15};
  return t[i];
}
template <int DIMS, int I>
struct PermAt {
  static constexpr int v = DIMS == 3 ? perm3(I & 63) : DIMS == 2 ? perm2(I & 15) : I;
};

// ---- lifting (encode.cuh:73-99, shared.h:221-250) --------------------------------
// Arithmetic is done on unsigned patterns where C++ would overflow; the GPU
// reference simply wraps.
CSW_HD int wadd(int a, int b) { return (int)((uint32_t)a + (uint32_t)b); }
CSW_HD int wsub(int a, int b) { return (int)((uint32_t)a - (uint32_t)b); }
CSW_HD void fwd_lift(int& x, int& y, int& z, int& w) {
  x = wadd(x, w); x >>= 1; w = wsub(w, x);
  z = wadd(z, y); z >>= 1; y = wsub(y, z);
  x = wadd(x, z); x >>= 1; z = wsub(z, x);
  w = wadd(w, y); w >>= 1; y = wsub(y, w);
  w = wadd(w, y >> 1); y = wsub(y, w >> 1);
}
CSW_HD int twice_minus(int a, int b) { return (int)(((uint32_t)a << 1) - (uint32_t)b); }
CSW_HD void inv_lift(int& x, int& y, int& z, int& w) {
  y = wadd(y, w >> 1); w = wsub(w, y >> 1);
  y = wadd(y, w); w = twice_minus(w, y);
  z = wadd(z, x); x = twice_minus(x, z);
  y = wadd(y, z); z = twice_minus(z, y);
  w = wadd(w, x); x = twice_minus(x, w);
}

template <int DIMS>
CSW_HD void fwd_xform(int (&v)[1 << (2 * DIMS)]) {
  if constexpr (DIMS == 3) {
#pragma unroll
    for (int i = 0; i < 16; i++) fwd_lift(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
#pragma unroll
    for (int z = 0; z < 4; z++)
#pragma unroll
      for (int x = 0; x < 4; x++)
        fwd_lift(v[16 * z + x], v[16 * z + x + 4], v[16 * z + x + 8], v[16 * z + x + 12]);
#pragma unroll
    for (int i = 0; i < 16; i++) fwd_lift(v[i], v[i + 16], v[i + 32], v[i + 48]);
  } else if constexpr (DIMS == 2) {
#pragma unroll
    for (int y = 0; y < 4; y++) fwd_lift(v[4 * y], v[4 * y + 1], v[4 * y + 2], v[4 * y + 3]);
#pragma unroll
    for (int x = 0; x < 4; x++) fwd_lift(v[x], v[x + 4], v[x + 8], v[x + 12]);
  } else {
    fwd_lift(v[0], v[1], v[2], v[3]);
  }
}

template <int DIMS>
CSW_HD void inv_xform(int (&v)[1 << (2 * DIMS)]) {
  if constexpr (DIMS == 3) {
#pragma unroll
    for (int i = 0; i < 16; i++) inv_lift(v[i], v[i + 16], v[i + 32], v[i + 48]);
#pragma unroll
    for (int z = 0; z < 4; z++)
#pragma unroll
      for (int x = 0; x < 4; x++)
        inv_lift(v[16 * z + x], v[16 * z + x + 4], v[16 * z + x + 8], v[16 * z + x + 12]);
#pragma unroll
    for (int i = 0; i < 16; i++) inv_lift(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else if constexpr (DIMS == 2) {
#pragma unroll
    for (int x = 0; x < 4; x++) inv_lift(v[x], v[x + 4], v[x + 8], v[x + 12]);
#pragma unroll
    for (int y = 0; y < 4; y++) inv_lift(v[4 * y], v[4 * y + 1], v[4 * y + 2], v[4 * y + 3]);
  } else {
    inv_lift(v[0], v[1], v[2], v[3]);
  }
}

// ---- negabinary (shared.h:176-181, decode.cuh:33-37) ------------------------------
CSW_HD uint32_t int2uint(int x) { return ((uint32_t)x + 0xaaaaaaaau) ^ 0xaaaaaaaau; }
CSW_HD int uint2int(uint32_t x) { return (int)((x ^ 0xaaaaaaaau) - 0xaaaaaaaau); }

template <int DIMS, int... I>
CSW_HD void fwd_order(const int (&v)[sizeof...(I)], uint32_t (&u)[sizeof...(I)], std::integer_sequence<int, I...>) {
  ((u[I] = int2uint(v[PermAt<DIMS, I>::v])), ...);
}
template <int DIMS, int... I>
CSW_HD void inv_order(const uint32_t (&u)[sizeof...(I)], int (&v)[sizeof...(I)], std::integer_sequence<int, I...>) {
  ((v[PermAt<DIMS, I>::v] = uint2int(u[I])), ...);
}

// ---- block exponent and cast (encode.cuh:40-71,120-149) ---------------------------
// Biased exponent field e = emax + 127 (0 for an all-zero block) from the bit
// pattern of max|v|: frexp's exponent of a normal float with exponent field E
// is E - 126, and denormals are floored at -126 (field 1).
CSW_HD uint32_t biased_emax(float maxabs) {
  uint32_t b = f2u(maxabs);
  return b == 0 ? 0u : (b >> 23) + 1u;
}
// 2^(30 - emax) as a float; +inf for emax < -97, exactly what the reference's
// ldexp-then-narrow yields, so with the saturating conversion such
// (denormal-range) blocks code the way the reference codes them on a GPU.
CSW_HD float quant_scale(uint32_t e) {
  int f = 284 - (int)e;  // exponent field of 2^(30-emax), emax = e - 127
  f = f > 255 ? 255 : f;
  return u2f((uint32_t)f << 23);
}
// 2^(emax - 30) (shared.h:197-203, decode.cuh:278); denormal below emax = -96.
CSW_HD float dequant_scale(uint32_t e) {
  int f = (int)e - 30;  // exponent field of 2^(emax-30) = e - 127 - 30 + 127
  if (f >= 1) return u2f((uint32_t)f << 23);
  return f > -23 ? u2f(1u << (22 + f)) : 0.0f;  // denormal results of ldexp
}

// ---- 8-plane slices by bit-matrix transpose ---------------------------------------
// One masked swap of an 8x8 (per byte lane) bit transpose.
template <int S, uint32_t M>
CSW_HD void tswap(uint32_t& a, uint32_t& b) {
  uint32_t na = (a & M) | ((b << S) & ~M);
  uint32_t nb = ((a >> S) & M) | (b & ~M);
  a = na;
  b = nb;
}
// In every byte lane: bit k of word j <-> bit j of word k.  Its own inverse.
CSW_HD void transpose8(uint32_t (&r)[8]) {
#pragma unroll
  for (int j = 0; j < 4; j++) tswap<4, 0x0f0f0f0fu>(r[j], r[j + 4]);
#pragma unroll
  for (int j = 0; j < 8; j += 4) {
    tswap<2, 0x33333333u>(r[j], r[j + 2]);
    tswap<2, 0x33333333u>(r[j + 1], r[j + 3]);
  }
#pragma unroll
  for (int j = 0; j < 8; j += 2) tswap<1, 0x55555555u>(r[j], r[j + 1]);
}

// p[k] (k = 0..7) <- bit (8c + k) of coefficients 32G .. 32G+31, coefficient
// 32G + i at bit i.  Byte m of gather word j holds coefficient 8m + j, so after
// the transpose bit 8m + j of a plane word is coefficient 8m + j.
// sel = c | (4 + c) << 4 picks byte c of both PRMT operands.
template <int G, int N>
CSW_HD void planes_of_byte(const uint32_t (&u)[N], uint32_t sel, uint32_t (&p)[8]) {
  static_assert(N == 64 || N == 16 || N == 4, "block size");
#pragma unroll
  for (int j = 0; j < 8; j++) {
    if constexpr (N == 64) {
      uint32_t t0 = byte_perm(u[32 * G + j], u[32 * G + 8 + j], sel);
      uint32_t t1 = byte_perm(u[32 * G + 16 + j], u[32 * G + 24 + j], sel);
      p[j] = byte_perm(t0, t1, 0x5410);
    } else if constexpr (N == 16) {
      p[j] = byte_perm(u[j], u[8 + j], sel) & 0xffffu;
    } else {
      p[j] = j < 4 ? (byte_perm(u[j & 3], 0, sel) & 0xffu) : 0u;
    }
  }
  transpose8(p);
}

// Inverse: write byte c of each coefficient from eight plane words.
// sel0 keeps the other three bytes of the destination and takes byte 0 of the
// second PRMT operand into byte c; adding m << 4c takes byte m instead.
template <int G, int N>
CSW_HD void bytes_from_planes(uint32_t (&p)[8], uint32_t sel0, uint32_t step, uint32_t (&u)[N]) {
  transpose8(p);
#pragma unroll
  for (int j = 0; j < 8; j++) {
    if constexpr (N == 64) {
#pragma unroll
      for (int m = 0; m < 4; m++) u[32 * G + 8 * m + j] = byte_perm(u[32 * G + 8 * m + j], p[j], sel0 + m * step);
    } else if constexpr (N == 16) {
      u[j] = byte_perm(u[j], p[j], sel0);
      u[8 + j] = byte_perm(u[8 + j], p[j], sel0 + step);
    } else {
      if (j < 4) u[j & 3] = byte_perm(u[j & 3], p[j], sel0);
    }
  }
}

// ---- coder tables -----------------------------------------------------------------
// Encoder: entry for the eight positions v of a plane word past the already
// significant prefix.  Each 0 position codes as '0'; each 1 position codes as
// '1' followed by the next group-test bit, which is '1' whenever a later set
// bit exists.  bits 0..15: that pattern; bits 16..20: its length 8 + popc(v);
// bits 24..28: length when the byte holds the last set bit of the plane
// (positions up to the top set bit, plus one per set bit; the final group-test
// bit is then the '0' terminator).
constexpr int ENC_LUT_SIZE = 256;
constexpr CSW_HD uint32_t enc_lut_entry(uint32_t v) {
  uint32_t pat = 0;
  int len = 0, top = -1, ones = 0;
  for (int i = 0; i < 8; i++) {
    if ((v >> i) & 1u) {
      pat |= 3u << len;
      len += 2;
      top = i;
      ones++;
    } else {
      len += 1;
    }
  }
  uint32_t lf = top < 0 ? 0u : (uint32_t)(top + 1 + ones);
  return pat | ((uint32_t)len << 16) | (lf << 24);
}

// Decoder: entry for (limit L in 0..8, state, next stream byte).  Simulates the
// group-test parser of decode.cuh:147-164 over at most L stream bits.
// State 0: expecting a group-test bit; state 1: inside a unary run (expecting
// value bits until a one); state 2: negative group test seen, plane finished.
// L = 0 (no open position left, or the budget is spent) finishes the plane
// without reading: from state 1 the run's final one is implied.
// One field per byte, so that each is a single byte-permute away:
// byte 0: stream bits consumed; byte 1: positions advanced;
// byte 2: plane bits found, relative to the starting position;
// byte 3: state afterwards.
constexpr int DEC_LUT_SIZE = 9 * 2 * 256;
constexpr CSW_HD int dec_lut_index(int L, int state, uint32_t byte) { return (L * 2 + state) * 256 + (int)byte; }
constexpr CSW_HD uint32_t dec_lut_entry(int idx) {
  uint32_t byte = idx & 255;
  int st = (idx >> 8) & 1, L = idx >> 9;
  int c = 0, dn = 0;
  uint32_t pat = 0;
  if (L == 0) {
    if (st == 1) { pat = 1u; dn = 1; }
    st = 2;
  }
  while (c < L) {
    uint32_t bit = (byte >> c) & 1u;
    c++;
    if (st == 0) {
      if (bit) st = 1;
      else { st = 2; break; }
    } else {
      if (bit) { pat |= 1u << dn; st = 0; }
      dn++;
    }
  }
  return (uint32_t)c | ((uint32_t)dn << 8) | (pat << 16) | ((uint32_t)st << 24);
}
CSW_HD int dec_lut_used(uint32_t e) { return (int)(e & 0xffu); }
CSW_HD int dec_lut_advance(uint32_t e) { return (int)byte_perm(e, 0u, 0x4441u); }
CSW_HD uint32_t dec_lut_pattern(uint32_t e) { return byte_perm(e, 0u, 0x4442u); }
CSW_HD int dec_lut_state(uint32_t e) { return (int)(e >> 24); }

// ---- bit emitter ------------------------------------------------------------------
// WordSink::put(w, word) receives the block's w-th 32-bit stream word; words
// arrive in increasing w, each once.  Everything is written for predication
// rather than branches: lanes of a warp code different blocks and would
// otherwise diverge on every word boundary.
CSW_HD uint32_t funnel_l(uint32_t lo, uint32_t hi, int s) {  // ((hi:lo) << s) >> 32, s taken mod 32
#if defined(__CUDA_ARCH__)
  return __funnelshift_l(lo, hi, s);
#else
  return (uint32_t)(((((uint64_t)hi << 32) | lo) << (s & 31)) >> 32);
#endif
}
CSW_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, int s) {  // low word of (hi:lo) >> s, s taken mod 32
#if defined(__CUDA_ARCH__)
  return __funnelshift_r(lo, hi, s);
#else
  return (uint32_t)((((uint64_t)hi << 32) | lo) >> (s & 31));
#endif
}

template <class WordSink>
struct Emitter {
  uint32_t a0;  // the word being filled; bits at and above `fill` are zero
  int fill;     // 0..31
  int wpos;     // words already handed to the sink
  int nwords;   // ceil(maxbits / 32)
  WordSink& sink;
  CSW_HD Emitter(WordSink& s, int nw) : a0(0), fill(0), wpos(0), nwords(nw), sink(s) {}
  CSW_HD int total() const { return 32 * wpos + fill; }
  CSW_HD void flush_word(uint32_t next) {
    if (wpos < nwords) sink.put(wpos, a0);
    wpos++;
    a0 = next;
  }
  // append the low `len` (0..32) bits of v; bits of v at and above len must be zero
  CSW_HD void emit32(uint32_t v, int len) {
    const uint32_t t1 = funnel_l(v, 0u, fill);
    a0 |= v << fill;
    int nf = fill + len;
    if (nf >= 32) {
      flush_word(t1);
      nf -= 32;
    }
    fill = nf;
  }
  // append the low `len` (0..64) bits of hi:lo; bits at and above len must be zero
  CSW_HD void emit64(uint32_t lo, uint32_t hi, int len) {
    uint32_t t1 = funnel_l(lo, hi, fill);
    const uint32_t t2 = funnel_l(hi, 0u, fill);
    a0 |= lo << fill;
    int nf = fill + len;
    if (nf >= 32) {
      flush_word(t1);
      t1 = t2;
      nf -= 32;
    }
    if (nf >= 32) {
      flush_word(t1);
      nf -= 32;
    }
    fill = nf;
  }
  // hand over whatever is buffered and zero-fill the rest of the block
  CSW_HD void finish() {
    while (wpos < nwords) flush_word(0u);
  }
};

// ---- encoder: coefficient-count state ----------------------------------------------
// n coefficients are significant so far; the masks select plane bits below n
// and the single bit at position n (zero when n == 64).
struct SigState {
  int n;
  uint32_t mlo, mhi;  // low n bits of a 64-bit plane word
  uint32_t glo, ghi;  // bit n
  CSW_HD void set(int nn) {
    n = nn;
    mlo = nn >= 32 ? 0xffffffffu : ((1u << nn) - 1u);
    mhi = nn <= 32 ? 0u : low_mask32(nn - 32);
    glo = nn < 32 ? (1u << nn) : 0u;
    ghi = (nn >= 32 && nn < 64) ? (1u << (nn - 32)) : 0u;
  }
};

// ---- encoder: one plane -----------------------------------------------------------
// Codes plane word hi:lo (coefficient i at bit i, N coefficients) given the
// significance state (encode.cuh:336-343).  Emission ignores the bit budget:
// the stream is an exact prefix of the unlimited-budget stream, so the caller
// stops once total() reaches maxbits and the emitter drops the overrun.
//
// The first group-test bit rides on the verbatim prefix (it is bit n of the
// same word).  The rest of the group-test phase is produced eight positions
// per step from enc_lut; the loop body has no branches, so lanes only differ
// in how many steps they take.
template <int N, class WordSink>
CSW_HD void encode_plane(uint32_t lo, uint32_t hi, SigState& sg, Emitter<WordSink>& em, const uint32_t* enc_lut) {
  if (sg.n >= N) {  // everything significant: the plane is copied verbatim
    em.emit64(lo, hi, N);
    return;
  }
  // remaining positions xs = x >> n (n < 64)
  const int n = sg.n, s = n & 31;
  const uint32_t fl = funnel_r(lo, hi, s), sh = hi >> s;
  uint32_t xl = n < 32 ? fl : sh;
  uint32_t xh = n < 32 ? sh : 0u;
  const bool any = (xl | xh) != 0u;
  em.emit64((lo & sg.mlo) | (any ? sg.glo : 0u), (hi & sg.mhi) | (any ? sg.ghi : 0u), n + 1);
  if (!any) return;
  const int top = (int)((N == 64 ? hi >> 31 : lo >> (N - 1)) & 1u);  // last position set: its 1 is implied
  bool more;
  do {
    const uint32_t e = enc_lut[xl & 0xffu];
    xl = funnel_r(xl, xh, 8);
    xh >>= 8;
    more = (xl | xh) != 0u;
    // a byte that holds the plane's last set bit ends with the '0' terminator
    // (dropped from the pattern) or, on the last position, with nothing at all
    const int lf = (int)(e >> 24);
    const int len = more ? (int)((e >> 16) & 0x1fu) : lf - 2 * top;
    const uint32_t keep = more ? 0xffffu : low_mask32(lf - 1 - top);
    em.emit32(e & keep, len);
  } while (more);
  const int msb = hi ? 64 - clz32(hi) : 32 - clz32(lo);
  sg.set(msb);  // xs != 0, so the top set bit lies at or above n
}

// ---- encoder: whole block ---------------------------------------------------------
// f: the block's values, x fastest (index x + 4y + 16z).  Produces exactly
// ceil(maxbits/32) words through the sink (the last one masked by the caller
// when maxbits is not a multiple of 32).
template <int DIMS, class WordSink>
CSW_HD void encode_block(const float (&f)[1 << (2 * DIMS)], int maxbits, WordSink& sink, const uint32_t* enc_lut) {
  constexpr int N = 1 << (2 * DIMS);
  Emitter<WordSink> em(sink, (maxbits + 31) >> 5);
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < N; i++) m = fmaxf(m, fabsf(f[i]));
  const uint32_t e = biased_emax(m);
  if (e == 0) {  // all-zero block: nothing is coded (encode.cuh:356-357)
    em.finish();
    return;
  }
  em.emit32((2u * e + 1u) & 0x1ffu, 9);
  int v[N];
  {
    const float s = quant_scale(e);
#pragma unroll
    for (int i = 0; i < N; i++) v[i] = f2i_rz(s * f[i]);
  }
  fwd_xform<DIMS>(v);
  uint32_t u[N];
  fwd_order<DIMS>(v, u, std::make_integer_sequence<int, N>{});

  SigState sg;
  sg.set(0);
  for (int c = 3; c >= 0; c--) {  // planes 8c+7 .. 8c
    const uint32_t sel = (uint32_t)c | ((uint32_t)(4 + c) << 4);
    uint32_t lo[8], hi[8];
    planes_of_byte<0>(u, sel, lo);
    if constexpr (N == 64) {
      planes_of_byte<1>(u, sel, hi);
    } else {
#pragma unroll
      for (int k = 0; k < 8; k++) hi[k] = 0u;
    }
#pragma unroll
    for (int k = 7; k >= 0; k--) {
      if (em.total() < maxbits) encode_plane<N>(lo[k], hi[k], sg, em, enc_lut);
    }
    if (em.total() >= maxbits) break;
  }
  em.finish();
}

// ---- staged encoder (3-D blocks, whole words per block) ----------------------------
// Same stream as encode_block, produced in a way that suits a warp whose lanes
// code 32 different blocks:
//
//  * every plane's bit offset is known before its bits are made: a plane costs
//    n verbatim bits, one group-test bit and, when new coefficients turn
//    significant in it, (top - n) value bits + one group-test bit per set bit
//    (minus the implied final 1 and its terminator when the plane ends on the
//    last position).  So the verbatim parts are OR-ed into the staged words at
//    their offsets, one plane after the other, by all lanes in step;
//  * the expansions (the data-dependent part) are queued per lane and worked off
//    in one flat loop per eight planes, each lane running through its own queue,
//    so lanes do not wait for each other plane by plane.
//
// On sm_100 shifts, logic and compares issue on the integer ALU pipe at half
// the warp rate while integer multiply-adds go down the (otherwise idle)
// multiply-add pipe at the same rate.  Additions and left shifts are therefore
// written as multiply-adds with multipliers the compiler cannot see (they come
// in as kernel arguments), which moves about half of the lifting and transpose
// work off the ALU pipe.
struct PipeConsts {
  int one, mone;         // 1, -1
  uint32_t p1, p2, p4;   // 1 << 1, 1 << 2, 1 << 4
  uint32_t nb;           // 0xaaaaaaaa, the negabinary mask
};
CSW_HD PipeConsts pipe_consts() { return PipeConsts{1, -1, 2u, 4u, 16u, 0xaaaaaaaau}; }

CSW_HD int imad(int a, int b, int c) {
#if defined(__CUDA_ARCH__)
  int d;
  asm("mad.lo.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
#else
  return (int)((uint32_t)a * (uint32_t)b + (uint32_t)c);
#endif
}
CSW_HD uint32_t umad(uint32_t a, uint32_t b, uint32_t c) { return (uint32_t)imad((int)a, (int)b, (int)c); }

// fwd_lift with eight of its ten additions on the multiply-add pipe
CSW_HD void fwd_lift_bal(int& x, int& y, int& z, int& w, const PipeConsts& k) {
  x = imad(x, k.one, w); x >>= 1; w = imad(x, k.mone, w);
  z = imad(z, k.one, y); z >>= 1; y = imad(z, k.mone, y);
  x = imad(x, k.one, z); x >>= 1; z = imad(x, k.mone, z);
  w = imad(w, k.one, y); w >>= 1; y = imad(w, k.mone, y);
  w = wadd(w, y >> 1); y = wsub(y, w >> 1);
}
CSW_HD void fwd_xform3_bal(int (&v)[64], const PipeConsts& k) {
#pragma unroll
  for (int i = 0; i < 16; i++) fwd_lift_bal(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3], k);
#pragma unroll
  for (int z = 0; z < 4; z++)
#pragma unroll
    for (int x = 0; x < 4; x++)
      fwd_lift_bal(v[16 * z + x], v[16 * z + x + 4], v[16 * z + x + 8], v[16 * z + x + 12], k);
#pragma unroll
  for (int i = 0; i < 16; i++) fwd_lift_bal(v[i], v[i + 16], v[i + 32], v[i + 48], k);
}

template <int S, uint32_t M>
CSW_HD void tswap_bal(uint32_t& a, uint32_t& b, uint32_t pow) {  // pow = 1 << S
  const uint32_t bs = umad(b, pow, 0u);
  const uint32_t na = (a & M) | (bs & ~M);
  const uint32_t nb = ((a >> S) & M) | (b & ~M);
  a = na;
  b = nb;
}
CSW_HD void transpose8_bal(uint32_t (&r)[8], const PipeConsts& k) {
#pragma unroll
  for (int j = 0; j < 4; j++) tswap_bal<4, 0x0f0f0f0fu>(r[j], r[j + 4], k.p4);
#pragma unroll
  for (int j = 0; j < 8; j += 4) {
    tswap_bal<2, 0x33333333u>(r[j], r[j + 2], k.p2);
    tswap_bal<2, 0x33333333u>(r[j + 1], r[j + 3], k.p2);
  }
#pragma unroll
  for (int j = 0; j < 8; j += 2) tswap_bal<1, 0x55555555u>(r[j], r[j + 1], k.p1);
}
template <int G>
CSW_HD void planes_of_byte_bal(const uint32_t (&u)[64], uint32_t sel, uint32_t (&p)[8], const PipeConsts& k) {
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const uint32_t t0 = byte_perm(u[32 * G + j], u[32 * G + 8 + j], sel);
    const uint32_t t1 = byte_perm(u[32 * G + 16 + j], u[32 * G + 24 + j], sel);
    p[j] = byte_perm(t0, t1, 0x5410);
  }
  transpose8_bal(p, k);
  // the coefficients came in as v + 0xaaaaaaaa; the xor half of the negabinary
  // map flips every odd bit, i.e. it complements the odd planes
  p[1] = ~p[1]; p[3] = ~p[3]; p[5] = ~p[5]; p[7] = ~p[7];
}

constexpr int STAGE_SPARE_ROWS = 2;  // words a write may run past the block's last word
constexpr int QUEUE_SLOTS = 8;       // expansions per lane per eight planes
constexpr int QUEUE_FIELDS = 3;

// Stage: or_word(w, v) ORs v into the block's w-th staged word (rows
// 0 .. nwords + STAGE_SPARE_ROWS - 1 exist and rows below nwords start as 0);
// q_put / q_get access the lane's expansion queue.
template <class Stage>
CSW_HD void stage_put64(Stage& st, int off, uint32_t lo, uint32_t hi) {
  const int s = off & 31, w = off >> 5;
  st.or_word(w, lo << s);
  st.or_word(w + 1, funnel_l(lo, hi, s));
  st.or_word(w + 2, funnel_l(hi, 0u, s));
}

template <int... I>
CSW_HD void fwd_order3_add(const int (&v)[64], uint32_t (&u)[64], uint32_t nb, int one,
                           std::integer_sequence<int, I...>) {
  ((u[I] = umad((uint32_t)v[PermAt<3, I>::v], (uint32_t)one, nb)), ...);
}

template <class Stage>
CSW_HD void encode_block3_staged(const float (&f)[64], int maxbits, Stage& st, const uint32_t* enc_lut,
                                 const PipeConsts& kc) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 64; i++) m = fmaxf(m, fabsf(f[i]));
  const uint32_t e = biased_emax(m);
  if (e == 0) return;  // all-zero block: the staged words stay zero
  st.or_word(0, (2u * e + 1u) & 0x1ffu);
  int v[64];
  {
    const float s = quant_scale(e);
#pragma unroll
    for (int i = 0; i < 64; i++) v[i] = f2i_rz(s * f[i]);
  }
  fwd_xform3_bal(v, kc);
  uint32_t u[64];
  fwd_order3_add(v, u, kc.nb, kc.one, std::make_integer_sequence<int, 64>{});

  SigState sg;
  sg.set(0);
  int off = 9;
  for (int c = 3; c >= 0; c--) {  // planes 8c+7 .. 8c
    const uint32_t sel = (uint32_t)c | ((uint32_t)(4 + c) << 4);
    uint32_t lo[8], hi[8];
    planes_of_byte_bal<0>(u, sel, lo, kc);
    planes_of_byte_bal<1>(u, sel, hi, kc);
    int count = 0;
#pragma unroll
    for (int k = 7; k >= 0; k--) {
      if (off < maxbits) {
        // one path for every lane: with n == 64 the masks select the whole
        // word, no position is left over and no group test is coded
        const int n = sg.n, s = n & 31;
        const uint32_t fl = funnel_r(lo[k], hi[k], s), sh = hi[k] >> s;
        const uint32_t xl = n >= 64 ? 0u : (n < 32 ? fl : sh);
        const uint32_t xh = n < 32 ? sh : 0u;
        const bool any = (xl | xh) != 0u;
        stage_put64(st, off, (lo[k] & sg.mlo) | (any ? sg.glo : 0u), (hi[k] & sg.mhi) | (any ? sg.ghi : 0u));
        off += n < 64 ? n + 1 : 64;
        if (any) {
          const int top = (int)(hi[k] >> 31);
          const int msb = hi[k] ? 64 - clz32(hi[k]) : 32 - clz32(lo[k]);
          if (off < maxbits) {
            st.q_put(count, 0, xl);
            st.q_put(count, 1, xh);
            st.q_put(count, 2, (uint32_t)off | ((uint32_t)top << 31));
            count++;
          }
          off += (msb - n) + popc32(xl) + popc32(xh) - 2 * top;
          sg.set(msb);
        }
      }
    }
    // work off this lane's expansions
    int slot = 0;
    bool have = count > 0;
    uint32_t xl = 0, xh = 0;
    int boff = 0, top = 0;
    if (have) {
      xl = st.q_get(0, 0);
      xh = st.q_get(0, 1);
      const uint32_t meta = st.q_get(0, 2);
      boff = (int)(meta & 0x7fffffffu);
      top = (int)(meta >> 31);
    }
    while (have) {
      const uint32_t en = enc_lut[xl & 0xffu];
      xl = funnel_r(xl, xh, 8);
      xh >>= 8;
      const bool more = (xl | xh) != 0u;
      const int lf = (int)(en >> 24);
      const int len = more ? (int)((en >> 16) & 0x1fu) : lf - 2 * top;
      const uint32_t keep = more ? 0xffffu : low_mask32(lf - 1 - top);
      const uint32_t pat = en & keep;
      const int s = boff & 31, w = boff >> 5;
      st.or_word(w, pat << s);
      st.or_word(w + 1, funnel_l(pat, 0u, s));
      boff += len;
      if (!more || boff >= maxbits) {
        slot++;
        have = slot < count;
        if (have) {
          xl = st.q_get(slot, 0);
          xh = st.q_get(slot, 1);
          const uint32_t meta = st.q_get(slot, 2);
          boff = (int)(meta & 0x7fffffffu);
          top = (int)(meta >> 31);
        }
      }
    }
    if (off >= maxbits) break;
  }
}

// ---- bit reader -------------------------------------------------------------------
// WordSource::get(w) returns the block's w-th 32-bit stream word (0 past the
// end of the block).
template <class WordSource>
struct Reader {
  uint64_t win;
  int avail;  // valid bits in win, >= 32 between calls
  int wi;     // next word to fetch
  WordSource& src;
  CSW_HD Reader(WordSource& s) : win(0), avail(0), wi(0), src(s) {
    win = src.get(0);
    win |= (uint64_t)src.get(1) << 32;
    avail = 64;
    wi = 2;
  }
  CSW_HD uint32_t peek() const { return (uint32_t)win; }
  CSW_HD void skip(int nb) {  // nb in 0..32
    win >>= nb;
    avail -= nb;
    if (avail < 32) {
      win |= (uint64_t)src.get(wi) << avail;
      wi++;
      avail += 32;
    }
  }
  CSW_HD uint32_t take(int nb) {  // nb in 0..32
    uint32_t r = peek() & low_mask32(nb);
    skip(nb);
    return r;
  }
};

// ---- decoder: one plane -----------------------------------------------------------
// decode.cuh:141-165 for one plane; returns the plane word.
template <int N, class WordSource>
CSW_HD uint64_t decode_plane(Reader<WordSource>& rd, int& n, int& bits, const uint32_t* dec_lut) {
  // step 1: first min(n, bits) bits verbatim
  int m = n < bits ? n : bits;
  bits -= m;
  uint64_t x;
  if (m <= 32) {
    x = rd.take(m);
  } else {
    x = rd.take(32);
    x |= (uint64_t)rd.take(m - 32) << 32;
  }
  // step 2: group tests + unary runs
  int st = 0;
  for (;;) {
    if (st == 1 && (n == N - 1 || bits == 0)) {  // run cut short: the one is implied
      x |= (uint64_t)1 << n;
      n++;
      st = 0;
    }
    if (st == 0 && (n >= N || bits == 0)) break;
    int lim = (st == 0 ? N : N - 1) - n;
    int L = lim < 8 ? lim : 8;
    L = bits < L ? bits : L;
    uint32_t e = dec_lut[dec_lut_index(L, st, rd.peek() & 0xffu)];
    int used = dec_lut_used(e);
    x |= (uint64_t)dec_lut_pattern(e) << n;
    n += dec_lut_advance(e);
    bits -= used;
    rd.skip(used);
    st = dec_lut_state(e);
    if (st == 2) break;
  }
  return x;
}

// ---- decoder: whole block ---------------------------------------------------------
template <int DIMS, class WordSource>
CSW_HD void decode_block(WordSource& src, int maxbits, float (&f)[1 << (2 * DIMS)], const uint32_t* dec_lut) {
  constexpr int N = 1 << (2 * DIMS);
  Reader<WordSource> rd(src);
  if (!(rd.peek() & 1u)) {  // zero block (decode.cuh:240-243, decode3.cuh:72-73)
#pragma unroll
    for (int i = 0; i < N; i++) f[i] = 0.0f;
    return;
  }
  const uint32_t e = (rd.peek() >> 1) & 0xffu;
  rd.skip(9);
  int bits = maxbits - 9, n = 0;
  uint32_t u[N];
#pragma unroll
  for (int i = 0; i < N; i++) u[i] = 0;
  for (int c = 3; c >= 0; c--) {
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int k = 7; k >= 0; k--) {
      uint64_t x = 0;
      if (bits > 0) x = decode_plane<N>(rd, n, bits, dec_lut);
      lo[k] = (uint32_t)x;
      hi[k] = (uint32_t)(x >> 32);
    }
    const uint32_t sel0 = (0x3210u & ~(0xfu << (4 * c))) | (4u << (4 * c));
    const uint32_t step = 1u << (4 * c);
    bytes_from_planes<0>(lo, sel0, step, u);
    if constexpr (N == 64) bytes_from_planes<1>(hi, sel0, step, u);
    if (bits <= 0) break;
  }
  int v[N];
  inv_order<DIMS>(u, v, std::make_integer_sequence<int, N>{});
  inv_xform<DIMS>(v);
  const float w = dequant_scale(e);
#pragma unroll
  for (int i = 0; i < N; i++) f[i] = w * (float)v[i];
}

// ---- decoder for the slab kernel (3-D blocks, whole words per block) ----------------
// Same result as decode_block<3>.  Instead of shifting a 64-bit window along
// the stream (integer-pipe work on every read), the parser keeps one bit
// position and fetches what it needs from the staged words with two or three
// shared-memory loads and a funnel shift; the bit budget is simply
// maxbits - pos.  WordSrc::word(w) returns the block's w-th 32-bit word and 0
// for the two rows past the end.
template <class WordSrc>
CSW_HD uint32_t peek_at(const WordSrc& src, int pos) {
  const int w = pos >> 5;
  return funnel_r(src.word(w), src.word(w + 1), pos);  // the shift uses pos mod 32
}
// low min(max(n, 0), 32) bits set, for any n
CSW_HD uint32_t low_mask_sat(int n) {
  const int k = n > 0 ? n : 0;
#if defined(__CUDA_ARCH__)
  uint32_t m;
  asm("bmsk.clamp.b32 %0, 0, %1;" : "=r"(m) : "r"(k));
  return m;
#else
  return k >= 32 ? 0xffffffffu : ((1u << k) - 1u);
#endif
}
// (h:l) rotated right by r, r in 0..31
CSW_HD void ror64_small(uint32_t& l, uint32_t& h, int r) {
  const uint32_t t = funnel_r(l, h, r);
  h = funnel_r(h, l, r);
  l = t;
}
// (h:l) rotated left by r, r in 0..63
CSW_HD void rol64(uint32_t& l, uint32_t& h, int r) {
  const uint32_t a = (r & 32) ? h : l, b = (r & 32) ? l : h;  // halves after a rotation by 32
  l = funnel_l(b, a, r);
  h = funnel_l(a, b, r);
}

template <int... I>
CSW_HD void inv_order3_sub(const uint32_t (&u)[64], int (&v)[64], uint32_t nb, int mone,
                           std::integer_sequence<int, I...>) {
  ((v[PermAt<3, I>::v] = imad((int)nb, mone, (int)u[I])), ...);  // u - 0xaaaaaaaa on the multiply-add pipe
}
// Planes 8c+7 .. 8c of one block: (hi[k]:lo[k]) <- plane 8c+k, odd planes
// complemented (the xor half of the inverse negabinary map, applied to planes
// instead of coefficients).  `skip` leading planes of the slice are known to be
// empty and have been stepped over already (warp-uniform).
template <class WordSrc>
CSW_HD void decode_slice3(const WordSrc& src, int maxbits, const uint32_t* dec_lut, int skip, int& pos, int& n,
                          uint32_t (&lo)[8], uint32_t (&hi)[8]) {
#pragma unroll
  for (int k = 7; k >= 0; k--) {
    uint32_t xl = 0u, xh = 0u;
    if (7 - k >= skip && pos < maxbits) {
      // first min(n, budget) bits verbatim (decode.cuh:143-145)
      const int left0 = maxbits - pos;
      const int m = n < left0 ? n : left0;
      const int w = pos >> 5;
      const uint32_t w0 = src.word(w), w1 = src.word(w + 1), w2 = src.word(w + 2);
      xl = funnel_r(w0, w1, pos) & low_mask_sat(m);
      xh = funnel_r(w1, w2, pos) & low_mask_sat(m - 32);
      pos += m;
      // group tests and unary runs (decode.cuh:147-164), up to eight stream
      // bits per step; none once every coefficient is significant.  The bits
      // found are gathered in (ah:al), kept rotated so that position n is bit
      // 0: a step ORs its pattern in at the bottom and rotates by the positions
      // it advanced.
      if (n < 64) {
        uint32_t al = 0u, ah = 0u;
        int st = 0;
        do {
          // stream bits this step may read: up to eight, no further than the
          // last open position (a run's final one is implied, so it stops one
          // short) and no further than the block's budget; none at all ends
          // the plane through the table's L = 0 rows
          const int left = maxbits - pos;
          const int lim = 64 - st - n;
          int L = lim < 8 ? lim : 8;
          L = left < L ? left : L;
          const uint32_t en = dec_lut[dec_lut_index(L, st, peek_at(src, pos) & 0xffu)];
          const int dn = dec_lut_advance(en);
          al |= dec_lut_pattern(en);
          ror64_small(al, ah, dn);
          n += dn;
          pos += dec_lut_used(en);
          st = dec_lut_state(en);
        } while (st != 2);
        rol64(al, ah, n);  // position 0 back to bit 0
        xl |= al;
        xh |= ah;
      }
    }
    lo[k] = (k & 1) ? ~xl : xl;
    hi[k] = (k & 1) ? ~xh : xh;
  }
}

template <class WordSrc>
CSW_HD void decode_block3_pos(const WordSrc& src, int maxbits, float (&f)[64], const uint32_t* dec_lut,
                              const PipeConsts& kc) {
  const uint32_t head = src.word(0);
  // While no coefficient is significant a plane is a single '0' bit (the group
  // test of decode.cuh:147 fails at n = 0), so the zeros that follow the header
  // are whole planes.  The count common to the warp (at most the first slice)
  // is skipped in one go; a lane's further empty planes go through the loop
  // like any other.
  int lead = 8;
  if (head & 1u) {
    const uint32_t first = funnel_r(head, src.word(1), 9);  // stream bits 9..40
    const int zeros = first ? ctz32(first) : 32;
    const int budget = maxbits - 9;
    lead = zeros < lead ? zeros : lead;
    lead = budget < lead ? budget : lead;
  }
  lead = warp_min(lead);  // every lane of the warp is here: the tile test before the call is warp-uniform
  if (!(head & 1u)) {  // zero block
#pragma unroll
    for (int i = 0; i < 64; i++) f[i] = 0.0f;
    return;
  }
  const uint32_t e = (head >> 1) & 0xffu;
  int pos = 9 + lead, n = 0;
  uint32_t u[64], lo[8], hi[8];
  // u holds coefficient ^ 0xaaaaaaaa throughout: planes never decoded are zero, i.e. 0xaa bytes.
  // The first slice is peeled so that these constants are operands of its byte permutes
  // instead of sixty-four register initialisations carried into a loop.
  decode_slice3(src, maxbits, dec_lut, lead, pos, n, lo, hi);
#pragma unroll
  for (int i = 0; i < 64; i++) u[i] = 0xaaaaaaaau;
  bytes_from_planes<0>(lo, 0x4210u, 0x1000u, u);
  bytes_from_planes<1>(hi, 0x4210u, 0x1000u, u);
  for (int c = 2; c >= 0 && pos < maxbits; c--) {
    decode_slice3(src, maxbits, dec_lut, 0, pos, n, lo, hi);
    const uint32_t sel0 = (0x3210u & ~(0xfu << (4 * c))) | (4u << (4 * c));
    const uint32_t step = 1u << (4 * c);
    bytes_from_planes<0>(lo, sel0, step, u);
    bytes_from_planes<1>(hi, sel0, step, u);
  }
  int v[64];
  inv_order3_sub(u, v, kc.nb, kc.mone, std::make_integer_sequence<int, 64>{});
  inv_xform<3>(v);
  const float w = dequant_scale(e);
#pragma unroll
  for (int i = 0; i < 64; i++) f[i] = w * (float)v[i];
}

}  // namespace csw
