// Diagnostic, not part of the library: issue throughput of the instruction
// kinds the ZFP kernels are made of, alone and mixed, on the GPU it runs on.
//
// Every SM runs 8 CTAs x 256 threads; a thread keeps 8 independent dependency
// chains and executes 64 operations per loop iteration (so loop overhead is
// under 5 %).  Time is taken per SM from the cycle counter (first start to last
// end of the SM's CTAs), so the figures are thread-operations per clock per SM
// whatever the clock frequency is.  Build: python -m cswap_b200.build --probe
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <vector>

#define ITER 1024
#define L(i) "lop3.b32 %" #i ",%" #i ",%8,%9,0x6a;\n"
#define M(i) "mad.lo.u32 %" #i ",%" #i ",%10,%9;\n"
#define F(i) "fma.rn.f32 %" #i ",%" #i ",%11,%12;\n"
#define S(i) "shf.l.wrap.b32 %" #i ",%" #i ",%9,%8;\n"
#define P(i) "prmt.b32 %" #i ",%" #i ",%9,%8;\n"
#define C(i) "cvt.rzi.s32.f32 %" #i ",%" #i ";\n"
#define B(i) "popc.b32 %" #i ",%" #i ";\n"
#define Z(i) "clz.b32 %" #i ",%" #i ";\n"
#define BODY(s)                                                                                              \
  asm volatile(s s s s s s s s                                                                               \
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]) \
               : "r"(a), "r"(b), "r"(one), "f"(fa), "f"(fb));

template <int OP>
__global__ void __launch_bounds__(256) probe(uint32_t* out, long long* clk, uint32_t a, uint32_t b, uint32_t one,
                                             float fa, float fb) {
  uint32_t r[8];
  for (int i = 0; i < 8; i++) r[i] = threadIdx.x * 8 + i + a;
  __syncthreads();
  const long long t0 = clock64();
#pragma unroll 1
  for (int it = 0; it < ITER; it++) {
    if (OP == 0) BODY(L(0) L(1) L(2) L(3) L(4) L(5) L(6) L(7))
    if (OP == 1) BODY(M(0) M(1) M(2) M(3) M(4) M(5) M(6) M(7))
    if (OP == 2) BODY(F(0) F(1) F(2) F(3) F(4) F(5) F(6) F(7))
    if (OP == 3) BODY(S(0) S(1) S(2) S(3) S(4) S(5) S(6) S(7))
    if (OP == 4) BODY(P(0) P(1) P(2) P(3) P(4) P(5) P(6) P(7))
    if (OP == 5) BODY(C(0) C(1) C(2) C(3) C(4) C(5) C(6) C(7))
    if (OP == 6) BODY(B(0) B(1) B(2) B(3) B(4) B(5) B(6) B(7))
    if (OP == 7) BODY(Z(0) Z(1) Z(2) Z(3) Z(4) Z(5) Z(6) Z(7))
    if (OP == 8) BODY(L(0) S(1) L(2) S(3) L(4) S(5) L(6) S(7))
    if (OP == 9) BODY(L(0) M(1) L(2) M(3) L(4) M(5) L(6) M(7))
    if (OP == 10) BODY(L(0) F(1) L(2) F(3) L(4) F(5) L(6) F(7))
    if (OP == 11) BODY(M(0) F(1) M(2) F(3) M(4) F(5) M(6) F(7))
    if (OP == 12) BODY(L(0) L(1) L(2) M(3) L(4) L(5) L(6) M(7))
    if (OP == 13) BODY(L(0) S(1) M(2) F(3) L(4) S(5) M(6) F(7))
    if (OP == 14) BODY(L(0) C(1) L(2) L(3) L(4) C(5) L(6) L(7))
  }
  const long long t1 = clock64();
  uint32_t s = 0;
  for (int i = 0; i < 8; i++) s ^= r[i];
  out[blockIdx.x * 256 + threadIdx.x] = s;
  if (threadIdx.x == 0) {
    uint32_t sm;
    asm("mov.u32 %0,%%smid;" : "=r"(sm));
    clk[blockIdx.x * 3] = t0;
    clk[blockIdx.x * 3 + 1] = t1;
    clk[blockIdx.x * 3 + 2] = sm;
  }
}

template <int OP>
static void run(const char* name, int sms, uint32_t* d, long long* dc) {
  const int nblk = sms * 8;
  for (int rep = 0; rep < 2; rep++) {  // the second launch is the measured one
    probe<OP><<<nblk, 256>>>(d, dc, 3, 5, 1, 1.0001f, 0.5f);
    cudaDeviceSynchronize();
  }
  std::vector<long long> h(nblk * 3);
  cudaMemcpy(h.data(), dc, nblk * 3 * sizeof(long long), cudaMemcpyDeviceToHost);
  std::vector<long long> lo(1024, 1LL << 62), hi(1024, 0);
  std::vector<int> cnt(1024, 0);
  for (int b = 0; b < nblk; b++) {
    const int sm = (int)h[b * 3 + 2] & 1023;
    lo[sm] = std::min(lo[sm], h[b * 3]);
    hi[sm] = std::max(hi[sm], h[b * 3 + 1]);
    cnt[sm]++;
  }
  std::vector<double> thr;
  for (int s = 0; s < 1024; s++)
    if (cnt[s]) thr.push_back((double)cnt[s] * 256 * ITER * 64 / (double)(hi[s] - lo[s]));
  std::sort(thr.begin(), thr.end());
  printf("%-30s %6.1f thread-ops/clk/SM (median of %zu SMs; min %.1f max %.1f)  %s\n", name, thr[thr.size() / 2],
         thr.size(), thr.front(), thr.back(), cudaGetErrorString(cudaGetLastError()));
}

int main() {
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  uint32_t* d;
  long long* dc;
  cudaMalloc(&d, (size_t)sms * 8 * 256 * 4);
  cudaMalloc(&dc, (size_t)sms * 8 * 3 * sizeof(long long));
  run<0>("lop3", sms, d, dc);
  run<1>("mad.lo (opaque multiplier)", sms, d, dc);
  run<2>("fma.rn.f32", sms, d, dc);
  run<3>("shf.l.wrap", sms, d, dc);
  run<4>("prmt", sms, d, dc);
  run<5>("cvt.rzi.s32.f32", sms, d, dc);
  run<6>("popc", sms, d, dc);
  run<7>("clz", sms, d, dc);
  run<8>("lop3 + shf 1:1", sms, d, dc);
  run<9>("lop3 + mad.lo 1:1", sms, d, dc);
  run<10>("lop3 + fma 1:1", sms, d, dc);
  run<11>("mad.lo + fma 1:1", sms, d, dc);
  run<12>("lop3 + mad.lo 3:1", sms, d, dc);
  run<13>("lop3 shf mad.lo fma 1:1:1:1", sms, d, dc);
  run<14>("lop3 + cvt 3:1", sms, d, dc);
  return 0;
}
