// Self-tuning cost model: measures codec and host-link throughput on the
// device at hand and decides, per tensor, whether compressing beats a raw copy.
//
// Stands in for the reference's PolicyMaker (c10::GetPolicyMaker(), whose
// source is not part of the reference tree; its inputs are the per-layer
// compute times, tensor sizes and producer/consumer steps recorded at
// CSWAP+/Execution.h:224-233 and its output the per-tensor policy vector used
// at CSWAP+/resnet-cifar10.cpp:407-437).
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "../../include/cswap_b200.h"
#include "internal.h"

namespace csw {
namespace {

// deterministic pseudo-random activations: about half zeros, the rest in (-1,1)
__global__ void fill_kernel(float* p, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    uint32_t h = (uint32_t)i * 2654435761u;
    h ^= h >> 15;
    h *= 2246822519u;
    h ^= h >> 13;
    p[i] = (h & 1u) ? 0.0f : ((float)(h >> 8) * (1.0f / 8388608.0f) - 1.0f);
  }
}

struct Fit {
  double a, b;
};
// least squares t = a + b x, a clamped at >= 0
Fit fit_line(const std::vector<double>& x, const std::vector<double>& t) {
  const size_t n = x.size();
  double sx = 0, st = 0, sxx = 0, sxt = 0;
  for (size_t i = 0; i < n; i++) { sx += x[i]; st += t[i]; sxx += x[i] * x[i]; sxt += x[i] * t[i]; }
  const double den = n * sxx - sx * sx;
  Fit f{0, 0};
  if (den > 0) {
    f.b = (n * sxt - sx * st) / den;
    f.a = (st - f.b * sx) / n;
  }
  if (f.a < 0 || f.b <= 0) {  // degenerate: through the origin
    f.a = 0;
    f.b = sxx > 0 ? sxt / sxx : 0;
  }
  return f;
}

template <class F>
csw_status time_op(cudaStream_t s, cudaEvent_t e0, cudaEvent_t e1, int reps, F op, double* seconds) {
  csw_status st = op();  // warm-up
  if (st != CSW_OK) return st;
  float best = 1e30f;
  for (int r = 0; r < reps; r++) {
    cudaEventRecord(e0, s);
    st = op();
    if (st != CSW_OK) return st;
    cudaEventRecord(e1, s);
    cudaError_t e = cudaEventSynchronize(e1);
    if (e != cudaSuccess) return cuda_fail(e);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    best = std::min(best, ms);
  }
  *seconds = best * 1e-3;
  return CSW_OK;
}

}  // namespace
}  // namespace csw

using namespace csw;

extern "C" {

csw_status csw_cost_fit(csw_mgr* m, csw_cost_model* model) {
  if (!m || !model) return CSW_ERR_ARG;
  csw_mgr_stats stats;
  csw_status st = csw_mgr_get_stats(m, &stats);  // also validates the handle
  if (st != CSW_OK) return st;
  // sizes of the probe tensors (floats): 1, 4, 16, 64 MiB
  const size_t sizes[4] = {(size_t)1 << 18, (size_t)1 << 20, (size_t)1 << 22, (size_t)1 << 24};
  const size_t nmax = sizes[3];
  // rate to fit at: the caller's (zero-initialised struct means 512 = rate 8)
  const unsigned mb = model->zfp_maxbits ? model->zfp_maxbits : 512;
  {
    size_t probe = 0;
    if (csw_zfp_max_bytes(32, 32, 4, mb, &probe) != CSW_OK || (mb & 31)) return CSW_ERR_ARG;
  }
  float *d_x = nullptr, *d_y = nullptr;
  void* d_c = nullptr;
  void* h = nullptr;
  uint32_t* d_nnz = nullptr;
  cudaStream_t s = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  csw_sparse_layout L;
  csw_sparse_layout_of(nmax, &L);
  cudaError_t e = cudaMalloc(&d_x, nmax * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d_y, nmax * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d_c, L.bound);
  if (e == cudaSuccess) e = cudaMalloc(&d_nnz, 4);
  if (e == cudaSuccess) e = cudaHostAlloc(&h, nmax * 4, cudaHostAllocDefault);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreate(&e0);
  if (e == cudaSuccess) e = cudaEventCreate(&e1);
  if (e == cudaSuccess) {
    fill_kernel<<<1024, 256, 0, s>>>(d_x, nmax);
    e = cudaGetLastError();
  }
  st = e == cudaSuccess ? CSW_OK : cuda_fail(e);

  std::vector<double> xb, t_ze, t_zd, t_se, t_sd, t_d2h, t_h2d;
  for (int i = 0; i < 4 && st == CSW_OK; i++) {
    const size_t n = sizes[i], nz = n / 1024;
    size_t zb = 0;
    csw_zfp_max_bytes(32, 32, nz, mb, &zb);
    double t = 0;
    xb.push_back((double)n * 4);
    st = time_op(s, e0, e1, 5, [&] { return csw_zfp_compress(d_x, 32, 32, nz, mb, d_c, L.bound, nullptr, s); }, &t);
    t_ze.push_back(t);
    if (st == CSW_OK)
      st = time_op(s, e0, e1, 5, [&] { return csw_zfp_decompress(d_c, zb, 32, 32, nz, mb, d_y, s); }, &t);
    t_zd.push_back(t);
    if (st == CSW_OK)
      st = time_op(s, e0, e1, 5, [&] { return csw_sparse_compress(d_x, n, d_c, L.bound, d_nnz, s); }, &t);
    t_se.push_back(t);
    if (st == CSW_OK) st = time_op(s, e0, e1, 5, [&] { return csw_sparse_decompress(d_c, n, d_y, s); }, &t);
    t_sd.push_back(t);
    if (st == CSW_OK)
      st = time_op(s, e0, e1, 3, [&] {
        cudaError_t ce = cudaMemcpyAsync(h, d_x, n * 4, cudaMemcpyDeviceToHost, s);
        return ce == cudaSuccess ? CSW_OK : cuda_fail(ce);
      }, &t);
    t_d2h.push_back(t);
    if (st == CSW_OK)
      st = time_op(s, e0, e1, 3, [&] {
        cudaError_t ce = cudaMemcpyAsync(d_y, h, n * 4, cudaMemcpyHostToDevice, s);
        return ce == cudaSuccess ? CSW_OK : cuda_fail(ce);
      }, &t);
    t_h2d.push_back(t);
  }
  if (st == CSW_OK) {
    Fit f;
    f = fit_line(xb, t_ze); model->zfp_enc_a = f.a; model->zfp_enc_b = f.b;
    f = fit_line(xb, t_zd); model->zfp_dec_a = f.a; model->zfp_dec_b = f.b;
    f = fit_line(xb, t_se); model->sparse_enc_a = f.a; model->sparse_enc_b = f.b;
    f = fit_line(xb, t_sd); model->sparse_dec_a = f.a; model->sparse_dec_b = f.b;
    f = fit_line(xb, t_d2h); model->d2h_a = f.a; model->d2h_bps = f.b > 0 ? 1.0 / f.b : 0;
    f = fit_line(xb, t_h2d); model->h2d_a = f.a; model->h2d_bps = f.b > 0 ? 1.0 / f.b : 0;
    model->zfp_maxbits = mb;
  }
  if (s) cudaStreamSynchronize(s);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (s) cudaStreamDestroy(s);
  if (h) cudaFreeHost(h);
  if (d_nnz) cudaFree(d_nnz);
  if (d_c) cudaFree(d_c);
  if (d_y) cudaFree(d_y);
  if (d_x) cudaFree(d_x);
  return st;
}

// Forward and backward are each simulated as one serial link shared by the
// tensors in order.  A swap-out may start when its tensor's consumer has run
// (time 0 of its window) and is "exposed" by however long it outlasts the
// window overlap_fwd; a swap-in may start overlap_bwd before it is needed.
// Link occupancy carries over from tensor to tensor, so compressing an early
// tensor helps the later ones.  Lossless choices win ties; ZFP is chosen only
// when it lowers the exposed time by more than 2 %.
csw_status csw_cost_decide(const csw_cost_model* cm, const csw_tensor_desc* td, size_t n, int* policy,
                           double* exposed) {
  if (!cm || (!td && n) || (!policy && n)) return CSW_ERR_ARG;
  if (cm->d2h_bps <= 0 || cm->h2d_bps <= 0) return CSW_ERR_ARG;
  const double rate = cm->zfp_maxbits ? cm->zfp_maxbits / 64.0 : 8.0;  // bits per value
  double out_busy = 0, in_busy = 0;  // backlog (seconds) the links carry into the next tensor
  for (size_t i = 0; i < n; i++) {
    const double raw = (double)td[i].numel * 4.0;
    struct Cand { int policy; double enc, dec, moved; bool ok; } c[3];
    c[0] = {CSW_POLICY_RAW, 0, 0, raw, true};
    const double zf = td[i].zero_fraction;
    c[1] = {CSW_POLICY_SPARSE, cm->sparse_enc_a + cm->sparse_enc_b * raw, cm->sparse_dec_a + cm->sparse_dec_b * raw,
            raw * (1.0 - (zf < 0 ? 0 : zf)) + raw / 32.0 + (double)td[i].numel / 1024.0, zf >= 0};
    c[2] = {CSW_POLICY_ZFP, cm->zfp_enc_a + cm->zfp_enc_b * raw, cm->zfp_dec_a + cm->zfp_dec_b * raw,
            raw * rate / 32.0, td[i].lossy_ok && td[i].numel % 1024 == 0 && td[i].numel > 0};
    int best = 0;
    double best_cost = 0, best_out = 0, best_in = 0;
    for (int k = 0; k < 3; k++) {
      if (!c[k].ok) continue;
      const double t_out = out_busy + c[k].enc + cm->d2h_a + c[k].moved / cm->d2h_bps;
      const double t_in = in_busy + cm->h2d_a + c[k].moved / cm->h2d_bps + c[k].dec;
      const double ex = std::max(0.0, t_out - td[i].overlap_fwd_s) + std::max(0.0, t_in - td[i].overlap_bwd_s);
      const double need = k == 2 ? 0.98 : 1.0;  // lossy must clearly pay
      if (k == 0 || ex < best_cost * need - 1e-12) {
        best = k;
        best_cost = ex;
        best_out = std::max(0.0, t_out - td[i].overlap_fwd_s);
        best_in = std::max(0.0, t_in - td[i].overlap_bwd_s);
      }
    }
    policy[i] = c[best].policy;
    if (exposed) exposed[i] = best_cost;
    // whatever did not fit in this tensor's window delays the next one
    out_busy = best_out;
    in_busy = best_in;
  }
  return CSW_OK;
}

}  // extern "C"
