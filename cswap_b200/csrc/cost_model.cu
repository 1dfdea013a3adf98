// Self-tuning cost model: measures codec and host-link throughput on the
// device at hand and decides, per tensor, whether compressing beats a raw copy.
//
// Stands in for the reference's PolicyMaker (c10::GetPolicyMaker(), whose
// source is not part of the reference tree; its inputs are the per-layer
// compute times, tensor sizes and producer/consumer steps recorded at
// CSWAP+/Execution.h:224-233 and its output the per-tensor policy vector used
// at CSWAP+/resnet-cifar10.cpp:407-437).
#include <cuda_runtime.h>

#include <time.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "../../include/cswap_b200.h"
#include "internal.h"

namespace csw {
namespace {

// deterministic pseudo-random activations: `zeros256` / 256 of them zero, the rest in (-1,1)
__global__ void fill_kernel(float* p, size_t n, uint32_t zeros256) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    uint32_t h = (uint32_t)i * 2654435761u;
    h ^= h >> 15;
    h *= 2246822519u;
    h ^= h >> 13;
    p[i] = (h & 0xffu) < zeros256 ? 0.0f : ((float)(h >> 8) * (1.0f / 8388608.0f) - 1.0f);
  }
}

// per-byte slope of the sparse codec at a zero fraction: piecewise linear through the fits at 50, 75 and 90 %
double sparse_slope(double b50, double b75, double b90, double zf) {
  if (b75 <= 0 || b90 <= 0 || zf <= 0.5) return b50;
  if (zf <= 0.75) return b50 + (b75 - b50) * (zf - 0.5) / 0.25;
  if (zf <= 0.9) return b75 + (b90 - b75) * (zf - 0.75) / 0.15;
  return b90;
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
  // the compressed-side buffer holds the larger of the sparse bound and the ZFP stream at this rate
  size_t c_bytes = L.bound, z_bytes = 0;
  csw_zfp_max_bytes(32, 32, nmax / 1024, mb, &z_bytes);
  if (z_bytes > c_bytes) c_bytes = z_bytes;
  cudaError_t e = cudaMalloc(&d_x, nmax * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d_y, nmax * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d_c, c_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&d_nnz, 4);
  if (e == cudaSuccess) e = cudaHostAlloc(&h, nmax * 4, cudaHostAllocDefault);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreate(&e0);
  if (e == cudaSuccess) e = cudaEventCreate(&e1);
  if (e == cudaSuccess) {
    fill_kernel<<<1024, 256, 0, s>>>(d_x, nmax, 128);
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
    st = time_op(s, e0, e1, 5, [&] { return csw_zfp_compress(d_x, 32, 32, nz, mb, d_c, c_bytes, nullptr, s); }, &t);
    t_ze.push_back(t);
    if (st == CSW_OK)
      st = time_op(s, e0, e1, 5, [&] { return csw_zfp_decompress(d_c, zb, 32, 32, nz, mb, d_y, s); }, &t);
    t_zd.push_back(t);
    if (st == CSW_OK)
      st = time_op(s, e0, e1, 5, [&] { return csw_sparse_compress_onepass(d_x, n, d_c, L.bound, d_nnz, s); }, &t);
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
  // the sparse codec again at 75 % and 90 % zeros (two largest sizes: the slope is what changes)
  double slopes[2][2] = {{0, 0}, {0, 0}};
  const uint32_t zeros256[2] = {192, 230};
  for (int z = 0; z < 2 && st == CSW_OK; z++) {
    fill_kernel<<<1024, 256, 0, s>>>(d_x, nmax, zeros256[z]);
    double te[2] = {0, 0}, td[2] = {0, 0};
    for (int i = 2; i < 4 && st == CSW_OK; i++) {
      const size_t n = sizes[i];
      st = time_op(s, e0, e1, 5, [&] { return csw_sparse_compress_onepass(d_x, n, d_c, L.bound, d_nnz, s); }, &te[i - 2]);
      if (st == CSW_OK) st = time_op(s, e0, e1, 5, [&] { return csw_sparse_decompress(d_c, n, d_y, s); }, &td[i - 2]);
    }
    const double db = (double)(sizes[3] - sizes[2]) * 4;
    slopes[z][0] = (te[1] - te[0]) / db;
    slopes[z][1] = (td[1] - td[0]) / db;
  }
  // what a swapped tensor costs the calling thread: swap-out + release of a 1 MiB tensor, raw
  double host_swap = 0;
  if (st == CSW_OK) {
    const int reps = 16;
    csw_ticket* tk[reps];
    cudaStreamSynchronize(s);
    timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    int made = 0;
    for (; made < reps; made++)
      if (csw_swap_out(m, d_x, (size_t)1 << 18, CSW_POLICY_RAW, s, &tk[made]) != CSW_OK) break;
    for (int i = 0; i < made; i++) csw_ticket_release(m, tk[i]);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    if (made) host_swap = ((t1.tv_sec - t0.tv_sec) + (t1.tv_nsec - t0.tv_nsec) * 1e-9) / made;
    csw_mgr_sync(m);
  }
  if (st == CSW_OK) {
    Fit f;
    model->sparse_enc_b75 = slopes[0][0] > 0 ? slopes[0][0] : 0;
    model->sparse_dec_b75 = slopes[0][1] > 0 ? slopes[0][1] : 0;
    model->sparse_enc_b90 = slopes[1][0] > 0 ? slopes[1][0] : 0;
    model->sparse_dec_b90 = slopes[1][1] > 0 ? slopes[1][1] : 0;
    model->host_swap_s = host_swap;
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

namespace {

struct Cand {
  int policy;
  double enc, dec, moved;
  bool ok;
};

// One step under a given choice per tensor.  Swap-outs queue on the D2H link
// in forward order, each no earlier than its tensor is ready plus its encode
// time; forward compute never waits for them.  Backward needs the tensors in
// reverse order; the H2D copy of a tensor starts when the tensor swapped out
// after it was asked for (one step of prefetch), not before its own D2H has
// finished and not before the link is free; if copy + decode end after the
// tensor is needed, backward stalls and everything later shifts.  Returns the
// total stall and writes the per-tensor stalls.
// With `take_back`, a losslessly swapped tensor whose copy out has not finished
// when backward asks for it is handed back as it is (what the Execution classes
// do): no copy in and no stall for it - and no memory freed, which is why the
// decision itself does not count on it.
double simulate(const csw_cost_model* cm, const csw_tensor_desc* td, size_t n, const std::vector<Cand>& c,
                double fwd_total, double* stalls, bool take_back = false) {
  std::vector<double> on_host(n);
  double link = 0;
  for (size_t i = 0; i < n; i++) {
    if (c[i].policy == CSW_POLICY_KEEP) { on_host[i] = 0; continue; }
    const double start = std::max(td[i].ready_s + c[i].enc, link);
    link = start + cm->d2h_a + c[i].moved / cm->d2h_bps;
    on_host[i] = link;
  }
  double stall = 0, h2d = fwd_total, asked = fwd_total;
  for (size_t j = n; j-- > 0;) {
    if (stalls) stalls[j] = 0;
    if (c[j].policy == CSW_POLICY_KEEP) continue;
    const double need = fwd_total + td[j].need_s + stall;
    if (take_back && (c[j].policy == CSW_POLICY_RAW || c[j].policy == CSW_POLICY_SPARSE) && on_host[j] > need) {
      asked = std::max(asked, need);
      continue;
    }
    const double start = std::max(std::max(h2d, on_host[j]), asked);
    h2d = start + cm->h2d_a + c[j].moved / cm->h2d_bps;
    const double arrive = h2d + c[j].dec;
    if (arrive > need) {
      stall += arrive - need;
      if (stalls) stalls[j] = arrive - need;
    }
    asked = std::max(need, arrive);
  }
  return stall;
}

}  // namespace

// Starts from raw swap everywhere and switches tensors, largest first, to the
// sparse codec (lossless, needs a measured zero fraction) or to ZFP (only where
// loss is allowed) whenever the simulated stall of the whole step drops -
// by anything for the lossless codec; ZFP must beat the best lossless choice by
// 2 % of the tensor's raw link time (and 5 us).
// Ties go to the smaller payload (a last pass codes whatever may be coded unless
// the simulated stall gets worse), so when the links keep up with compute the
// table is "ZFP where loss is allowed, sparse where zeros were measured".
csw_status csw_cost_decide(const csw_cost_model* cm, const csw_tensor_desc* td, size_t n, double fwd_total_s,
                           int* policy, double* exposed) {
  if (!cm || (!td && n) || (!policy && n)) return CSW_ERR_ARG;
  if (cm->d2h_bps <= 0 || cm->h2d_bps <= 0) return CSW_ERR_ARG;
  const double rate = cm->zfp_maxbits ? cm->zfp_maxbits / 64.0 : 8.0;  // bits per value
  std::vector<Cand> raw(n), sparse(n), zfp(n), cur(n);
  std::vector<size_t> order(n);
  for (size_t i = 0; i < n; i++) {
    const double b = (double)td[i].numel * 4.0, zf = td[i].zero_fraction;
    raw[i] = {CSW_POLICY_RAW, 0, 0, b, true};
    sparse[i] = {CSW_POLICY_SPARSE,
                 cm->sparse_enc_a + sparse_slope(cm->sparse_enc_b, cm->sparse_enc_b75, cm->sparse_enc_b90, zf) * b,
                 cm->sparse_dec_a + sparse_slope(cm->sparse_dec_b, cm->sparse_dec_b75, cm->sparse_dec_b90, zf) * b,
                 b * (1.0 - (zf < 0 ? 0 : zf)) + b / 32.0 + (double)td[i].numel / 1024.0, zf >= 0};
    zfp[i] = {CSW_POLICY_ZFP, cm->zfp_enc_a + cm->zfp_enc_b * b, cm->zfp_dec_a + cm->zfp_dec_b * b, b * rate / 32.0,
              td[i].lossy_ok && td[i].numel >= 1024};
    cur[i] = raw[i];
    order[i] = i;
  }
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b2) { return td[a].numel > td[b2].numel; });
  double best = simulate(cm, td, n, cur, fwd_total_s, nullptr);
  for (int pass = 0; pass < 3 && best > 0; pass++) {
    bool changed = false;
    for (size_t oi = 0; oi < n && best > 0; oi++) {
      const size_t i = order[oi];
      const Cand keep = cur[i];
      Cand pick = keep;
      double pick_stall = best;
      if (sparse[i].ok && keep.policy != CSW_POLICY_SPARSE) {
        cur[i] = sparse[i];
        const double st = simulate(cm, td, n, cur, fwd_total_s, nullptr);
        if (st < pick_stall - 1e-7) { pick = sparse[i]; pick_stall = st; }
      }
      if (zfp[i].ok && keep.policy != CSW_POLICY_ZFP) {
        cur[i] = zfp[i];
        const double st = simulate(cm, td, n, cur, fwd_total_s, nullptr);
        // lossy has to buy a real gain: at least 2 % of the tensor's own raw link time (and 5 us)
        const double margin = std::max(5e-6, 0.02 * raw[i].moved / cm->d2h_bps);
        if (st < pick_stall - margin) { pick = zfp[i]; pick_stall = st; }
      }
      cur[i] = pick;
      if (pick.policy != keep.policy) { changed = true; best = pick_stall; }
    }
    if (!changed) break;
  }
  // Ties go to the smaller payload: a tensor left raw because nothing was gained by coding
  // it still occupies the link and the copy engine's queue, which serves copies strictly in
  // the order they were submitted - costs this simulation does not see (measured: two raw
  // 48 MiB tensors among 119 ZFP ones added a quarter to a BERT-shaped step).  So whatever
  // may be coded is coded unless that makes the simulated stall worse.
  for (size_t oi = 0; oi < n; oi++) {
    const size_t i = order[oi];
    if (cur[i].policy != CSW_POLICY_RAW) continue;
    const Cand keep = cur[i];
    const bool sparse_first = sparse[i].ok && (!zfp[i].ok || sparse[i].moved <= zfp[i].moved);
    for (const Cand* alt : {sparse_first ? &sparse[i] : &zfp[i], sparse_first ? &zfp[i] : &sparse[i]}) {
      if (!alt->ok || alt->moved >= keep.moved) continue;
      cur[i] = *alt;
      const double st = simulate(cm, td, n, cur, fwd_total_s, nullptr);
      if (st <= best + 1e-7) {
        best = st < best ? st : best;
        break;
      }
      cur[i] = keep;
    }
  }
  std::vector<double> stalls(n);
  simulate(cm, td, n, cur, fwd_total_s, stalls.data());
  for (size_t i = 0; i < n; i++) {
    policy[i] = cur[i].policy;
    if (exposed) exposed[i] = stalls[i];
  }
  return CSW_OK;
}

csw_status csw_cost_simulate(const csw_cost_model* cm, const csw_tensor_desc* td, size_t n, double fwd_total_s,
                             const int* policy, double* exposed, double* total_stall_s) {
  if (!cm || (!td && n) || (!policy && n) || !total_stall_s) return CSW_ERR_ARG;
  if (cm->d2h_bps <= 0 || cm->h2d_bps <= 0) return CSW_ERR_ARG;
  const double rate = cm->zfp_maxbits ? cm->zfp_maxbits / 64.0 : 8.0;
  std::vector<Cand> cur(n);
  for (size_t i = 0; i < n; i++) {
    const double b = (double)td[i].numel * 4.0, zf = td[i].zero_fraction;
    int p = policy[i];
    if (p == CSW_POLICY_ZFP && td[i].numel < 1024) p = CSW_POLICY_RAW;
    if (p == CSW_POLICY_SPARSE && zf < 0) p = CSW_POLICY_RAW;
    if (p == CSW_POLICY_ZFP)
      cur[i] = {p, cm->zfp_enc_a + cm->zfp_enc_b * b, cm->zfp_dec_a + cm->zfp_dec_b * b, b * rate / 32.0, true};
    else if (p == CSW_POLICY_SPARSE)
      cur[i] = {p, cm->sparse_enc_a + sparse_slope(cm->sparse_enc_b, cm->sparse_enc_b75, cm->sparse_enc_b90, zf) * b,
                cm->sparse_dec_a + sparse_slope(cm->sparse_dec_b, cm->sparse_dec_b75, cm->sparse_dec_b90, zf) * b,
                b * (1.0 - zf) + b / 32.0 + (double)td[i].numel / 1024.0, true};
    else if (p == CSW_POLICY_RAW)
      cur[i] = {p, 0, 0, b, true};
    else
      cur[i] = {CSW_POLICY_KEEP, 0, 0, 0, true};
  }
  std::vector<double> stalls(n ? n : 1);
  *total_stall_s = simulate(cm, td, n, cur, fwd_total_s, stalls.data(), /*take_back=*/true);
  if (exposed)
    for (size_t i = 0; i < n; i++) exposed[i] = stalls[i];
  return CSW_OK;
}

}  // extern "C"
