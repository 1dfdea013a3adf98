// BERT-style encoder training step under cswap::Execution, every linear /
// matmul / softmax / dropout / layer-norm / activation wrapped in exe.pre /
// exe.post the way the reference's driver wraps them (CSWAP+/bert.cpp:370-801:
// one pre/post pair around each op, the vector overloads for ops with two
// inputs).  Dimensions are arguments; the benchmark uses the BERT-base shape
// (12 layers, hidden 768, 12 heads, FFN 3072, seq 512, batch 32).
//
//   bert_step --check [--layers 2]   raw and sparse swap of every activation leave
//                                    loss and gradients bit-identical to the step
//                                    without swapping (same dropout seed); ZFP rate 16
//                                    leaves the loss identical and the gradients close.
//   bert_step --bench [--steps K] [--warmup W]
//                                    one JSON line: step time, link bytes, swapped
//                                    activation bytes and peak device memory for no
//                                    swap, raw swap, ZFP-16 everywhere and the
//                                    self-tuned table (loss allowed on every float
//                                    activation, as BASELINE's config 5 has it).
//
// A tensor is swapped at its LAST forward use: the layer input x feeds the three
// projections and the residual add, and its storage is empty once it has been
// swapped.  The table of last uses comes from one profiled step.
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <torch/torch.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <functional>
#include <map>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include "cswap_execution.hpp"

using cswap::Execution;
using cswap::Layer_type;
using torch::Tensor;

struct Dims {
  int vocab = 30522, hidden = 768, layers = 12, heads = 12, ffn = 3072, seq = 512, batch = 32;
  double dropout = 0.1;
};

struct Bert : torch::nn::Module {
  Dims d;
  torch::nn::Embedding tok{nullptr}, pos{nullptr};
  torch::nn::LayerNorm emb_ln{nullptr};
  std::vector<torch::nn::Linear> q, k, v, o, f1, f2;
  std::vector<torch::nn::LayerNorm> ln1, ln2;
  torch::nn::Linear head{nullptr};

  explicit Bert(const Dims& dims) : d(dims) {
    tok = register_module("tok", torch::nn::Embedding(d.vocab, d.hidden));
    pos = register_module("pos", torch::nn::Embedding(d.seq, d.hidden));
    emb_ln = register_module("emb_ln", torch::nn::LayerNorm(torch::nn::LayerNormOptions({d.hidden})));
    for (int l = 0; l < d.layers; l++) {
      const std::string s = std::to_string(l);
      q.push_back(register_module("q" + s, torch::nn::Linear(d.hidden, d.hidden)));
      k.push_back(register_module("k" + s, torch::nn::Linear(d.hidden, d.hidden)));
      v.push_back(register_module("v" + s, torch::nn::Linear(d.hidden, d.hidden)));
      o.push_back(register_module("o" + s, torch::nn::Linear(d.hidden, d.hidden)));
      ln1.push_back(register_module("ln1_" + s, torch::nn::LayerNorm(torch::nn::LayerNormOptions({d.hidden}))));
      f1.push_back(register_module("f1_" + s, torch::nn::Linear(d.hidden, d.ffn)));
      f2.push_back(register_module("f2_" + s, torch::nn::Linear(d.ffn, d.hidden)));
      ln2.push_back(register_module("ln2_" + s, torch::nn::LayerNorm(torch::nn::LayerNormOptions({d.hidden}))));
    }
    head = register_module("head", torch::nn::Linear(d.hidden, 2));
  }

  Tensor forward(Execution& exe, Tensor ids, Tensor target) {
    const int64_t B = ids.size(0), S = ids.size(1), H = d.hidden, nh = d.heads, dh = H / nh;
    const double p = d.dropout;
    const bool train = is_training();
    auto one = [&](const std::function<Tensor(const Tensor&)>& f, Tensor& in, Layer_type lt = cswap::ACT,
                   bool omit = false) {
      exe.pre(in, lt);
      Tensor out = f(in);
      exe.post(in, out, lt, omit);
      return out;
    };
    auto two = [&](const std::function<Tensor(const Tensor&, const Tensor&)>& f, Tensor& a, Tensor& b,
                   Layer_type lt = cswap::ACT, bool omit = false) {
      exe.pre({a, b}, lt);
      Tensor out = f(a, b);
      exe.post({a, b}, out, lt, omit);
      return out;
    };
    exe.preforward();
    Tensor positions = torch::arange(S, ids.options()).unsqueeze(0).expand({B, S});
    Tensor x = one([&](const Tensor& i) { return tok->forward(i) + pos->forward(positions); }, ids, cswap::ACT, true);
    x = one([&](const Tensor& t) { return emb_ln->forward(t); }, x, cswap::BN);
    x = one([&](const Tensor& t) { return torch::dropout(t, p, train); }, x);
    for (int l = 0; l < d.layers; l++) {
      Tensor qq = one([&](const Tensor& t) { return q[l]->forward(t); }, x, cswap::FC);
      Tensor kk = one([&](const Tensor& t) { return k[l]->forward(t); }, x, cswap::FC);
      Tensor vv = one([&](const Tensor& t) { return v[l]->forward(t); }, x, cswap::FC);
      Tensor qh = one([&](const Tensor& t) { return t.view({B, S, nh, dh}).transpose(1, 2).contiguous(); }, qq);
      Tensor kh = one([&](const Tensor& t) { return t.view({B, S, nh, dh}).permute({0, 2, 3, 1}).contiguous(); }, kk);
      Tensor vh = one([&](const Tensor& t) { return t.view({B, S, nh, dh}).transpose(1, 2).contiguous(); }, vv);
      Tensor sc = two([&](const Tensor& a, const Tensor& b) { return torch::matmul(a, b) * (1.0 / std::sqrt((double)dh)); },
                      qh, kh, cswap::FC);
      Tensor pr = one([&](const Tensor& t) { return torch::softmax(t, -1); }, sc);
      pr = one([&](const Tensor& t) { return torch::dropout(t, p, train); }, pr);
      Tensor ctx = two([&](const Tensor& a, const Tensor& b) { return torch::matmul(a, b); }, pr, vh, cswap::FC);
      ctx = one([&](const Tensor& t) { return t.transpose(1, 2).reshape({B, S, H}); }, ctx);
      Tensor ao = one([&](const Tensor& t) { return o[l]->forward(t); }, ctx, cswap::FC);
      ao = one([&](const Tensor& t) { return torch::dropout(t, p, train); }, ao);
      x = two([&](const Tensor& a, const Tensor& b) { return ln1[l]->forward(a + b); }, ao, x, cswap::BN);
      Tensor h = one([&](const Tensor& t) { return f1[l]->forward(t); }, x, cswap::FC);
      h = one([&](const Tensor& t) { return torch::gelu(t); }, h);
      h = one([&](const Tensor& t) { return f2[l]->forward(t); }, h, cswap::FC);
      h = one([&](const Tensor& t) { return torch::dropout(t, p, train); }, h);
      x = two([&](const Tensor& a, const Tensor& b) { return ln2[l]->forward(a + b); }, h, x, cswap::BN);
    }
    Tensor cls = one([&](const Tensor& t) { return t.select(1, 0); }, x, cswap::ACT, true);
    Tensor logits = one([&](const Tensor& t) { return head->forward(t); }, cls, cswap::FC, true);
    Tensor loss = two([&](const Tensor& a, const Tensor& b) { return torch::nn::functional::cross_entropy(a, b); },
                      logits, target, cswap::ACT, true);
    exe.postforward();
    return loss;
  }
};

struct Batch {
  Tensor hx, hy;  // pinned host memory
};

static void zero_grads(Bert& net) {
  for (auto& p : net.parameters()) p.mutable_grad() = Tensor();
}

struct StepStats {
  double ms_mean = 0, ms_median = 0;
  float loss = 0;
  double act_out = 0, act_back = 0, link_out = 0, link_in = 0, peak_mib = 0;
  long swapped = 0, reclaimed = 0;
};

static StepStats timed_steps(Bert& net, Execution& exe, const Batch& b, int steps, int warmup) {
  torch::manual_seed(4321);  // the same dropout masks under every table: the rows' losses compare
  StepStats r;
  std::vector<double> ms;
  const int dev = c10::cuda::current_device();
  for (int it = 0; it < warmup + steps; it++) {
    if (it == warmup) {
      torch::cuda::synchronize();
      exe.reset_stats();
      exe.reclaimed = 0;
      c10::cuda::CUDACachingAllocator::resetPeakStats(dev);
    }
    at::cuda::CUDAEvent e0(cudaEventDefault), e1(cudaEventDefault);
    e0.record();
    auto x = b.hx.to(torch::kCUDA, /*non_blocking=*/true);
    auto y = b.hy.to(torch::kCUDA, /*non_blocking=*/true);
    zero_grads(net);
    auto loss = net.forward(exe, x, y);
    loss.backward();
    r.loss = loss.item<float>();  // device -> host read of the step's result
    e1.record();
    torch::cuda::synchronize();
    if (it >= warmup) ms.push_back(e0.elapsed_time(e1));
  }
  csw_mgr_sync(exe.manager());
  const csw_mgr_stats s = exe.stats();
  const double n = std::max(steps, 1);
  std::sort(ms.begin(), ms.end());
  r.ms_median = ms.empty() ? 0 : ms[ms.size() / 2];
  for (double m : ms) r.ms_mean += m / n;
  r.act_out = s.raw_bytes_out / n;
  r.act_back = s.raw_bytes_in / n;
  r.link_out = s.moved_bytes_out / n;
  r.link_in = s.moved_bytes_in / n;
  r.swapped = (long)(s.swap_outs / n);
  r.reclaimed = exe.reclaimed / std::max(steps, 1);
  r.peak_mib = c10::cuda::CUDACachingAllocator::getDeviceStats(dev).allocated_bytes[0].peak / 1048576.0;
  return r;
}

static int g_lookahead = 1;  // --lookahead: tensors whose return starts before backward asks

static void init_exe(Execution& exe, const Dims& d, int nids, unsigned maxbits) {
  exe.lookahead = g_lookahead;
  // pools sized for the model: about 1.5 GB of activations per layer at the BERT-base shape
  const size_t per_layer = (size_t)d.batch * d.seq * ((size_t)12 * d.hidden + 2 * d.ffn + 3 * (size_t)d.heads * d.seq) * 4;
  const size_t pinned = std::max<size_t>(size_t(1) << 30, per_layer * d.layers * 5 / 4);
  exe.init_(nids, maxbits, pinned, std::max<size_t>(size_t(512) << 20, pinned / 6));
}

// every tensor swapped under `pol` at its last forward use
static void fill(Execution& exe, const std::map<int, int>& last_use, int pol) {
  std::fill(exe.policy.begin(), exe.policy.end(), 0);
  for (auto& kv : last_use)
    if (kv.first < (int)exe.policy.size()) {
      exe.policy[kv.first] = pol;
      exe.begin_stage[kv.first] = kv.second;
    }
}

static std::map<int, cswap::LayerProfile> profile_step(Bert& net, Execution& exe, const Batch& b) {
  exe.profile = true;
  auto x = b.hx.to(torch::kCUDA);
  auto y = b.hy.to(torch::kCUDA);
  zero_grads(net);
  net.forward(exe, x, y).backward();
  return exe.finish_profile();
}

struct Result {
  float loss;
  std::vector<Tensor> grads;
};
static Result one_step(Bert& net, Execution& exe, const Batch& b, uint64_t seed) {
  torch::manual_seed(seed);  // dropout masks
  auto x = b.hx.to(torch::kCUDA);
  auto y = b.hy.to(torch::kCUDA);
  zero_grads(net);
  Result r;
  {
    auto loss = net.forward(exe, x, y);
    loss.backward();
    torch::cuda::synchronize();
    r.loss = loss.item<float>();
  }
  for (auto& p : net.parameters()) r.grads.push_back(p.grad().defined() ? p.grad().clone() : Tensor());
  return r;
}
static bool same(const Result& a, const Result& b) {
  bool ok = a.loss == b.loss && a.grads.size() == b.grads.size();
  for (size_t i = 0; ok && i < a.grads.size(); i++)
    ok = a.grads[i].defined() == b.grads[i].defined() && (!a.grads[i].defined() || torch::equal(a.grads[i], b.grads[i]));
  return ok;
}

static int run_check(Dims d) {
  torch::manual_seed(0);
  at::globalContext().setDeterministicCuDNN(true);
  at::globalContext().setDeterministicAlgorithms(true, /*warn_only=*/true);
  Bert net(d);
  net.to(torch::kCUDA);
  net.train();
  Batch b{torch::randint(0, d.vocab, {d.batch, d.seq}, torch::kLong).pin_memory(),
          torch::randint(0, 2, {d.batch}, torch::kLong).pin_memory()};
  const int nids = 20 * d.layers + 16;
  int bad = 0;
  Result base;
  std::map<int, int> last_use;
  {
    Execution exe;
    init_exe(exe, d, nids, 1024);
    auto prof = profile_step(net, exe, b);
    last_use = Execution::last_consumers(prof);
    base = one_step(net, exe, b, 5);
    Result again = one_step(net, exe, b, 5);
    std::printf("profiled %zu layers, %zu tensors with a consumer; step reproducible %d\n", prof.size(), last_use.size(),
                (int)same(again, base));
    if (!same(again, base)) bad++;
  }
  for (int pol : {CSW_POLICY_RAW, CSW_POLICY_SPARSE, CSW_POLICY_ZFP}) {
    Execution exe;
    init_exe(exe, d, nids, 1024);
    fill(exe, last_use, pol);
    Result r = one_step(net, exe, b, 5);
    const csw_mgr_stats s = exe.stats();
    // deviation of the whole gradient: |g - g0| / |g0| over all parameters (a per-parameter ratio
    // is meaningless for parameters whose true gradient is zero, like the key projection's bias)
    double num = 0, den = 0;
    for (size_t i = 0; i < r.grads.size(); i++)
      if (r.grads[i].defined()) {
        num += (r.grads[i] - base.grads[i]).to(torch::kFloat64).pow(2).sum().item<double>();
        den += base.grads[i].to(torch::kFloat64).pow(2).sum().item<double>();
      }
    const double maxrel = std::sqrt(num / (den + 1e-300));
    std::printf("policy %d: swap_outs %3llu swap_ins %3llu taken-back %3ld moved/raw %.3f identical %d relative gradient deviation "
                "%.3g\n",
                pol, (unsigned long long)s.swap_outs, (unsigned long long)s.swap_ins, exe.reclaimed,
                s.raw_bytes_out ? (double)s.moved_bytes_out / (double)s.raw_bytes_out : 0.0, (int)same(r, base), maxrel);
    if (s.swap_outs < 10u * d.layers) bad++;
    if (pol != CSW_POLICY_ZFP && !same(r, base)) bad++;
    // rate 16: the forward pass is untouched, the gradients move a little and only a little
    if (pol == CSW_POLICY_ZFP && (r.loss != base.loss || maxrel == 0.0 || maxrel > 0.05 ||
                                  (double)s.moved_bytes_out / (double)s.raw_bytes_out > 0.55))
      bad++;
  }
  std::printf(bad ? "FAIL\n" : "PASS\n");
  return bad ? 1 : 0;
}

static std::string row_json(const StepStats& r) {
  std::ostringstream o;
  o << "{\"ms_per_step_mean\": " << r.ms_mean << ", \"ms_per_step_median\": " << r.ms_median
    << ", \"activation_bytes_swapped\": " << r.act_out << ", \"activation_bytes_back\": " << r.act_back
    << ", \"link_bytes_out\": " << r.link_out << ", \"link_bytes_in\": " << r.link_in
    << ", \"peak_device_mib\": " << r.peak_mib << ", \"swap_outs\": " << r.swapped << ", \"taken_back\": " << r.reclaimed
    << ", \"loss\": " << r.loss << "}";
  return o.str();
}

static int run_bench(Dims d, int steps, int warmup, int seed) {
  torch::manual_seed(seed);
  Bert net(d);
  net.to(torch::kCUDA);
  net.train();
  Batch b{torch::randint(0, d.vocab, {d.batch, d.seq}, torch::kLong).pin_memory(),
          torch::randint(0, 2, {d.batch}, torch::kLong).pin_memory()};
  const int nids = 20 * d.layers + 16;
  Execution exe;
  init_exe(exe, d, nids, 1024);
  auto prof = profile_step(net, exe, b);
  const std::map<int, int> last_use = Execution::last_consumers(prof);
  std::ostringstream o;
  o << "{\"host_side\": \"cswap::Execution over libtorch (include/cswap_execution.hpp)\", \"layers\": " << d.layers
    << ", \"hidden\": " << d.hidden << ", \"heads\": " << d.heads << ", \"ffn\": " << d.ffn << ", \"seq\": " << d.seq
    << ", \"batch\": " << d.batch << ", \"zfp_maxbits\": 1024, \"steps\": " << steps << ", \"warmup\": " << warmup
    << ", \"rows\": {";
  fill(exe, {}, 0);
  const StepStats none = timed_steps(net, exe, b, steps, warmup);
  o << "\"no_swap\": " << row_json(none);
  fill(exe, last_use, CSW_POLICY_RAW);
  o << ", \"raw_swap\": " << row_json(timed_steps(net, exe, b, steps, warmup));
  fill(exe, last_use, CSW_POLICY_ZFP);
  o << ", \"zfp16_everywhere\": " << row_json(timed_steps(net, exe, b, steps, warmup));
  // the same with every staged payload released once it is on the host: all of it comes back over the link
  exe.keep_staged(false);
  o << ", \"zfp16_everywhere_nothing_kept_staged\": " << row_json(timed_steps(net, exe, b, steps, warmup));
  exe.keep_staged(true);
  // self-tuned: loss allowed on every float activation
  std::set<int> lossy;
  for (auto& kv : prof)
    if (kv.second.float32) lossy.insert(kv.first);
  exe.make_policy(prof, &lossy);
  int counts[7] = {0, 0, 0, 0, 0, 0, 0};
  for (int pcode : exe.policy) counts[pcode]++;
  const double predicted = exe.predicted_overhead_s(prof) * 1e3;
  const StepStats tuned = timed_steps(net, exe, b, steps, warmup);
  o << ", \"self_tuned\": " << row_json(tuned) << "}, \"self_tuned_policy_counts\": {\"0\": " << counts[0]
    << ", \"2\": " << counts[2] << ", \"3\": " << counts[3] << ", \"6\": " << counts[6]
    << "}, \"self_tuned_predicted_vs_measured_overhead_ms\": [" << predicted << ", " << tuned.ms_mean - none.ms_mean << "]}";
  std::printf("%s\n", o.str().c_str());
  return 0;
}

int main(int argc, char** argv) {
  if (!torch::cuda::is_available()) {
    std::fprintf(stderr, "needs a CUDA device\n");
    return 2;
  }
  bool check = false, bench = false;
  Dims d;
  int steps = 5, warmup = 3, device = 0, seed = 1;
  bool layers_given = false;
  for (int i = 1; i < argc; i++) {
    const std::string a = argv[i];
    auto val = [&](int& v) { if (i + 1 < argc) v = std::atoi(argv[++i]); };
    if (a == "--check") check = true;
    else if (a == "--bench") bench = true;
    else if (a == "--layers") { val(d.layers); layers_given = true; }
    else if (a == "--lookahead") val(g_lookahead);
    else if (a == "--hidden") val(d.hidden);
    else if (a == "--heads") val(d.heads);
    else if (a == "--ffn") val(d.ffn);
    else if (a == "--seq") val(d.seq);
    else if (a == "--batch") val(d.batch);
    else if (a == "--steps") val(steps);
    else if (a == "--warmup") val(warmup);
    else if (a == "--device") val(device);
    else if (a == "--seed") val(seed);
  }
  if (check && !layers_given) d.layers = 2;
  c10::cuda::set_device((c10::DeviceIndex)device);
  try {
    if (check) return run_check(d);
    if (bench) return run_bench(d, steps, warmup, seed);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "bert_step: %s\n", e.what());
    return 1;
  }
  std::fprintf(stderr, "usage: bert_step --check | --bench [--steps K] [--warmup W] [--layers L] [--batch B] [--device D]\n");
  return 2;
}
