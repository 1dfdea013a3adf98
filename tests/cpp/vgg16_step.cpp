// VGG16 training step for 3x32x32 inputs under cswap::Execution, laid out the
// way the reference's driver is (CSWAP+/vgg16-cifar10.cpp:77-245): a list of 45
// layer functions with their Layer_type, every layer wrapped in exe.pre /
// exe.post, then flatten, fc and the loss with the vector overloads.
//
//   vgg16_step --check            policies 0/1/2/3, the vDNN and SuperNeurons
//                                 planners and the self-tuned table must leave loss
//                                 and gradients bit-identical; policy 6 must hand
//                                 backward exactly decode(encode(x)).  Prints PASS.
//   vgg16_step --bench [--steps K] [--warmup W] [--batch B]
//                                 one JSON line: step time, link bytes and peak
//                                 device memory per policy table, and the
//                                 activation bytes that can be swapped within a
//                                 stated stretch of the no-swap step.
//
// Inputs are synthetic (N(0,1) images, uniform labels) and come from pinned host
// memory every step; the loss is read back every step.
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <torch/torch.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include "cswap_execution.hpp"

using cswap::Execution;
using cswap::Layer_type;
using Fn = std::function<torch::Tensor(const torch::Tensor&)>;

// ids of the conv inputs the reference compresses (vgg16-cifar10.cpp:396-397)
static const std::set<int> kConvInputs = {2, 6, 9, 13, 16, 19, 23, 26, 29, 33, 36, 39};

struct Net : torch::nn::Module {
  std::vector<Fn> v;
  std::vector<Layer_type> types;
  std::vector<torch::nn::Conv2d> convs;
  std::vector<int> conv_at;  // layer index of each conv
  torch::nn::Linear fc1{nullptr};
  std::function<void(int, torch::Tensor&)> tap;  // called with every layer's output (tests)

  Net() {
    const int cfg[] = {64, 64, 0, 128, 128, 0, 256, 256, 256, 0, 512, 512, 512, 0, 512, 512, 512, 0};
    int c_in = 3, nconv = 0, nbn = 0;
    for (int c : cfg) {
      if (c == 0) {
        v.push_back([](const torch::Tensor& t) { return torch::max_pool2d(t, 2); });
        types.push_back(cswap::POOL);
        continue;
      }
      auto conv = register_module("conv" + std::to_string(nconv++),
                                  torch::nn::Conv2d(torch::nn::Conv2dOptions(c_in, c, 3).padding(1)));
      auto bn = register_module("batchnorm_" + std::to_string(nbn++), torch::nn::BatchNorm2d(c));
      convs.push_back(conv);
      conv_at.push_back((int)v.size());
      v.push_back([conv](const torch::Tensor& t) mutable { return conv->forward(t); });
      // batch statistics only: running a layer a second time to rebuild a dropped
      // output must not move the running averages
      v.push_back([bn](const torch::Tensor& t) mutable {
        return torch::batch_norm(t, bn->weight, bn->bias, {}, {}, true, 0.0, bn->options.eps(), true);
      });
      v.push_back([](const torch::Tensor& t) { return torch::relu(t); });
      types.insert(types.end(), {cswap::CONV, cswap::BN, cswap::ACT});
      c_in = c;
    }
    v.push_back([](const torch::Tensor& t) { return torch::avg_pool2d(t, 1); });
    types.push_back(cswap::POOL);
    fc1 = register_module("fc1", torch::nn::Linear(512, 10));
  }

  // vgg16-cifar10.cpp:215-245
  torch::Tensor forward(Execution& exe, torch::Tensor x, torch::Tensor target) {
    torch::Tensor pre = x;
    exe.preforward();
    for (size_t index = 0; index < v.size(); index++) {
      exe.pre(pre, types[index]);
      x = v[index](pre);
      exe.post(pre, x, types[index], false, v[index]);
      if (tap) tap((int)index, x);
      pre = x;
    }
    exe.pre(pre, cswap::ACT);
    x = pre.view({pre.size(0), -1});
    exe.post(pre, x, cswap::ACT, true);
    pre = x;
    exe.pre(pre, cswap::ACT);
    x = fc1->forward(pre);
    exe.post(pre, x, cswap::FC, true);
    pre = x;
    exe.pre({pre, target}, cswap::ACT);
    x = torch::nn::functional::cross_entropy(pre, target);
    exe.post({pre, target}, x, cswap::ACT, true);
    exe.postforward();
    return x;
  }
};

struct Batch {
  torch::Tensor hx, hy;  // pinned host memory
};

struct StepStats {
  double ms_median = 0, ms_mean = 0;
  float loss = 0;
  double act_out = 0, act_back = 0, link_out = 0, link_in = 0;
  double peak_mib = 0;
  long swapped = 0, skipped = 0, reclaimed = 0, dropped = 0, recomputed = 0;
};

static void zero_grads(Net& net) {
  for (auto& p : net.parameters()) p.mutable_grad() = torch::Tensor();
}

// forward + backward `steps` times under exe's tables: the batch comes from pinned
// host memory and the loss is read back, both inside the timed region
static StepStats timed_steps(Net& net, Execution& exe, const Batch& b, int steps, int warmup) {
  StepStats r;
  std::vector<double> ms;
  const int dev = c10::cuda::current_device();
  for (int it = 0; it < warmup + steps; it++) {
    if (it == warmup) {
      torch::cuda::synchronize();
      exe.reset_stats();
      exe.skipped_unsaved = exe.reclaimed = exe.dropped = exe.recomputed = 0;
      c10::cuda::CUDACachingAllocator::resetPeakStats(dev);
    }
    at::cuda::CUDAEvent e0(cudaEventDefault), e1(cudaEventDefault);
    e0.record();
    auto x = b.hx.to(torch::kCUDA, /*non_blocking=*/true).requires_grad_(true);
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
  r.skipped = exe.skipped_unsaved / std::max(steps, 1);
  r.reclaimed = exe.reclaimed / std::max(steps, 1);
  r.dropped = exe.dropped / std::max(steps, 1);
  r.recomputed = exe.recomputed / std::max(steps, 1);
  const auto st = c10::cuda::CUDACachingAllocator::getDeviceStats(dev);
  r.peak_mib = st.allocated_bytes[0].peak / 1048576.0;
  return r;
}

static int g_lookahead = 1;  // --lookahead: tensors whose return starts before backward asks

static void init_tables(Execution& exe, int pol) {
  exe.init_(64, 512, size_t(2) << 30, size_t(512) << 20);
  exe.lookahead = g_lookahead;
  for (int i = 0; i < 50; i++) {
    exe.begin_stage[i] = i + 1;
    exe.policy[i] = pol;
  }
}
// the hard-wired setting of vgg16-cifar10.cpp:381-397
static void reference_split(Execution& exe) {
  init_tables(exe, CSW_POLICY_RAW);
  for (int i : kConvInputs) exe.policy[i] = CSW_POLICY_ZFP;
}

static std::map<int, cswap::LayerProfile> profile_step(Net& net, Execution& exe, const Batch& b) {
  exe.profile = true;
  auto x = b.hx.to(torch::kCUDA).requires_grad_(true);
  auto y = b.hy.to(torch::kCUDA);
  zero_grads(net);
  net.forward(exe, x, y).backward();
  return exe.finish_profile();
}

// the cost model's table against its ZFP-eager neighbour, three timed steps each
static std::string self_tune(Net& net, Execution& exe, const Batch& b, const std::map<int, cswap::LayerProfile>& prof,
                             const std::set<int>* lossy) {
  std::vector<int> model = exe.make_policy(prof, lossy);
  const std::vector<int> begin = exe.begin_stage;
  std::vector<int> eager = exe.make_policy(prof, lossy, 2.0, size_t(1) << 20, true);
  double best = 1e30;
  std::string chosen;
  std::vector<int> best_table;
  for (auto& cand : {std::make_pair(std::string("model"), model), std::make_pair(std::string("zfp_where_allowed"), eager)}) {
    exe.policy = cand.second;
    exe.begin_stage = begin;
    timed_steps(net, exe, b, 1, 0);
    const double t = timed_steps(net, exe, b, 3, 0).ms_mean;
    if (t < best) {
      best = t;
      chosen = cand.first;
      best_table = cand.second;
    }
  }
  exe.policy = best_table;
  exe.begin_stage = begin;
  return chosen;
}

// ---------------------------------------------------------------------------------------------
// --check
// ---------------------------------------------------------------------------------------------
struct Result {
  float loss;
  std::vector<torch::Tensor> grads;
};
static Result one_step(Net& net, Execution& exe, const Batch& b) {
  auto x = b.hx.to(torch::kCUDA).requires_grad_(true);
  auto y = b.hy.to(torch::kCUDA);
  zero_grads(net);
  Result r;
  {
    auto loss = net.forward(exe, x, y);
    loss.backward();
    torch::cuda::synchronize();
    r.loss = loss.item<float>();
  }
  for (auto& p : net.parameters()) r.grads.push_back(p.grad().clone());
  return r;
}
static bool same(const Result& a, const Result& b) {
  bool ok = a.loss == b.loss && a.grads.size() == b.grads.size();
  for (size_t i = 0; ok && i < a.grads.size(); i++) ok = torch::equal(a.grads[i], b.grads[i]);
  return ok;
}

static torch::Tensor through_codec(const torch::Tensor& act, unsigned maxbits) {
  auto flat = act.detach().contiguous().view(-1).clone();
  const size_t n = (size_t)flat.numel(), nz = n / 1024;
  size_t bytes = 0;
  csw_zfp_max_bytes(32, 32, nz, maxbits, &bytes);
  auto stream = torch::empty({(int64_t)bytes}, torch::TensorOptions().device(torch::kCUDA).dtype(torch::kUInt8));
  auto s = c10::cuda::getCurrentCUDAStream().stream();
  if (csw_zfp_compress(flat.data_ptr<float>(), 32, 32, nz, maxbits, stream.data_ptr(), bytes, nullptr, s) != CSW_OK ||
      csw_zfp_decompress(stream.data_ptr(), bytes, 32, 32, nz, maxbits, flat.data_ptr<float>(), s) != CSW_OK)
    throw std::runtime_error("codec call failed");
  return flat.view(act.sizes());
}

static int run_check(int batch) {
  torch::manual_seed(0);
  at::globalContext().setDeterministicCuDNN(true);
  at::globalContext().setBenchmarkCuDNN(false);
  Net net;
  net.to(torch::kCUDA);
  net.train();
  Batch b{torch::randn({batch, 3, 32, 32}).pin_memory(),
          torch::randint(0, 10, {batch}, torch::kLong).pin_memory()};
  int bad = 0;
  Result base;
  {
    Execution exe;
    init_tables(exe, CSW_POLICY_KEEP);
    base = one_step(net, exe, b);
  }
  auto report = [&](const char* name, const Result& r, Execution& exe, bool must_swap, bool must_drop) {
    const csw_mgr_stats s = exe.stats();
    const bool ok = same(r, base) && (!must_swap || s.swap_outs >= 10) && (!must_drop || exe.recomputed >= 5);
    std::printf("%-22s swap_outs %3llu swap_ins %3llu not-kept %3ld taken-back %3ld dropped %3ld rebuilt %3ld "
                "moved/raw %.3f identical %d\n",
                name, (unsigned long long)s.swap_outs, (unsigned long long)s.swap_ins, exe.skipped_unsaved,
                exe.reclaimed, exe.dropped, exe.recomputed,
                s.raw_bytes_out ? (double)s.moved_bytes_out / (double)s.raw_bytes_out : 0.0, (int)same(r, base));
    if (!ok) bad++;
  };
  for (int pol : {CSW_POLICY_RAW, CSW_POLICY_SPARSE}) {
    Execution exe;
    init_tables(exe, pol);
    Result r = one_step(net, exe, b);
    report(pol == CSW_POLICY_RAW ? "policy 2 (raw)" : "policy 3 (sparse)", r, exe, true, false);
  }
  {
    Execution exe;  // policy 1 everywhere: every rebuild pulls in the one before it
    init_tables(exe, CSW_POLICY_DROP);
    Result r = one_step(net, exe, b);
    report("policy 1 (drop)", r, exe, false, true);
  }
  for (int planner : {3, 4}) {
    Execution exe;
    init_tables(exe, CSW_POLICY_KEEP);
    exe.policy_ = planner;
    Result r = one_step(net, exe, b);
    report(planner == 3 ? "policy_ 3 (vDNN)" : "policy_ 4 (SuperNeurons)", r, exe, true, planner == 4);
  }
  {
    // self-tuned with loss allowed nowhere: raw and sparse only, so still bit-identical
    Execution exe;
    init_tables(exe, CSW_POLICY_KEEP);
    auto prof = profile_step(net, exe, b);
    const std::set<int> nowhere;
    exe.make_policy(prof, &nowhere);
    int n2 = 0, n3 = 0, n6 = 0;
    for (int p : exe.policy) n2 += p == 2, n3 += p == 3, n6 += p == 6;
    Result r = one_step(net, exe, b);
    std::printf("self-tuned lossless table: %d raw, %d sparse, %d zfp; profile says %zu layers\n", n2, n3, n6,
                prof.size());
    // BatchNorm outputs feed ReLUs that keep only their own result: the profile must know
    if (prof.size() < 48 || prof.at(1).saved || !prof.at(2).saved || !prof.at(0).saved || n6 != 0 || n2 + n3 < 5) bad++;
    report("self-tuned (lossless)", r, exe, false, false);
  }
  {
    // policy 6 on the two kinds of conv input (a ReLU output, id 2, and a pool output, id 6):
    // the conv's weight gradient must be the one computed from decode(encode(x))
    for (int id : {2, 6}) {
      Execution exe;
      init_tables(exe, CSW_POLICY_KEEP);
      exe.policy[id] = CSW_POLICY_ZFP;
      torch::Tensor act, grad_out;
      net.tap = [&](int index, torch::Tensor& x) {
        if (index == id) act = x.detach().clone();
        if (index == id + 1) x.register_hook([&](torch::Tensor g) { grad_out = g.detach().clone(); return g; });
      };
      Result r = one_step(net, exe, b);
      net.tap = nullptr;
      size_t ci = 0;
      while (net.conv_at[ci] != id + 1) ci++;
      auto& conv = net.convs[ci];
      auto lossy = through_codec(act, 512);
      auto bw = [&](const torch::Tensor& input) {
        return std::get<1>(at::convolution_backward(grad_out, input, conv->weight.detach(),
                                                    at::OptionalIntArrayRef(conv->bias.sizes()), {1, 1}, {1, 1}, {1, 1},
                                                    false, {0, 0}, 1, {true, true, true}));
      };
      auto got = conv->weight.grad();
      const double d_lossy = (got - bw(lossy)).abs().max().item<double>();
      const double d_exact = (got - bw(act)).abs().max().item<double>();
      const csw_mgr_stats s = exe.stats();
      std::printf("policy 6 on id %d: swap_outs %llu moved/raw %.3f  |dW - dW(codec(x))| %.3g  |dW - dW(x)| %.3g\n", id,
                  (unsigned long long)s.swap_outs, (double)s.moved_bytes_out / (double)s.raw_bytes_out, d_lossy, d_exact);
      if (r.loss != base.loss || s.swap_outs != 1 || d_exact == 0.0 || d_lossy > 1e-3 * d_exact) bad++;
    }
  }
  {
    // The engine's knobs change WHEN things move, never what comes back: ZFP-8 on every kept
    // activation gives the same loss and gradients, bit for bit, whether blocks are freed in
    // stream order or by polling, however many tensors are brought back ahead of need, and
    // whether staged payloads are kept on the device or come back over the link.
    Result z0;
    {
      Execution exe;
      init_tables(exe, CSW_POLICY_ZFP);
      z0 = one_step(net, exe, b);
    }
    struct Knobs { const char* name; bool free_after_codec; int lookahead; bool keep_staged; };
    for (const Knobs k : {Knobs{"blocks freed by polling", false, 1, true}, Knobs{"three tensors ahead", true, 3, true},
                          Knobs{"nothing kept staged", true, 1, false}, Knobs{"nothing ahead", false, 0, false}}) {
      Execution exe;
      init_tables(exe, CSW_POLICY_ZFP);
      exe.free_after_codec = k.free_after_codec;
      exe.lookahead = k.lookahead;
      exe.keep_staged(k.keep_staged);
      Result r = one_step(net, exe, b);
      const csw_mgr_stats s = exe.stats();
      const bool ok = same(r, z0) && s.swap_outs >= 10 && s.swap_ins == s.swap_outs;
      std::printf("ZFP-8 everywhere, %-24s swap_outs %3llu link bytes in %9llu identical to the default engine %d\n", k.name,
                  (unsigned long long)s.swap_outs, (unsigned long long)s.moved_bytes_in, (int)same(r, z0));
      if (!ok) bad++;
    }
  }
  std::printf(bad ? "FAIL\n" : "PASS\n");
  return bad ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------
// --bench
// ---------------------------------------------------------------------------------------------
static std::string row_json(const StepStats& r) {
  std::ostringstream o;
  o << "{\"ms_per_step_median\": " << r.ms_median << ", \"ms_per_step_mean\": " << r.ms_mean
    << ", \"activation_bytes_swapped\": " << r.act_out << ", \"activation_bytes_back\": " << r.act_back
    << ", \"link_bytes_out\": " << r.link_out << ", \"link_bytes_in\": " << r.link_in
    << ", \"peak_device_mib\": " << r.peak_mib << ", \"swap_outs\": " << r.swapped << ", \"not_kept\": " << r.skipped
    << ", \"taken_back\": " << r.reclaimed << ", \"dropped\": " << r.dropped << ", \"rebuilt\": " << r.recomputed
    << ", \"loss\": " << r.loss << "}";
  return o.str();
}

struct Sweep {
  std::vector<StepStats> curve;
  std::vector<double> hidden;  // per eps
  size_t candidates = 0;
};

// The k largest kept activations swapped under policy_of(id), k = 0, 1, 2, ...:
// how many activation bytes go out and come back while the median step stays
// within (1 + eps) of the no-swap step.
static Sweep hidden_sweep(Net& net, const Batch& b, const std::map<int, cswap::LayerProfile>& prof,
                          const std::function<int(int)>& policy_of, double t0, const std::vector<double>& eps,
                          int steps, int warmup) {
  std::map<int, int> consumer;
  for (auto& kv : prof)
    for (int tid : kv.second.inputs)
      if (tid >= 0 && !consumer.count(tid)) consumer[tid] = kv.first;
  std::vector<int> ids;
  for (auto& kv : prof) {
    const auto& p = kv.second;
    if (p.saved && p.float32 && p.has_grad && !p.omit && p.numel >= (size_t(1) << 18) && consumer.count(kv.first))
      ids.push_back(kv.first);
  }
  std::stable_sort(ids.begin(), ids.end(), [&](int a, int c) { return prof.at(a).numel > prof.at(c).numel; });
  Sweep sw;
  sw.candidates = ids.size();
  Execution exe;
  init_tables(exe, CSW_POLICY_KEEP);
  exe.keep_staged(false);  // strict: whatever comes back crosses the link again
  for (size_t k = 0; k <= ids.size(); k++) {
    std::fill(exe.policy.begin(), exe.policy.end(), 0);
    for (size_t j = 0; j < k; j++) {
      exe.policy[ids[j]] = policy_of(ids[j]);
      exe.begin_stage[ids[j]] = consumer[ids[j]];
    }
    sw.curve.push_back(timed_steps(net, exe, b, steps, warmup));
  }
  for (double e : eps) {
    double best = 0;
    for (auto& c : sw.curve)
      if (c.ms_median <= (1 + e) * t0) best = std::max(best, c.act_back);
    sw.hidden.push_back(best);
  }
  return sw;
}

static std::string sweep_json(const Sweep& s, const std::vector<double>& eps) {
  std::ostringstream o;
  o << "{\"candidates\": " << s.candidates << ", \"hidden_activation_bytes\": {";
  for (size_t i = 0; i < eps.size(); i++) o << (i ? ", " : "") << "\"" << eps[i] << "\": " << s.hidden[i];
  o << "}, \"curve\": [";
  for (size_t k = 0; k < s.curve.size(); k++)
    o << (k ? ", " : "") << "{\"k\": " << k << ", \"ms_median\": " << s.curve[k].ms_median
      << ", \"activation_bytes\": " << s.curve[k].act_back << ", \"link_bytes_out\": " << s.curve[k].link_out
      << ", \"link_bytes_in\": " << s.curve[k].link_in << "}";
  o << "]}";
  return o.str();
}

static int run_bench(int batch, int steps, int warmup, int seed) {
  torch::manual_seed(seed);
  Net net;
  net.to(torch::kCUDA);
  net.train();
  Batch b{torch::randn({batch, 3, 32, 32}).pin_memory(),
          torch::randint(0, 10, {batch}, torch::kLong).pin_memory()};
  std::ostringstream o;
  o << "{\"host_side\": \"cswap::Execution over libtorch (include/cswap_execution.hpp)\", \"batch\": " << batch
    << ", \"steps\": " << steps << ", \"warmup\": " << warmup << ", \"rows\": {";
  StepStats none;
  {
    Execution exe;
    init_tables(exe, CSW_POLICY_KEEP);
    none = timed_steps(net, exe, b, steps, warmup);
    o << "\"no_swap\": " << row_json(none);
  }
  {
    Execution exe;
    init_tables(exe, CSW_POLICY_RAW);
    o << ", \"raw_swap\": " << row_json(timed_steps(net, exe, b, steps, warmup));
  }
  {
    Execution exe;
    reference_split(exe);
    o << ", \"reference_split_zfp8\": " << row_json(timed_steps(net, exe, b, steps, warmup));
  }
  {
    Execution exe;
    init_tables(exe, CSW_POLICY_ZFP);
    o << ", \"zfp8_everywhere\": " << row_json(timed_steps(net, exe, b, steps, warmup));
  }
  {
    // the same with every staged payload released once it is on the host: all of it comes back over the link
    Execution exe;
    init_tables(exe, CSW_POLICY_ZFP);
    exe.keep_staged(false);
    o << ", \"zfp8_everywhere_nothing_kept_staged\": " << row_json(timed_steps(net, exe, b, steps, warmup));
  }
  for (int planner : {3, 4}) {
    Execution exe;
    init_tables(exe, CSW_POLICY_KEEP);
    exe.policy_ = planner;
    o << (planner == 3 ? ", \"vdnn_baseline\": " : ", \"superneurons_baseline\": ")
      << row_json(timed_steps(net, exe, b, steps, warmup));
  }
  std::map<int, cswap::LayerProfile> prof;
  {
    Execution exe;
    init_tables(exe, CSW_POLICY_KEEP);
    prof = profile_step(net, exe, b);
    const std::string chosen = self_tune(net, exe, b, prof, nullptr);
    int counts[7] = {0, 0, 0, 0, 0, 0, 0};
    for (int p : exe.policy) counts[p]++;
    o << ", \"self_tuned\": " << row_json(timed_steps(net, exe, b, steps, warmup)) << "}";
    o << ", \"self_tuned_chosen\": \"" << chosen << "\", \"self_tuned_policy_counts\": {\"0\": " << counts[0]
      << ", \"2\": " << counts[2] << ", \"3\": " << counts[3] << ", \"6\": " << counts[6] << "}";
    const csw_cost_model& cm = exe.cost_model();
    o << ", \"cost_model\": {\"d2h_GBps\": " << cm.d2h_bps / 1e9 << ", \"h2d_GBps\": " << cm.h2d_bps / 1e9
      << ", \"host_swap_us\": " << cm.host_swap_s * 1e6 << ", \"sparse_enc_ps_per_byte\": [" << cm.sparse_enc_b * 1e12
      << ", " << cm.sparse_enc_b75 * 1e12 << ", " << cm.sparse_enc_b90 * 1e12 << "]}";
    // what the model expects each table to add to the no-swap step, beside what it measured
    o << ", \"predicted_vs_measured_overhead_ms\": {";
    const std::vector<int> tuned = exe.policy, tuned_begin = exe.begin_stage;
    struct Case { const char* name; int fill; };
    bool first = true;
    for (Case c : {Case{"raw_swap", CSW_POLICY_RAW}, Case{"zfp8_everywhere", CSW_POLICY_ZFP}, Case{"self_tuned", -1}}) {
      if (c.fill >= 0) {
        for (int i = 0; i < 50; i++) {
          exe.begin_stage[i] = i + 1;
          exe.policy[i] = c.fill;
        }
      } else {
        exe.policy = tuned;
        exe.begin_stage = tuned_begin;
      }
      const double predicted = exe.predicted_overhead_s(prof) * 1e3;
      const double measured = timed_steps(net, exe, b, steps, warmup).ms_median - none.ms_median;
      o << (first ? "" : ", ") << "\"" << c.name << "\": [" << predicted << ", " << measured << "]";
      first = false;
    }
    o << "}";
    exe.policy = tuned;
    exe.begin_stage = tuned_begin;
  }
  const std::vector<double> eps = {0.1, 0.25, 0.5, 1.0};
  const double t0 = none.ms_median;
  auto lossless = [&](int id) { return prof.at(id).zero_fraction >= 0.3 ? CSW_POLICY_SPARSE : CSW_POLICY_RAW; };
  Sweep raw = hidden_sweep(net, b, prof, [](int) { return (int)CSW_POLICY_RAW; }, t0, eps, 6, 2);
  Sweep ref_rule = hidden_sweep(
      net, b, prof, [&](int id) { return kConvInputs.count(id) ? (int)CSW_POLICY_ZFP : lossless(id); }, t0, eps, 6, 2);
  Sweep zfp_all = hidden_sweep(net, b, prof, [](int) { return (int)CSW_POLICY_ZFP; }, t0, eps, 6, 2);
  o << ", \"hidden_activation_bytes\": {\"definition\": \"uncompressed activation bytes swapped out and back per step "
       "by the configuration that swaps the most while the median step stays within (1 + eps) of the no-swap step; "
       "candidates are the kept activations, largest first; no staged payload is kept on the device in this sweep, "
       "so everything that comes back crosses the link\", \"no_swap_ms\": "
    << t0 << ", \"target_ratio\": 2.0, \"per_policy\": {\"raw\": " << sweep_json(raw, eps)
    << ", \"compressed_reference_rule\": " << sweep_json(ref_rule, eps)
    << ", \"compressed_zfp8_everywhere\": " << sweep_json(zfp_all, eps) << "}, \"ratio_to_raw\": {";
  const Sweep* cmp[2] = {&ref_rule, &zfp_all};
  const char* names[2] = {"compressed_reference_rule", "compressed_zfp8_everywhere"};
  for (int c = 0; c < 2; c++) {
    o << (c ? ", " : "") << "\"" << names[c] << "\": {";
    for (size_t i = 0; i < eps.size(); i++) {
      o << (i ? ", " : "") << "\"" << eps[i] << "\": ";
      if (raw.hidden[i] > 0) o << cmp[c]->hidden[i] / raw.hidden[i];
      else o << "null";
    }
    o << "}";
  }
  o << "}}}";
  std::printf("%s\n", o.str().c_str());
  return 0;
}

int main(int argc, char** argv) {
  if (!torch::cuda::is_available()) {
    std::fprintf(stderr, "needs a CUDA device\n");
    return 2;
  }
  bool check = false, bench = false;
  int batch = 128, steps = 10, warmup = 3, device = 0, seed = 1;
  for (int i = 1; i < argc; i++) {
    const std::string a = argv[i];
    auto val = [&](int& v) { if (i + 1 < argc) v = std::atoi(argv[++i]); };
    if (a == "--check") check = true;
    else if (a == "--bench") bench = true;
    else if (a == "--batch") val(batch);
    else if (a == "--steps") val(steps);
    else if (a == "--warmup") val(warmup);
    else if (a == "--device") val(device);
    else if (a == "--seed") val(seed);
    else if (a == "--lookahead") val(g_lookahead);
  }
  c10::cuda::set_device((c10::DeviceIndex)device);
  try {
    if (check) return run_check(batch);
    if (bench) return run_bench(batch, steps, warmup, seed);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "vgg16_step: %s\n", e.what());
    return 1;
  }
  std::fprintf(stderr, "usage: vgg16_step --check | --bench [--steps K] [--warmup W] [--batch B] [--device D]\n");
  return 2;
}
