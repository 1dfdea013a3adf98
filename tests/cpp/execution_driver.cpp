// A small libtorch driver written the way the reference's drivers are
// (CSWAP+/vgg16-cifar10.cpp:215-245): every layer wrapped in exe.pre / exe.post.
// Runs one training step under policy 0 (keep), 2 (raw), 3 (sparse) and 6 (ZFP)
// and checks that the lossless policies leave loss and gradients bit-identical
// and that the lossy one stays close.  Prints PASS and exits 0 on success.
#include <torch/torch.h>

#include <cstdio>
#include <functional>
#include <vector>

#include "cswap_execution.hpp"

using cswap::Execution;
using cswap::Layer_type;

struct Net : torch::nn::Module {
  torch::nn::Conv2d c1{nullptr}, c2{nullptr}, c3{nullptr};
  torch::nn::Linear fc{nullptr};
  std::vector<std::function<torch::Tensor(const torch::Tensor&)>> v;
  std::vector<Layer_type> types;
  Net() {
    c1 = register_module("c1", torch::nn::Conv2d(torch::nn::Conv2dOptions(3, 32, 3).padding(1)));
    c2 = register_module("c2", torch::nn::Conv2d(torch::nn::Conv2dOptions(32, 32, 3).padding(1)));
    c3 = register_module("c3", torch::nn::Conv2d(torch::nn::Conv2dOptions(32, 64, 3).padding(1)));
    fc = register_module("fc", torch::nn::Linear(64 * 16 * 16, 10));
    v = {[this](const torch::Tensor& t) { return c1->forward(t); }, [](const torch::Tensor& t) { return torch::relu(t); },
         [this](const torch::Tensor& t) { return c2->forward(t); }, [](const torch::Tensor& t) { return torch::relu(t); },
         [](const torch::Tensor& t) { return torch::max_pool2d(t, 2); },
         [this](const torch::Tensor& t) { return c3->forward(t); }, [](const torch::Tensor& t) { return torch::relu(t); }};
    types = {cswap::CONV, cswap::ACT, cswap::CONV, cswap::ACT, cswap::POOL, cswap::CONV, cswap::ACT};
  }
  torch::Tensor forward(Execution& exe, torch::Tensor x, torch::Tensor target) {
    torch::Tensor pre = x;
    exe.preforward();
    for (size_t i = 0; i < v.size(); i++) {
      exe.pre(pre, types[i]);
      x = v[i](pre);
      exe.post(pre, x, types[i]);
      pre = x;
    }
    exe.pre(pre);
    x = pre.view({pre.size(0), -1});
    exe.post(pre, x, cswap::ACT, true);
    pre = x;
    exe.pre(pre);
    x = fc->forward(pre);
    exe.post(pre, x, cswap::FC, true);
    pre = x;
    exe.pre({pre, target});
    x = torch::nn::functional::cross_entropy(pre, target);
    exe.post({pre, target}, x, cswap::ACT, true);
    exe.postforward();
    return x;
  }
};

struct StepResult {
  float loss;
  std::vector<torch::Tensor> grads;
  csw_mgr_stats stats;
};

// pol 6 follows the reference's split (vgg16-cifar10.cpp:381-397): ZFP on the
// conv inputs (the ReLU / pool outputs), raw swap for everything else
static StepResult step(Net& net, int pol, const torch::Tensor& x, const torch::Tensor& y) {
  Execution exe;
  exe.init_(32, 512, size_t(256) << 20, size_t(128) << 20);
  for (int i = 0; i < 8; i++) {
    exe.begin_stage[i] = i + 1;
    exe.policy[i] = pol == 6 ? 2 : pol;
  }
  if (pol == 6) exe.policy[1] = exe.policy[4] = 6;
  for (auto& p : net.parameters()) p.mutable_grad() = torch::Tensor();
  StepResult r;
  {
    torch::Tensor loss = net.forward(exe, x, y);
    loss.backward();
    torch::cuda::synchronize();
    r.loss = loss.item<float>();
  }
  for (auto& p : net.parameters()) r.grads.push_back(p.grad().clone());
  r.stats = exe.stats();
  return r;
}

int main() {
  if (!torch::cuda::is_available()) {
    std::fprintf(stderr, "needs a CUDA device\n");
    return 2;
  }
  torch::manual_seed(0);
  at::globalContext().setDeterministicCuDNN(true);
  Net net;
  net.to(torch::kCUDA);
  auto x = torch::randn({64, 3, 32, 32}, torch::kCUDA);
  auto y = torch::randint(0, 10, {64}, torch::TensorOptions().device(torch::kCUDA).dtype(torch::kLong));
  StepResult base = step(net, 0, x, y);
  int bad = 0;
  for (int pol : {2, 3}) {
    StepResult r = step(net, pol, x, y);
    bool same = r.loss == base.loss;
    for (size_t i = 0; i < r.grads.size(); i++) same = same && torch::equal(r.grads[i], base.grads[i]);
    std::printf("policy %d: swap_outs %llu swap_ins %llu moved/raw %.3f identical %d\n", pol,
                (unsigned long long)r.stats.swap_outs, (unsigned long long)r.stats.swap_ins,
                (double)r.stats.moved_bytes_out / (double)r.stats.raw_bytes_out, (int)same);
    if (!same || r.stats.swap_outs < 5 || r.stats.swap_ins < 3) bad++;
  }
  {
    StepResult r = step(net, 6, x, y);
    double maxrel = 0;
    bool finite = true;
    for (size_t i = 0; i < r.grads.size(); i++) {
      finite = finite && torch::isfinite(r.grads[i]).all().item<bool>();
      double d = (r.grads[i] - base.grads[i]).abs().max().item<double>();
      double s = base.grads[i].abs().max().item<double>() + 1e-12;
      maxrel = std::max(maxrel, d / s);
    }
    std::printf("policy 6: swap_outs %llu moved/raw %.3f max relative gradient deviation %.4f\n",
                (unsigned long long)r.stats.swap_outs, (double)r.stats.moved_bytes_out / (double)r.stats.raw_bytes_out,
                maxrel);
    if (!finite || r.loss != base.loss || maxrel > 2.0 || maxrel == 0.0 ||
        (double)r.stats.moved_bytes_out / (double)r.stats.raw_bytes_out > 0.9)
      bad++;
  }
  std::printf(bad ? "FAIL\n" : "PASS\n");
  return bad ? 1 : 0;
}
