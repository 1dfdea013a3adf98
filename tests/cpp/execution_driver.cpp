// A small libtorch driver written the way the reference's drivers are
// (CSWAP+/vgg16-cifar10.cpp:215-245): every layer wrapped in exe.pre / exe.post.
// Runs one training step under policy 0 (keep), 2 (raw), 3 (sparse) and 6 (ZFP)
// and checks that the lossless policies leave loss and gradients bit-identical
// and that under the lossy one the consuming convolution's weight gradient is
// the one computed from decode(encode(x)).  Prints PASS and exits 0 on success.
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
  std::function<void(size_t, torch::Tensor&)> tap;  // called with every layer's output
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
      if (tap) tap(i, x);
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
    // the three conv outputs feed ReLUs, which keep only their own result: they are not copied out
    if (!same || r.stats.swap_outs < 3 || r.stats.swap_ins < 2) bad++;
  }
  {
    // ids 1 (a ReLU output) and 4 (the pool output) go through ZFP: conv c2 consumes id 1
    torch::Tensor act, grad_out;
    net.tap = [&](size_t i, torch::Tensor& t) {
      if (i == 1) act = t.detach().clone();
      if (i == 2) t.register_hook([&](torch::Tensor g) { grad_out = g.detach().clone(); return g; });
    };
    StepResult r = step(net, 6, x, y);
    net.tap = nullptr;
    auto flat = act.contiguous().view(-1).clone();
    const size_t nz = (size_t)flat.numel() / 1024;
    size_t bytes = 0;
    csw_zfp_max_bytes(32, 32, nz, 512, &bytes);
    auto stream = torch::empty({(int64_t)bytes}, torch::TensorOptions().device(torch::kCUDA).dtype(torch::kUInt8));
    auto cu = c10::cuda::getCurrentCUDAStream().stream();
    bool codec_ok =
        csw_zfp_compress(flat.data_ptr<float>(), 32, 32, nz, 512, stream.data_ptr(), bytes, nullptr, cu) == CSW_OK &&
        csw_zfp_decompress(stream.data_ptr(), bytes, 32, 32, nz, 512, flat.data_ptr<float>(), cu) == CSW_OK;
    auto lossy = flat.view(act.sizes());
    auto bw = [&](const torch::Tensor& input) {
      return std::get<1>(at::convolution_backward(grad_out, input, net.c2->weight.detach(),
                                                  at::OptionalIntArrayRef(net.c2->bias.sizes()), {1, 1}, {1, 1}, {1, 1},
                                                  false, {0, 0}, 1, {true, true, true}));
    };
    auto got = net.c2->weight.grad();
    const double d_lossy = (got - bw(lossy)).abs().max().item<double>();
    const double d_exact = (got - bw(act)).abs().max().item<double>();
    std::printf("policy 6: swap_outs %llu moved/raw %.3f  |dW - dW(codec(x))| %.3g  |dW - dW(x)| %.3g\n",
                (unsigned long long)r.stats.swap_outs, (double)r.stats.moved_bytes_out / (double)r.stats.raw_bytes_out,
                d_lossy, d_exact);
    if (!codec_ok || r.loss != base.loss || d_exact == 0.0 || d_lossy > 1e-3 * d_exact ||
        (double)r.stats.moved_bytes_out / (double)r.stats.raw_bytes_out > 0.9)
      bad++;
  }
  std::printf(bad ? "FAIL\n" : "PASS\n");
  return bad ? 1 : 0;
}
