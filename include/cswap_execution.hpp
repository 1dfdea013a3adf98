// Execution - the reference's swap orchestrator (CSWAP+/Execution.h:38-447) on
// stock libtorch, over the C ABI of libcswap_b200.so.
//
// Same surface as the reference class: init_, preforward, pre, post,
// postforward, setRatio, the public tables policy / begin_stage / types, index
// and policy_, the Layer_type enum (Execution.h:28-35) and the policy codes
// 0 keep, 1 drop and rebuild, 2 raw, 3 sparse, 6 ZFP.  A driver wraps each
// layer exactly as the reference's drivers do (vgg16-cifar10.cpp:219-226):
//
//     exe.pre(pre, type);  x = layer(pre);  exe.post(pre, x, type, false, layer);  pre = x;
//
// What is different underneath:
//  * the fork-only members the reference writes (Tensor::tensor_id,
//    Node::com_and_tran / storage_impl_ / pre_node / func_ ...) do not exist
//    upstream; tensor ids are kept in a side table keyed by the tensor's
//    TensorImpl, the producer the reference stores in grad_fn()->func_
//    (vgg16-cifar10.cpp:223) is the optional last argument of post(), and the
//    swap-in runs from a FunctionPreHook on the consumer's grad_fn, which
//    autograd always runs before the producer's own backward;
//  * swap-out and swap-in go through csw_swap_out / csw_swap_in: events between
//    streams, pooled pinned memory, no stream synchronisation, no blocking read
//    of the sparse count (Execution.h:77,92,236);
//  * a tensor's device block goes back to the caching allocator as soon as it is
//    safe: under the compressed policies the compute stream waits for the codec's
//    read of it (tens of microseconds) and the block is freed at once, in stream
//    order, so the next layer reuses it however far the host runs ahead of the
//    GPU; under raw swap, whose read is the copy itself, the block is freed when
//    a poll finds the copy finished (never waited for);
//  * tensors come back one step ahead of need (copy and decode started when the
//    tensor swapped out after them is restored), from the payload still staged
//    on the device where the manager has kept it;
//  * a tensor that nothing holds for backward once its consumer has run is not
//    copied out at all, and a losslessly swapped tensor that backward asks for
//    before its copy out has finished is handed back as it is;
//  * the profiling record the reference sends to its policy maker
//    (Execution.h:220-234,318-331) is kept per layer here and make_policy()
//    turns it into a policy table through csw_cost_fit / csw_cost_decide.
//
// Constraints inherited from the reference's scheme: begin_stage[id] must be the
// LAST forward use of tensor id (its storage is empty afterwards until backward
// restores it), and only whole, contiguous float32 CUDA storages are swapped.
#pragma once
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/autograd/function.h>
#include <torch/csrc/autograd/function_hook.h>
#include <torch/torch.h>

#include <algorithm>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "cswap_b200.h"

namespace cswap {

enum Layer_type { CONV, POOL, ACT, BN, FC, MASKFILL };

using Producer = std::function<torch::Tensor(const torch::Tensor&)>;

// What one profiled layer recorded (Execution.h:220-234): its time, the size
// and sparsity of its output, which tensors it consumed and whether anything
// keeps its output for backward.
struct LayerProfile {
  double time_s = 0;
  size_t numel = 0;
  double zero_fraction = -1;
  std::vector<int> inputs;
  bool omit = false;
  int type = ACT;
  bool float32 = false, has_grad = false, saved = true, recomputable = false;
  double bwd_start_s = -1;  // backward compute that ran before this layer's own backward began (-1: not seen)
};

class Execution {
 public:
  Execution() = default;
  Execution(const Execution&) = delete;
  Execution& operator=(const Execution&) = delete;
  ~Execution() {
    drain();
    if (mgr_) csw_mgr_destroy(mgr_);
  }

  // Execution.h:46-64.  setRatio(bits per zfp block) is the zfp_maxbits argument.
  void init_(int n, unsigned zfp_maxbits = 512, size_t pinned_bytes = size_t(1) << 30,
             size_t staging_bytes = size_t(512) << 20) {
    policy.assign(n, 0);
    begin_stage.assign(n, 0);
    if (!mgr_) {
      csw_mgr_config cfg{};
      cfg.device = c10::cuda::current_device();
      cfg.pinned_bytes = pinned_bytes;
      cfg.staging_bytes = staging_bytes;
      cfg.zfp_maxbits = zfp_maxbits;
      check(csw_mgr_create(&cfg, &mgr_), "csw_mgr_create");
    } else {
      check(csw_mgr_set_zfp_maxbits(mgr_, zfp_maxbits), "csw_mgr_set_zfp_maxbits");
    }
    maxbits_ = zfp_maxbits;
  }
  // See csw_mgr_keep_staged: compressed payloads kept on the device while the staging pool has room.
  void keep_staged(bool keep) { check(csw_mgr_keep_staged(mgr_, keep ? 1 : 0), "csw_mgr_keep_staged"); }
  void setRatio(unsigned maxbits) {
    check(csw_mgr_set_zfp_maxbits(mgr_, maxbits), "csw_mgr_set_zfp_maxbits");
    maxbits_ = maxbits;
  }

  // Execution.h:403-412
  void preforward() {
    index = -1;
    ids_.clear();
    pending_.clear();
    deferred_.clear();
    order_.clear();
    by_storage_.clear();
    producers_.clear();
    handles_.clear();
    poll();
  }
  void postforward() {
    producers_.clear();  // they hold their layers' inputs: nothing is dropped after the forward pass
    handles_.clear();
    poll();
  }

  // Execution.h:65-133
  void pre(torch::Tensor& t, Layer_type layer_type = ACT) {
    index++;
    maybe_swap_out(t, layer_type, 0);
    begin_profile();
  }
  // Execution.h:135-212.  The braced form the reference's drivers use
  // (`exe.pre({pre, target})`) binds to the initializer_list overload, whose
  // backing array holds exactly one extra handle per tensor while the call runs;
  // a vector passed by name holds none beyond the caller's own.
  void pre(std::initializer_list<torch::Tensor> inputs, Layer_type layer_type = ACT) {
    index++;
    for (auto& t : inputs) maybe_swap_out(t, layer_type, 1);
    begin_profile();
  }
  void pre(const std::vector<torch::Tensor>& inputs, Layer_type layer_type = ACT) {
    index++;
    for (auto& t : inputs) maybe_swap_out(t, layer_type, 0);
    begin_profile();
  }
  // Execution.h:217-310.  `producer`, when given, is the layer itself: what
  // rebuilds x from pre_t should x be dropped under policy 1.
  void post(torch::Tensor& pre_t, torch::Tensor& x, Layer_type layer_type = ACT, bool isomit = false,
            Producer producer = nullptr) {
    const torch::Tensor* in[1] = {&pre_t};
    finish_layer(in, 1, 0, x, layer_type, isomit, std::move(producer));
  }
  // Execution.h:311-401
  void post(std::initializer_list<torch::Tensor> inputs, torch::Tensor& x, Layer_type layer_type = ACT,
            bool isomit = false) {
    std::vector<const torch::Tensor*> in;
    for (auto& t : inputs) in.push_back(&t);
    finish_layer(in.data(), in.size(), 1, x, layer_type, isomit, nullptr);
  }
  void post(const std::vector<torch::Tensor>& inputs, torch::Tensor& x, Layer_type layer_type = ACT,
            bool isomit = false) {
    std::vector<const torch::Tensor*> in;
    for (auto& t : inputs) in.push_back(&t);
    finish_layer(in.data(), in.size(), 0, x, layer_type, isomit, nullptr);
  }

  // ---- self-tuning (call sites Execution.h:224-233, resnet-cifar10.cpp:407-437) ----
  // Set before a forward + backward pass to record it; finish_profile() turns
  // the events into numbers (synchronises the device).
  bool profile = false;
  std::map<int, LayerProfile> finish_profile() {
    c10::cuda::device_synchronize();
    std::map<int, LayerProfile> out;
    // backward runs the layers last to first: the mark of the last layer seen is where it began
    const ProfEntry* first = nullptr;
    for (auto it = prof_.rbegin(); it != prof_.rend() && !first; ++it)
      if (it->second.bwd_seen) first = &it->second;
    for (auto& kv : prof_) {
      LayerProfile p = kv.second.p;
      p.time_s = kv.second.start.elapsed_time(kv.second.end) * 1e-3;
      if (kv.second.zeros.defined()) p.zero_fraction = kv.second.zeros.item<double>();
      if (first && kv.second.bwd_seen) p.bwd_start_s = first->bwd.elapsed_time(kv.second.bwd) * 1e-3;
      out[kv.first] = p;
    }
    prof_.clear();
    profile = false;
    return out;
  }

  // The fitted cost model of this device (measured once, on first use).
  const csw_cost_model& cost_model() {
    if (!fitted_) {
      cost_ = csw_cost_model{};
      cost_.zfp_maxbits = maxbits_;
      check(csw_cost_fit(mgr_, &cost_), "csw_cost_fit");
      fitted_ = true;
    }
    return cost_;
  }

  // Fill policy / begin_stage from a profiled iteration.  Tensor id i (the
  // output of layer i) becomes a swap candidate at the last layer that
  // consumes it; the cost model gets the forward time at which that consumer
  // starts and the backward compute that precedes the consumer's backward
  // (bwd_factor times the forward time of the later layers) and simulates the
  // step's link traffic to choose raw / sparse / ZFP.  ZFP is allowed on
  // `lossy_ids` (nullptr: the inputs of CONV layers, where the reference's
  // drivers apply it, vgg16-cifar10.cpp:381-397).  `all_zfp_where_allowed`
  // builds the table's neighbour instead: ZFP on every tensor where loss is
  // allowed, the model's choice elsewhere.
  std::vector<int> make_policy(const std::map<int, LayerProfile>& prof, const std::set<int>* lossy_ids = nullptr,
                               double bwd_factor = 2.0, size_t min_bytes = size_t(1) << 20,
                               bool all_zfp_where_allowed = false) {
    Candidates c = candidates(prof, lossy_ids, bwd_factor, min_bytes);
    if ((int)policy.size() < c.n) {
      policy.resize(c.n, 0);
      begin_stage.resize(c.n, 0);
    }
    std::vector<int> pol(c.descs.size() ? c.descs.size() : 1);
    std::vector<double> stall(pol.size());
    if (!c.descs.empty())
      check(csw_cost_decide(&cost_model(), c.descs.data(), c.descs.size(), c.fwd_total, pol.data(), stall.data()),
            "csw_cost_decide");
    for (int i = 0; i < c.n; i++) policy[i] = 0;
    for (size_t k = 0; k < c.ids.size(); k++) {
      int p = pol[k];
      if (all_zfp_where_allowed && c.descs[k].lossy_ok && c.descs[k].numel >= 1024) p = CSW_POLICY_ZFP;
      policy[c.ids[k]] = p;
      begin_stage[c.ids[k]] = c.consumer[c.ids[k]];
    }
    return policy;
  }

  // What the cost model expects the current policy table to cost: the step's
  // modelled stall in seconds (link and codec time that compute does not hide)
  // plus the host time of the swaps themselves.
  double predicted_overhead_s(const std::map<int, LayerProfile>& prof, double bwd_factor = 2.0) {
    Candidates c = candidates(prof, nullptr, bwd_factor, 0);
    std::vector<int> pol;
    size_t swaps = 0;
    for (int id : c.ids) {
      int p = id < (int)policy.size() ? policy[id] : 0;
      if (p != CSW_POLICY_RAW && p != CSW_POLICY_SPARSE && p != CSW_POLICY_ZFP) p = CSW_POLICY_KEEP;
      swaps += p != CSW_POLICY_KEEP;
      pol.push_back(p);
    }
    double total = 0;
    if (!c.descs.empty())
      check(csw_cost_simulate(&cost_model(), c.descs.data(), c.descs.size(), c.fwd_total, pol.data(), nullptr, &total),
            "csw_cost_simulate");
    return total + swaps * cost_model().host_swap_s;
  }

  // begin_stage for every tensor id of a profiled iteration: the last layer that consumes it.
  static std::map<int, int> last_consumers(const std::map<int, LayerProfile>& prof) {
    std::map<int, int> last;
    for (auto& kv : prof)
      for (int tid : kv.second.inputs)
        if (tid >= 0) last[tid] = kv.first;
    return last;
  }

  csw_mgr* manager() const { return mgr_; }
  csw_mgr_stats stats() const {
    csw_mgr_stats s{};
    csw_mgr_get_stats(mgr_, &s);
    return s;
  }
  void reset_stats() { csw_mgr_reset_stats(mgr_); }

  int index = -1;
  bool free_after_codec = true;  // compressed policies: the compute stream waits for the codec's read, the block is freed at once
  int lookahead = 1;          // swapped tensors whose return is started before backward asks for them
  long reclaimed = 0;         // tensors taken back before they had left the device
  long skipped_unsaved = 0;   // tensors nothing kept for backward: not copied out
  long dropped = 0;           // policy 1: let go without a copy
  long recomputed = 0;        // ... and rebuilt in backward
  std::vector<int> policy;
  std::vector<int> begin_stage;
  std::vector<Layer_type> types;
  int policy_ = 1;  // 1 CSWAP, 2 Capuchin, 3 vDNN, 4 SuperNeurons (Execution.h:420)

 private:
  // One swapped-out or dropped storage, shared between the tables below and the backward hook.
  struct Swapped {
    Execution* exe = nullptr;
    c10::intrusive_ptr<c10::StorageImpl> storage;
    csw_ticket* ticket = nullptr;
    size_t nbytes = 0;
    int order = -1;         // position among this step's swap-outs
    int policy = 0;
    bool restored = false;
    bool started = false;   // the copy out (or the drop) has been issued
    at::DataPtr reading;    // the device block while the manager still reads it
    at::DataPtr ahead;      // destination of a swap-in started before the tensor was asked for
    // policy 1: how to rebuild the tensor
    Producer producer;
    torch::Tensor producer_input;
    ~Swapped() {
      // a swap-in started ahead of time that nobody waited for may still be writing its block
      if (ahead.get() != nullptr && exe && exe->mgr_) csw_mgr_sync(exe->mgr_);
      if (ticket && exe && exe->mgr_) csw_ticket_release(exe->mgr_, ticket);
    }
  };

  // A tensor whose swap waits for its consumer to have run: only the consumer
  // can still save it for backward, and an unsaved tensor is not worth a copy.
  struct Deferred {
    torch::Tensor t;
    int pol;
  };

  struct RestoreHook : torch::autograd::FunctionPreHook {
    std::shared_ptr<Swapped> s;
    explicit RestoreHook(std::shared_ptr<Swapped> sw) : s(std::move(sw)) {}
    torch::autograd::variable_list operator()(const torch::autograd::variable_list& grads) override {
      if (!s->restored) s->exe->restore(*s);
      return grads;
    }
  };

  // Profiling: marks the moment a layer's backward begins.
  struct BackwardMark : torch::autograd::FunctionPreHook {
    Execution* exe;
    int layer;
    BackwardMark(Execution* e, int l) : exe(e), layer(l) {}
    torch::autograd::variable_list operator()(const torch::autograd::variable_list& grads) override {
      auto it = exe->prof_.find(layer);
      if (exe->profile && it != exe->prof_.end() && !it->second.bwd_seen) {
        it->second.bwd.record(c10::cuda::getCurrentCUDAStream());
        it->second.bwd_seen = true;
      }
      return grads;
    }
  };

  struct ProfEntry {
    at::cuda::CUDAEvent start{cudaEventDefault}, end{cudaEventDefault}, bwd{cudaEventDefault};
    bool bwd_seen = false;
    torch::Tensor zeros;  // fraction of zeros in the output, still on the device
    LayerProfile p;
  };

  // Swap candidates of a profiled iteration, in the order their consumers run,
  // with what the cost model needs to know about each.
  struct Candidates {
    int n = 0;
    double fwd_total = 0;
    std::map<int, int> consumer;
    std::vector<int> ids;
    std::vector<csw_tensor_desc> descs;
  };
  static Candidates candidates(const std::map<int, LayerProfile>& prof, const std::set<int>* lossy_ids,
                               double bwd_factor, size_t min_bytes) {
    Candidates c;
    c.n = prof.empty() ? 0 : prof.rbegin()->first + 1;
    std::vector<double> start(c.n + 1, 0.0);
    for (int i = 0; i < c.n; i++) {
      auto it = prof.find(i);
      start[i + 1] = start[i] + (it == prof.end() ? 0.0 : it->second.time_s);
    }
    c.fwd_total = start[c.n];
    // a tensor is swapped at its LAST forward use (its storage is empty from then on), which is
    // also the consumer whose backward runs first
    std::set<int> conv_inputs;
    for (auto& kv : prof)
      for (int tid : kv.second.inputs)
        if (tid >= 0) {
          c.consumer[tid] = kv.first;  // prof is ordered by layer: the last one wins
          if (kv.second.type == CONV) conv_inputs.insert(tid);
        }
    const std::set<int>& lossy = lossy_ids ? *lossy_ids : conv_inputs;
    std::vector<std::pair<int, int>> by_consumer;  // (consumer, id)
    for (auto& kv : c.consumer) by_consumer.push_back({kv.second, kv.first});
    std::sort(by_consumer.begin(), by_consumer.end());
    for (auto& ci : by_consumer) {
      auto it = prof.find(ci.second);
      if (it == prof.end()) continue;
      const LayerProfile& p = it->second;
      if (p.omit || !p.float32 || !p.has_grad || p.numel * 4 < min_bytes || !p.saved) continue;
      csw_tensor_desc d{};
      d.numel = p.numel;
      d.zero_fraction = p.zero_fraction;
      d.lossy_ok = lossy.count(ci.second) ? 1 : 0;
      d.ready_s = start[ci.first];
      // the tensor is needed when its consumer's backward begins: measured in the profiled
      // iteration where that was seen, else estimated from the forward times of the later layers
      auto cit = prof.find(ci.first);
      d.need_s = cit != prof.end() && cit->second.bwd_start_s >= 0 ? cit->second.bwd_start_s
                                                                  : bwd_factor * (c.fwd_total - start[ci.first + 1]);
      c.ids.push_back(ci.second);
      c.descs.push_back(d);
    }
    return c;
  }

  static void check(csw_status st, const char* what) {
    if (st != CSW_OK) throw std::runtime_error(std::string(what) + ": " + csw_status_string(st));
  }

  int id_of(const torch::Tensor& t) const {
    auto it = ids_.find(t.unsafeGetTensorImpl());
    return it == ids_.end() ? -1 : it->second;
  }

  static bool swappable(const torch::Tensor& t) {
    return t.defined() && t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous() &&
           t.storage_offset() == 0 && t.numel() >= 1024 && t.storage().nbytes() == size_t(t.numel()) * 4 &&
           t.storage().data() != nullptr;  // not already swapped out through another view
  }

  int effective_policy(int id, Layer_type layer_type) const {
    int pol = policy[id];
    if (pol == CSW_POLICY_DROP || (policy_ == 4 && layer_type != CONV))
      return CSW_POLICY_DROP;  // Execution.h:243: SuperNeurons rebuilds the inputs of non-conv layers
    if (layer_type == CONV && policy_ > 2) return CSW_POLICY_RAW;  // vDNN / SuperNeurons (Execution.h:70,248)
    return pol;
  }

  void maybe_swap_out(const torch::Tensor& t, Layer_type layer_type, size_t call_copies) {
    const int id = id_of(t);
    if (id < 0 || id >= (int)begin_stage.size() || index != begin_stage[id] || !t.grad_fn()) return;
    const int pol = effective_policy(id, layer_type);
    if ((pol != CSW_POLICY_DROP && pol != CSW_POLICY_RAW && pol != CSW_POLICY_SPARSE && pol != CSW_POLICY_ZFP) ||
        !swappable(t))
      return;
    {
      auto seen = by_storage_.find(t.storage().unsafeGetStorageImpl());
      if (seen != by_storage_.end() && !seen->second.expired()) return;
    }
    if (pol == CSW_POLICY_DROP && !producers_.count(t.unsafeGetTensorImpl()))
      return;  // without its producer the tensor simply stays
    // kept by its producer (a ReLU keeps its own result): it will be needed again, so the copy
    // out can start now and overlap with the layer about to run.  Otherwise decide in post().
    if (producer_kept(t)) start_swap(t, pol);
    else deferred_.push_back(Deferred{t, pol});
  }

  // Autograd adds a reference to the storage when a producer saves its own
  // result (it keeps a detached alias of it).
  bool producer_kept(const torch::Tensor& t) const {
    auto own = by_storage_.find(t.storage().unsafeGetStorageImpl());
    return t.storage().use_count() > 1 + ((own != by_storage_.end() && !own->second.expired()) ? 1u : 0u);
  }

  // Does anything hold `t` for backward?  Asked from post(), after the consumer
  // has run.  A consumer that saves its input adds a reference to the TensorImpl.
  // What the driver itself holds is what it held when the tensor came out of its
  // producer's post(): the reference's drivers hold a layer output through `x`
  // then, and through `pre` (with `x` overwritten) when its consumer's post() runs
  // (vgg16-cifar10.cpp:219-226) - one handle either time; a driver that keeps
  // every activation in a variable of its own holds one as well.  `copies` are the
  // handles this class and the running call have added.  For a tensor that did not
  // come out of a wrapped layer nothing is known, and the answer is "held", which
  // costs a copy, never correctness.
  bool held_for_backward(const torch::Tensor& t, size_t copies) const {
    if (producer_kept(t)) return true;
    auto h = handles_.find(t.unsafeGetTensorImpl());
    if (h == handles_.end()) return true;
    return t.use_count() - copies > h->second;
  }

  // Policy 1: nothing is copied; the storage is emptied after the consumer has
  // run and the tensor rebuilt from its producer when backward asks for it.
  void start_drop(const torch::Tensor& t) {
    auto it = producers_.find(t.unsafeGetTensorImpl());
    if (it == producers_.end()) return;
    auto s = std::make_shared<Swapped>();
    s->exe = this;
    s->storage = c10::intrusive_ptr<c10::StorageImpl>::reclaim_copy(t.storage().unsafeGetStorageImpl());
    s->nbytes = t.storage().nbytes();
    s->policy = CSW_POLICY_DROP;
    s->producer = std::move(it->second.first);
    s->producer_input = std::move(it->second.second);
    producers_.erase(it);
    s->started = true;
    by_storage_[s->storage.get()] = s;
    pending_.push_back(s);
    dropped++;
  }

  void start_swap(const torch::Tensor& t, int pol) {
    if (pol == CSW_POLICY_DROP) {
      start_drop(t);
      return;
    }
    auto s = std::make_shared<Swapped>();
    s->exe = this;
    s->storage = c10::intrusive_ptr<c10::StorageImpl>::reclaim_copy(t.storage().unsafeGetStorageImpl());
    s->nbytes = t.storage().nbytes();
    const csw_status st = csw_swap_out(mgr_, t.const_data_ptr<float>(), (size_t)t.numel(), pol,
                                       c10::cuda::getCurrentCUDAStream().stream(), &s->ticket);
    if (st == CSW_ERR_NOMEM) return;  // pools exhausted: the tensor stays on the device
    check(st, "csw_swap_out");
    s->policy = pol;
    s->started = true;
    s->order = (int)order_.size();
    order_.push_back(s);
    by_storage_[s->storage.get()] = s;
    pending_.push_back(s);
  }

  void begin_profile() {
    if (!profile) return;
    ProfEntry& e = prof_[index];
    e.start.record(c10::cuda::getCurrentCUDAStream());
  }

  // The layer has run: give the result its id, decide the deferred swaps, let
  // go of the swapped inputs' device blocks and arrange for their return before
  // the result's backward.
  void finish_layer(const torch::Tensor* const* inputs, size_t n_in, size_t call_copies, torch::Tensor& x,
                    Layer_type layer_type, bool isomit, Producer producer) {
    ids_[x.unsafeGetTensorImpl()] = index;
    handles_[x.unsafeGetTensorImpl()] = x.use_count();  // what the driver itself holds of this output
    auto fn = x.grad_fn();
    if (profile) {
      ProfEntry& e = prof_[index];
      e.end.record(c10::cuda::getCurrentCUDAStream());
      e.p.numel = (size_t)x.numel();
      e.p.omit = isomit;
      e.p.type = (int)layer_type;
      e.p.float32 = x.scalar_type() == torch::kFloat32;
      e.p.has_grad = (bool)fn;
      e.p.recomputable = (bool)producer && n_in == 1;
      if (fn) fn->add_pre_hook(std::make_unique<BackwardMark>(this, index));
      if (x.is_cuda() && e.p.float32) e.zeros = (x.detach() == 0).to(torch::kFloat64).mean();
      for (size_t i = 0; i < n_in; i++) {
        const int tid = id_of(*inputs[i]);
        e.p.inputs.push_back(tid);
        // does anything hold this consumed tensor for backward now that its consumer has run?
        if (tid >= 0 && inputs[i]->defined() && inputs[i]->is_cuda()) {
          auto pit = prof_.find(tid);
          if (pit != prof_.end()) pit->second.p.saved = held_for_backward(*inputs[i], call_copies);
        }
      }
    }
    for (auto& d : deferred_) {
      const bool view = x.storage().unsafeGetStorageImpl() == d.t.storage().unsafeGetStorageImpl();
      const bool saved = !view && held_for_backward(d.t, call_copies + 1);  // + the handle `d` holds
      if (saved && fn) start_swap(d.t, d.pol);
      else if (!saved && !view) skipped_unsaved++;
    }
    deferred_.clear();
    // remember how to rebuild x, should it be dropped when its own consumer runs
    if (producer && n_in == 1 && index < (int)policy.size() && (policy[index] == CSW_POLICY_DROP || policy_ == 4) &&
        swappable(x) && x.storage().unsafeGetStorageImpl() != inputs[0]->storage().unsafeGetStorageImpl())
      producers_[x.unsafeGetTensorImpl()] = {std::move(producer), *inputs[0]};
    for (auto& s : pending_) {
      // keep the tensor when nothing downstream will run backward through this
      // layer, or when the result is a view of it (same storage)
      if (!fn || x.storage().unsafeGetStorageImpl() == s->storage.get()) {
        s->restored = true;
        if (s->policy == CSW_POLICY_DROP) dropped--;
        continue;
      }
      // detach the device block from the storage; a swapped block is freed once the
      // manager's streams are done with it, a dropped one at once
      s->reading = s->storage->set_data_ptr(at::DataPtr(nullptr, s->storage->device()));
      if (s->policy == CSW_POLICY_DROP) {
        s->reading.clear();
      } else if (free_after_codec && (s->policy == CSW_POLICY_ZFP || s->policy == CSW_POLICY_SPARSE)) {
        // the codec reads the tensor in a fraction of the time the link needs for it: let the
        // compute stream wait for that read and give the block back at once, as a free in
        // stream order - the memory is reusable by the very next layer however far the host
        // runs ahead of the GPU, instead of whenever a poll finds the read finished
        check(csw_swap_out_wait(mgr_, s->ticket, c10::cuda::getCurrentCUDAStream().stream()), "csw_swap_out_wait");
        s->reading.clear();
      } else {
        reading_.push_back(s);
      }
      fn->add_pre_hook(std::make_unique<RestoreHook>(s));
    }
    pending_.clear();
    poll();
  }

  void restore(Swapped& s) {
    if (s.policy == CSW_POLICY_DROP) {
      rebuild(s);
      return;
    }
    // A losslessly swapped tensor that is needed again before the manager has
    // finished reading it never left the device: hand the block back as it is.
    // (A lossy one must come back as the decoded values whatever the timing.)
    if (s.reading.get() != nullptr && (s.policy == CSW_POLICY_RAW || s.policy == CSW_POLICY_SPARSE)) {
      int done = 1;
      csw_swap_out_done(mgr_, s.ticket, &done);
      if (!done) {
        s.storage->set_data_ptr_noswap(std::move(s.reading));
        s.reading.clear();  // a moved-from DataPtr keeps its raw pointer: make "no block held" visible
        settle(s);
        reclaimed++;
        poll();
        return;
      }
    }
    auto* alloc = c10::cuda::CUDACachingAllocator::get();
    const cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
    if (s.ahead.get() != nullptr) {
      // copy and decode were started when the tensor swapped out after this one came back
      check(csw_swap_in_wait(mgr_, s.ticket, stream), "csw_swap_in_wait");
      s.storage->set_data_ptr_noswap(std::move(s.ahead));
      s.ahead.clear();
    } else {
      at::DataPtr dp = alloc->allocate(s.nbytes);
      check(csw_swap_in(mgr_, s.ticket, static_cast<float*>(dp.get()), stream), "csw_swap_in");
      s.storage->set_data_ptr_noswap(std::move(dp));
    }
    const int order = s.order;
    settle(s);
    // Ahead of need: start bringing back - copy AND decode, into blocks taken now - the
    // `lookahead` tensors swapped out just before this one, so that their consumers'
    // backward finds them ready instead of waiting for a decode that starts only when
    // it asks.
    int started = 0;
    for (int i = order - 1; i >= 0 && started < lookahead; i--) {
      auto p = order_[i].lock();
      if (p && !p->restored && p->ticket) {
        started++;
        if (p->ahead.get() != nullptr) continue;  // already on its way
        int done = 1;
        // a lossless ticket still on its way out may yet be taken back whole
        if (p->policy != CSW_POLICY_ZFP) csw_swap_out_done(mgr_, p->ticket, &done);
        if (done) {
          p->ahead = alloc->allocate(p->nbytes);
          check(csw_swap_in_start(mgr_, p->ticket, static_cast<float*>(p->ahead.get()), stream), "csw_swap_in_start");
        }
      }
    }
    poll();
  }

  // Policy 1: run the producer again on its own input (swapped in or rebuilt
  // first if that is gone too) and give the result's block to the storage.
  void rebuild(Swapped& s) {
    auto* in_storage = s.producer_input.storage().unsafeGetStorageImpl();
    if (in_storage->data() == nullptr) {
      auto it = by_storage_.find(in_storage);
      std::shared_ptr<Swapped> in = it == by_storage_.end() ? nullptr : it->second.lock();
      if (!in) throw std::runtime_error("cswap: the input of a dropped tensor's producer is gone");
      if (!in->restored) restore(*in);
    }
    torch::Tensor out;
    {
      torch::NoGradGuard ng;
      out = s.producer(s.producer_input).contiguous();
    }
    if (out.storage().nbytes() != s.nbytes || out.storage_offset() != 0)
      throw std::runtime_error("cswap: recomputed activation does not match the dropped one");
    auto* os = out.storage().unsafeGetStorageImpl();
    s.storage->set_data_ptr_noswap(os->set_data_ptr(at::DataPtr(nullptr, os->device())));
    settle(s);
    recomputed++;
  }

  // The tensor is back.  The restore hooks keep this record alive until the
  // graph is destroyed, so everything it holds is let go here: with its own
  // reference to the storage gone, the block is freed as soon as the backward
  // nodes that saved the tensor have run; the ticket's host memory returns to the
  // pool once its copy has finished (csw_ticket_release never blocks).
  void settle(Swapped& s) {
    s.restored = true;
    s.storage.reset();
    if (s.reading.get() == nullptr) release_ticket(s);  // else poll() does, once the block has been read
    s.producer = nullptr;
    s.producer_input = torch::Tensor();
  }

  // free device blocks whose swap-out has finished reading them (never blocks)
  // An event query costs more than a microsecond of host time and this runs in every pre(),
  // post() and restore: raw tensors are read by one of the manager's streams and compressed
  // ones by another, each in the order the swaps were started, so within a kind nothing has
  // finished behind the first entry that has not.
  void poll() {
    size_t k = 0;
    bool busy[2] = {false, false};
    for (auto& s : reading_) {
      if (s->reading.get() == nullptr) continue;  // taken back: the storage owns the block again
      const int kind = s->policy == CSW_POLICY_RAW ? 0 : 1;
      int done = busy[kind] ? 0 : 1;
      if (!busy[kind] && s->ticket) csw_swap_out_done(mgr_, s->ticket, &done);
      if (done) {
        s->reading.clear();
        if (s->restored) release_ticket(*s);
      } else {
        busy[kind] = true;
        reading_[k++] = s;
      }
    }
    reading_.resize(k);
  }
  void release_ticket(Swapped& s) {
    if (s.ticket) csw_ticket_release(mgr_, s.ticket);
    s.ticket = nullptr;
  }
  void drain() {
    for (auto& s : reading_)
      if (s->ticket) csw_swap_out_sync(mgr_, s->ticket);
    reading_.clear();
    pending_.clear();
    deferred_.clear();
    order_.clear();
    by_storage_.clear();
    producers_.clear();
  }

  csw_mgr* mgr_ = nullptr;
  unsigned maxbits_ = 512;
  bool fitted_ = false;
  csw_cost_model cost_{};
  std::unordered_map<const c10::TensorImpl*, int> ids_;
  std::unordered_map<const c10::TensorImpl*, std::pair<Producer, torch::Tensor>> producers_;
  std::unordered_map<const c10::StorageImpl*, std::weak_ptr<Swapped>> by_storage_;
  std::vector<std::shared_ptr<Swapped>> pending_;  // swap-outs started by the current pre()
  std::vector<Deferred> deferred_;                 // swaps waiting for their consumer to have run
  std::unordered_map<const c10::TensorImpl*, size_t> handles_;  // driver handles per wrapped layer output
  std::vector<std::shared_ptr<Swapped>> reading_;  // device blocks still being read
  std::vector<std::weak_ptr<Swapped>> order_;      // this step's swap-outs, in order
  std::map<int, ProfEntry> prof_;
};

}  // namespace cswap
