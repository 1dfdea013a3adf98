// Execution - the reference's swap orchestrator (CSWAP+/Execution.h:38-447) on
// stock libtorch, over the C ABI of libcswap_b200.so.
//
// Same surface as the reference class: init_, preforward, pre, post,
// postforward, the public tables policy / begin_stage / types, index and
// policy_, the Layer_type enum (Execution.h:28-35) and the policy codes
// 0 keep, 2 raw, 3 sparse, 6 ZFP.  A driver wraps each layer exactly as the
// reference's drivers do (vgg16-cifar10.cpp:219-226):
//
//     exe.pre(pre);  x = layer(pre);  exe.post(pre, x);  pre = x;
//
// What is different underneath:
//  * the fork-only members the reference writes (Tensor::tensor_id,
//    Node::com_and_tran / storage_impl_ / pre_node ...) do not exist upstream;
//    tensor ids are kept in a side table keyed by the tensor's TensorImpl and
//    the swap-in runs from a FunctionPreHook on the consumer's grad_fn, which
//    autograd always runs before the producer's own backward;
//  * swap-out and swap-in go through csw_swap_out / csw_swap_in: events between
//    streams, pooled pinned memory, no stream synchronisation, no blocking read
//    of the sparse count (Execution.h:77,92,236);
//  * a tensor's device block is handed back to the caching allocator only once
//    the manager's streams have finished reading it (polled, never waited for).
//
// Constraints inherited from the reference's scheme: begin_stage[id] must be the
// LAST forward use of tensor id (its storage is empty afterwards until backward
// restores it), and only whole, contiguous float32 CUDA storages are swapped.
// Policy 1 (drop and recompute) is not implemented: such tensors are kept.
#pragma once
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/autograd/function.h>
#include <torch/csrc/autograd/function_hook.h>
#include <torch/torch.h>

#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "cswap_b200.h"

namespace cswap {

enum Layer_type { CONV, POOL, ACT, BN, FC, MASKFILL };

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
  }
  void setRatio(unsigned maxbits) { check(csw_mgr_set_zfp_maxbits(mgr_, maxbits), "csw_mgr_set_zfp_maxbits"); }

  // Execution.h:403-412
  void preforward() {
    index = -1;
    ids_.clear();
    pending_.clear();
    order_.clear();
    poll();
  }
  void postforward() { poll(); }

  // Execution.h:65-133
  void pre(torch::Tensor& t, Layer_type layer_type = ACT) {
    index++;
    maybe_swap_out(t, layer_type);
  }
  // Execution.h:135-212
  void pre(std::vector<torch::Tensor> inputs, Layer_type layer_type = ACT) {
    index++;
    for (auto& t : inputs) maybe_swap_out(t, layer_type);
  }
  // Execution.h:217-310
  void post(torch::Tensor& pre_t, torch::Tensor& x, Layer_type = ACT, bool = false) {
    (void)pre_t;
    finish_layer(x);
  }
  // Execution.h:311-401
  void post(std::vector<torch::Tensor> inputs, torch::Tensor& x, Layer_type = ACT, bool = false) {
    (void)inputs;
    finish_layer(x);
  }

  csw_mgr* manager() const { return mgr_; }
  csw_mgr_stats stats() const {
    csw_mgr_stats s{};
    csw_mgr_get_stats(mgr_, &s);
    return s;
  }

  int index = -1;
  long reclaimed = 0;  // tensors taken back before they had left the device
  std::vector<int> policy;
  std::vector<int> begin_stage;
  std::vector<Layer_type> types;
  int policy_ = 1;  // 1 CSWAP, 2 Capuchin, 3 vDNN, 4 SuperNeurons (Execution.h:420)

 private:
  // One swapped-out storage, shared between the table below and the backward hook.
  struct Swapped {
    Execution* exe = nullptr;
    c10::intrusive_ptr<c10::StorageImpl> storage;
    csw_ticket* ticket = nullptr;
    size_t nbytes = 0;
    int order = -1;         // position among this step's swap-outs
    int policy = 0;
    bool restored = false;
    at::DataPtr reading;    // the device block while the manager still reads it
    ~Swapped() {
      if (ticket && exe && exe->mgr_) csw_ticket_release(exe->mgr_, ticket);
    }
  };

  struct RestoreHook : torch::autograd::FunctionPreHook {
    std::shared_ptr<Swapped> s;
    explicit RestoreHook(std::shared_ptr<Swapped> sw) : s(std::move(sw)) {}
    torch::autograd::variable_list operator()(const torch::autograd::variable_list& grads) override {
      if (!s->restored) s->exe->restore(*s);
      return grads;
    }
  };

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

  void maybe_swap_out(torch::Tensor& t, Layer_type layer_type) {
    const int id = id_of(t);
    if (id < 0 || id >= (int)begin_stage.size() || index != begin_stage[id] || !t.grad_fn()) return;
    int pol = policy[id];
    if (layer_type == CONV && policy_ > 2) pol = CSW_POLICY_RAW;  // vDNN / SuperNeurons baselines (Execution.h:70)
    if ((pol != CSW_POLICY_RAW && pol != CSW_POLICY_SPARSE && pol != CSW_POLICY_ZFP) || !swappable(t)) return;
    auto s = std::make_shared<Swapped>();
    s->exe = this;
    s->storage = c10::intrusive_ptr<c10::StorageImpl>::reclaim_copy(t.storage().unsafeGetStorageImpl());
    s->nbytes = t.storage().nbytes();
    const csw_status st = csw_swap_out(mgr_, t.const_data_ptr<float>(), (size_t)t.numel(), pol,
                                       c10::cuda::getCurrentCUDAStream().stream(), &s->ticket);
    if (st == CSW_ERR_NOMEM) return;  // pools exhausted: the tensor stays on the device
    check(st, "csw_swap_out");
    s->policy = pol;
    s->order = (int)order_.size();
    order_.push_back(s);
    pending_.push_back(s);
  }

  // The layer has run: give the result its id, let go of the swapped inputs'
  // device blocks and arrange for their return before the result's backward.
  void finish_layer(torch::Tensor& x) {
    ids_[x.unsafeGetTensorImpl()] = index;
    auto fn = x.grad_fn();
    for (auto& s : pending_) {
      // keep the tensor when nothing downstream will run backward through this
      // layer, or when the result is a view of it (same storage)
      if (!fn || x.storage().unsafeGetStorageImpl() == s->storage.get()) {
        s->restored = true;
        continue;
      }
      // detach the device block from the storage; it is freed once the manager's streams are done with it
      s->reading = s->storage->set_data_ptr(at::DataPtr(nullptr, s->storage->device()));
      reading_.push_back(s);
      fn->add_pre_hook(std::make_unique<RestoreHook>(s));
    }
    pending_.clear();
    poll();
  }

  void restore(Swapped& s) {
    // A losslessly swapped tensor that is needed again before the manager has
    // finished reading it never left the device: hand the block back as it is.
    // (A lossy one must come back as the decoded values whatever the timing.)
    if (s.reading.get() != nullptr && (s.policy == CSW_POLICY_RAW || s.policy == CSW_POLICY_SPARSE)) {
      int done = 1;
      csw_swap_out_done(mgr_, s.ticket, &done);
      if (!done) {
        s.storage->set_data_ptr_noswap(std::move(s.reading));
        s.restored = true;
        reclaimed++;
        poll();
        return;
      }
    }
    auto* alloc = c10::cuda::CUDACachingAllocator::get();
    at::DataPtr dp = alloc->allocate(s.nbytes);
    check(csw_swap_in(mgr_, s.ticket, static_cast<float*>(dp.get()), c10::cuda::getCurrentCUDAStream().stream()),
          "csw_swap_in");
    s.storage->set_data_ptr_noswap(std::move(dp));
    s.restored = true;
    // one step ahead: start bringing back the tensor swapped out just before this one
    for (int i = s.order - 1; i >= 0; i--) {
      auto p = order_[i].lock();
      if (p && !p->restored && p->ticket) {
        csw_prefetch(mgr_, p->ticket);
        break;
      }
    }
    poll();
  }

  // free device blocks whose swap-out has finished reading them (never blocks)
  void poll() {
    size_t k = 0;
    for (auto& s : reading_) {
      int done = 1;
      if (s->restored && s->reading.get() == nullptr) continue;  // taken back: the storage owns the block again
      if (s->ticket) csw_swap_out_done(mgr_, s->ticket, &done);
      if (done) s->reading.clear();
      else reading_[k++] = s;
    }
    reading_.resize(k);
  }
  void drain() {
    for (auto& s : reading_)
      if (s->ticket) csw_swap_out_sync(mgr_, s->ticket);
    reading_.clear();
    pending_.clear();
    order_.clear();
  }

  csw_mgr* mgr_ = nullptr;
  std::unordered_map<const c10::TensorImpl*, int> ids_;
  std::vector<std::shared_ptr<Swapped>> pending_;  // swap-outs started by the current pre()
  std::vector<std::shared_ptr<Swapped>> reading_;  // device blocks still being read
  std::vector<std::weak_ptr<Swapped>> order_;      // this step's swap-outs, in order
};

}  // namespace cswap
