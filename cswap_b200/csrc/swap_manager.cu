// Swap manager: pinned host pool, device staging pool, dedicated codec / D2H /
// H2D streams, event-ordered swap-out and swap-in of one tensor at a time.
//
// Replaces the device/host mechanics of Execution::pre/post
// (CSWAP+/Execution.h:65-133,217-310) and the swap-in half that lives in the
// reference's modified autograd engine.  Differences that matter:
//  * ordering is by events between streams; the host never waits for the
//    device on the swap-out path (the reference synchronises the compute stream
//    in every pre() and post(), Execution.h:77,236, and blocks on a 4-byte copy
//    to size the sparse output, Execution.h:92);
//  * host and staging memory come from pools created once (the reference takes
//    a pinned allocation per tensor per step, Execution.h:76,97-99,114);
//  * the sparse payload, whose size is only known on the device, is moved by a
//    small copy kernel that reads the count itself and writes exactly
//    `header + 4 * nnz` bytes into mapped pinned memory.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <vector>

#include "../../include/cswap_b200.h"
#include "internal.h"
#include "sparse_kernels.h"

namespace csw {
namespace {

// ---- first-fit pool over one slab -----------------------------------------------
class Pool {
 public:
  static constexpr size_t kAlign = 512;
  void init(char* base, size_t cap) {
    base_ = base;
    cap_ = cap;
    free_.clear();
    if (cap) free_[0] = cap;
    used_ = high_ = 0;
  }
  char* base() const { return base_; }
  size_t in_use() const { return used_; }
  size_t high_water() const { return high_; }
  // returns nullptr when no free range is large enough
  void* alloc(size_t bytes, size_t* got) {
    bytes = round_up(bytes ? bytes : 1);
    for (auto it = free_.begin(); it != free_.end(); ++it) {
      if (it->second >= bytes) {
        const size_t off = it->first, len = it->second;
        free_.erase(it);
        if (len > bytes) free_[off + bytes] = len - bytes;
        used_ += bytes;
        if (used_ > high_) high_ = used_;
        *got = bytes;
        return base_ + off;
      }
    }
    return nullptr;
  }
  void release(void* p, size_t bytes) {
    if (!p) return;
    size_t off = (size_t)((char*)p - base_);
    used_ -= bytes;
    auto next = free_.lower_bound(off);
    if (next != free_.begin()) {
      auto prev = std::prev(next);
      if (prev->first + prev->second == off) {
        off = prev->first;
        bytes += prev->second;
        free_.erase(prev);
      }
    }
    if (next != free_.end() && off + bytes == next->first) {
      bytes += next->second;
      free_.erase(next);
    }
    free_[off] = bytes;
  }
  // give back the tail of a block, keeping the first `keep` bytes
  size_t shrink(void* p, size_t have, size_t keep) {
    keep = round_up(keep ? keep : 1);
    if (keep >= have) return have;
    release((char*)p + keep, have - keep);
    return keep;
  }

 private:
  static size_t round_up(size_t b) { return (b + kAlign - 1) / kAlign * kAlign; }
  char* base_ = nullptr;
  size_t cap_ = 0, used_ = 0, high_ = 0;
  std::map<size_t, size_t> free_;  // offset -> length
};

// Copies `fixed + 4 * (*nnz)` bytes (rounded up to 16) from device staging to
// mapped pinned host memory and publishes the count next to it.
__global__ void __launch_bounds__(256)
sparse_to_host_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const uint32_t* __restrict__ nnz_dev,
                      uint32_t* __restrict__ nnz_host, size_t fixed_bytes) {
  const uint32_t nnz = *nnz_dev;
  const size_t chunks = (fixed_bytes + 4 * (size_t)nnz + 15) / 16;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = src[i];
  if (blockIdx.x == 0 && threadIdx.x == 0) *nnz_host = nnz;
}

enum TicketState { T_OUT = 0, T_HOST = 1, T_IN = 2, T_DEAD = 3 };

}  // namespace
}  // namespace csw

using namespace csw;

struct csw_ticket {
  int policy = CSW_POLICY_RAW;
  size_t numel = 0;
  unsigned maxbits = 0;
  int state = T_OUT;
  // host copy
  void* host = nullptr;
  size_t host_cap = 0;
  size_t moved = 0;       // bytes on the link (final once moved_final)
  bool moved_final = false;
  // device staging (compressed form), present while a copy or codec uses it
  void* stage = nullptr;
  size_t stage_cap = 0;
  bool stage_loaded = false;  // prefetch already brought the payload back
  bool in_live = false;       // listed in the manager's housekeeping list
  bool cached = false;        // host copy complete, staged payload kept while the pool has room
  bool queued = false;        // raw: the copy out has not been handed to the copy stream yet
  const float* src = nullptr; // raw: the tensor to copy while queued
  cudaEvent_t ev_ready = nullptr;  // raw, while queued: the producer's work on the caller's stream
  uint32_t* nnz_host = nullptr;  // slot in the manager's mapped count array
  int nnz_slot = -1;
  cudaEvent_t ev_read = nullptr;   // source tensor no longer read
  cudaEvent_t ev_d2h = nullptr;    // host copy complete
  cudaEvent_t ev_h2d = nullptr;    // payload back on the device
  cudaEvent_t ev_done = nullptr;   // swap-in result ready
};

struct csw_mgr {
  int device = 0;
  unsigned maxbits = 512;
  cudaStream_t s_codec = nullptr, s_d2h = nullptr, s_h2d = nullptr;
  // Raw tensors and compressed payloads leave through the ONE copy stream s_d2h.  Giving the
  // payloads a stream of their own looked attractive (a small payload need not queue behind
  // large raw copies) and measured badly: with two raw 48 MiB tensors among 119 compressed
  // ones a BERT-shaped step took 288 ms instead of 236 - two outgoing copy streams at once
  // slow the link down for both.  The copy engine serves device-to-host copies strictly in
  // the order they were submitted, across streams and whatever their priorities or sizes
  // (measured: a 4-byte read-back on another stream returns only when 4 GiB queued before it
  // have left, 75 ms, also with the queue cut into 16 MiB pieces on a lowest-priority stream):
  // a caller that reads a result back every step waits for the swap traffic queued so far.
  char* pinned_base = nullptr;
  char* staging_base = nullptr;
  Pool pinned, staging;
  uint32_t* nnz_slots = nullptr;      // mapped pinned
  uint32_t* nnz_dev = nullptr;        // device copies of the counts
  std::vector<int> free_slots;
  std::vector<cudaEvent_t> free_events;
  std::vector<csw_ticket*> live;      // tickets whose staging may be reclaimable
  std::vector<csw_ticket*> zombies;   // released tickets whose copies are still in flight
  std::vector<csw_ticket*> cache;     // tickets whose payload is on the host AND still staged, oldest first
  bool keep_staged = true;
  // Raw copies out are handed to the copy stream a few at a time (see submit_raw): the rest
  // wait here, in order, and a ticket released while it waits is never copied at all.
  std::vector<csw_ticket*> raw_queue;
  std::vector<csw_ticket*> raw_flying;  // handed over, copy not yet known to be finished
  std::vector<csw_ticket*> all;       // every ticket not yet destroyed (so that destroy can free what callers kept)
  csw_mgr_stats stats{};
  std::mutex mu;
};

namespace {
constexpr int kCountSlots = 4096;

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

cudaError_t get_event(csw_mgr* m, cudaEvent_t* ev) {
  if (!m->free_events.empty()) {
    *ev = m->free_events.back();
    m->free_events.pop_back();
    return cudaSuccess;
  }
  return cudaEventCreateWithFlags(ev, cudaEventDisableTiming);
}
void put_event(csw_mgr* m, cudaEvent_t& ev) {
  if (ev) m->free_events.push_back(ev);
  ev = nullptr;
}

void uncache(csw_mgr* m, csw_ticket* t) {
  if (!t->cached) return;
  for (size_t i = 0; i < m->cache.size(); i++)
    if (m->cache[i] == t) {
      m->cache.erase(m->cache.begin() + i);
      break;
    }
  t->cached = false;
}

void free_stage(csw_mgr* m, csw_ticket* t) {
  uncache(m, t);
  if (t->stage) {
    m->staging.release(t->stage, t->stage_cap);
    t->stage = nullptr;
    t->stage_cap = 0;
    t->stage_loaded = false;
  }
}

// Learn the final size of a sparse payload once its copy kernel has run, and
// return the unused tail of its pinned block.
void finalize_moved(csw_mgr* m, csw_ticket* t) {
  if (t->moved_final) return;
  csw_sparse_layout L;
  csw_sparse_layout_of(t->numel, &L);
  t->moved = L.values + 4 * (size_t)(*t->nnz_host);
  t->moved_final = true;
  t->host_cap = m->pinned.shrink(t->host, t->host_cap, t->moved);
  m->stats.moved_bytes_out += t->moved;
}

bool event_done(cudaEvent_t ev) { return !ev || cudaEventQuery(ev) == cudaSuccess; }

// Return everything a released ticket holds to the pools and free it.
void forget_raw(csw_mgr* m, csw_ticket* t);
void pump_raw(csw_mgr* m);
void submit_raw_through(csw_mgr* m, csw_ticket* t);
void destroy_ticket(csw_mgr* m, csw_ticket* t) {
  forget_raw(m, t);
  free_stage(m, t);
  if (t->host) m->pinned.release(t->host, t->host_cap);
  if (t->nnz_slot >= 0) m->free_slots.push_back(t->nnz_slot);
  put_event(m, t->ev_read);
  put_event(m, t->ev_d2h);
  put_event(m, t->ev_h2d);
  put_event(m, t->ev_done);
  for (size_t i = 0; i < m->all.size(); i++)
    if (m->all[i] == t) {
      m->all[i] = m->all.back();
      m->all.pop_back();
      break;
    }
  delete t;
}

// Non-blocking housekeeping: release staging whose last user has finished.
// An event query costs more than a microsecond of host time, and this runs
// inside every call, so it asks as few as the stream order allows.
void poll(csw_mgr* m) {
  // released tickets with work in flight, oldest first: stop at the first that is not
  // finished (those behind it were released later and give their memory back a call or two
  // later; a caller that needs memory now waits for the front, see pool_alloc)
  size_t z = 0;
  while (z < m->zombies.size()) {
    csw_ticket* t = m->zombies[z];
    if (!(event_done(t->ev_done) && event_done(t->ev_h2d) && event_done(t->ev_d2h))) break;
    destroy_ticket(m, t);
    z++;
  }
  if (z) m->zombies.erase(m->zombies.begin(), m->zombies.begin() + z);
  size_t k = 0;
  // `live` is in submission order; copies out go down one stream, raw copies in down a
  // second and decodes down a third, so within a kind none has finished behind the first
  // unfinished one - on the way out and on the way back alike
  bool out_busy[2] = {false, false}, in_busy[2] = {false, false};
  for (size_t i = 0; i < m->live.size(); i++) {
    csw_ticket* t = m->live[i];
    const int kind = t->policy == CSW_POLICY_RAW ? 0 : 1;
    bool keep = true;
    if (t->state == T_OUT) {
      if (!out_busy[kind] && !t->queued && cudaEventQuery(t->ev_d2h) == cudaSuccess) {
        if (t->policy == CSW_POLICY_SPARSE) finalize_moved(m, t);
        // The payload is on the host now.  Its staged copy stays where it is until the pool
        // needs the room (pool_alloc evicts the oldest first): backward asks for the tensors
        // swapped out last first, and those then come back without crossing the link again.
        if (t->stage && m->keep_staged) {
          t->cached = true;
          m->cache.push_back(t);
        } else {
          free_stage(m, t);
        }
        t->state = T_HOST;
        keep = false;
      } else {
        out_busy[kind] = true;
      }
    } else if (t->state == T_IN && t->ev_done) {
      // the staged payload may still be on its way out when its decode has finished
      if (!in_busy[kind] && cudaEventQuery(t->ev_done) == cudaSuccess && event_done(t->ev_d2h)) {
        if (t->policy == CSW_POLICY_SPARSE && !t->moved_final) finalize_moved(m, t);
        free_stage(m, t);
        t->state = T_HOST;
        keep = false;
      } else {
        in_busy[kind] = true;
      }
    } else if (t->state == T_HOST || t->state == T_DEAD) {
      keep = false;
    }
    if (keep) m->live[k++] = t;
    else t->in_live = false;
  }
  cudaGetLastError();  // cudaErrorNotReady from the queries is not an error
  m->live.resize(k);
  pump_raw(m);
}

void drop_from_live(csw_mgr* m, csw_ticket* t) {
  if (!t->in_live) return;
  for (size_t i = 0; i < m->live.size(); i++)
    if (m->live[i] == t) {
      m->live.erase(m->live.begin() + i);
      break;
    }
  t->in_live = false;
}

// ---- raw copies out, a few at a time ------------------------------------------------
// The copy engine serves device-to-host copies strictly in the order they were
// submitted, so whatever is queued on it stands between the caller and its next
// read-back; and a raw tensor that backward wants before its copy has run is
// handed back as it is, which makes that copy wasted link time.  So at most
// kRawInFlight raw copies are on the copy stream at a time; the others wait in
// raw_queue and are submitted as those finish (every call pumps), or when a call
// needs one of them to have happened.
constexpr size_t kRawInFlight = 2;

cudaError_t submit_raw(csw_mgr* m, csw_ticket* t) {
  cudaError_t e = cudaStreamWaitEvent(m->s_d2h, t->ev_ready, 0);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(t->host, t->src, t->numel * sizeof(float), cudaMemcpyDeviceToHost, m->s_d2h);
  if (e == cudaSuccess) e = cudaEventRecord(t->ev_read, m->s_d2h);
  if (e == cudaSuccess) e = cudaEventRecord(t->ev_d2h, m->s_d2h);
  put_event(m, t->ev_ready);
  t->queued = false;
  t->src = nullptr;
  m->stats.moved_bytes_out += t->moved;
  m->raw_flying.push_back(t);
  return e;
}

void pump_raw(csw_mgr* m) {
  size_t done = 0;  // in order on one stream: nothing has finished behind the first that has not
  while (done < m->raw_flying.size() && cudaEventQuery(m->raw_flying[done]->ev_d2h) == cudaSuccess) done++;
  if (done) m->raw_flying.erase(m->raw_flying.begin(), m->raw_flying.begin() + done);
  cudaGetLastError();
  size_t n = 0;
  while (n < m->raw_queue.size() && m->raw_flying.size() < kRawInFlight) submit_raw(m, m->raw_queue[n++]);
  if (n) m->raw_queue.erase(m->raw_queue.begin(), m->raw_queue.begin() + n);
}

// A call needs this ticket's copy to have been issued: issue it and everything queued before it.
void submit_raw_through(csw_mgr* m, csw_ticket* t) {
  if (!t->queued) return;
  size_t n = 0;
  while (n < m->raw_queue.size()) {
    csw_ticket* q = m->raw_queue[n++];
    submit_raw(m, q);
    if (q == t) break;
  }
  m->raw_queue.erase(m->raw_queue.begin(), m->raw_queue.begin() + n);
}

void forget_raw(csw_mgr* m, csw_ticket* t) {  // the ticket is going away
  for (size_t i = 0; i < m->raw_queue.size(); i++)
    if (m->raw_queue[i] == t) {
      m->raw_queue.erase(m->raw_queue.begin() + i);
      break;
    }
  for (size_t i = 0; i < m->raw_flying.size(); i++)
    if (m->raw_flying[i] == t) {
      m->raw_flying.erase(m->raw_flying.begin() + i);
      break;
    }
  if (t->queued) {
    put_event(m, t->ev_ready);
    t->queued = false;
    t->src = nullptr;
  }
}

// Pool allocation that first reclaims finished work and, if still short, waits
// for the oldest outstanding transfers.
void* pool_alloc(csw_mgr* m, Pool& pool, size_t bytes, size_t* got) {
  void* p = pool.alloc(bytes, got);
  if (p) return p;
  poll(m);
  p = pool.alloc(bytes, got);
  // staged payloads that are kept only because there was room: oldest out first
  while (!p && &pool == &m->staging && !m->cache.empty()) {
    free_stage(m, m->cache.front());
    p = pool.alloc(bytes, got);
  }
  while (!p && (!m->live.empty() || !m->zombies.empty())) {
    csw_ticket* t = !m->zombies.empty() ? m->zombies.front() : m->live.front();
    submit_raw_through(m, t);
    cudaEvent_t ev = t->state == T_OUT ? t->ev_d2h : (t->ev_done ? t->ev_done : t->ev_d2h);
    if (ev) cudaEventSynchronize(ev);
    if ((t->state == T_DEAD || t->state == T_IN) && t->ev_d2h) cudaEventSynchronize(t->ev_d2h);
    if (t->state == T_DEAD && t->ev_h2d) cudaEventSynchronize(t->ev_h2d);
    const size_t before = m->live.size() + m->zombies.size();
    poll(m);
    p = pool.alloc(bytes, got);
    while (!p && &pool == &m->staging && !m->cache.empty()) {  // what the poll has just moved into the cache
      free_stage(m, m->cache.front());
      p = pool.alloc(bytes, got);
    }
    if (!p && m->live.size() + m->zombies.size() == before) break;
  }
  return p;
}

// A tensor under policy 6 travels as the ZFP stream of its first nz 32x32
// slabs followed by the numel % 1024 values that do not fill a slab, as they
// are.  `bytes` is the whole payload, `zbytes` the stream alone.
csw_status zfp_geometry(size_t numel, unsigned maxbits, size_t* nz, size_t* zbytes, size_t* bytes) {
  *nz = numel / 1024;
  if (*nz == 0) return CSW_ERR_UNSUPPORTED;  // less than one slab: not worth a codec launch
  csw_status st = csw_zfp_max_bytes(32, 32, *nz, maxbits, zbytes);
  if (st != CSW_OK) return st;
  *bytes = *zbytes + (numel % 1024) * sizeof(float);
  return CSW_OK;
}

}  // namespace

extern "C" {

csw_status csw_mgr_create(const csw_mgr_config* cfg, csw_mgr** out) {
  if (!cfg || !out) return CSW_ERR_ARG;
  DeviceGuard g(cfg->device);
  if (!g.ok) return CSW_ERR_ARG;
  csw_mgr* m = new (std::nothrow) csw_mgr;
  if (!m) return CSW_ERR_NOMEM;
  m->device = cfg->device;
  m->maxbits = cfg->zfp_maxbits ? cfg->zfp_maxbits : 512;
  const size_t pinned = cfg->pinned_bytes ? cfg->pinned_bytes : ((size_t)1 << 30);
  const size_t staging = cfg->staging_bytes ? cfg->staging_bytes : ((size_t)512 << 20);
  cudaError_t e = cudaSuccess;
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&m->s_codec, cudaStreamNonBlocking, hi);
  if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&m->s_d2h, cudaStreamNonBlocking, hi);
  if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&m->s_h2d, cudaStreamNonBlocking, hi);
  if (e == cudaSuccess) e = cudaHostAlloc((void**)&m->pinned_base, pinned, cudaHostAllocPortable | cudaHostAllocMapped);
  if (e == cudaSuccess) e = cudaMalloc((void**)&m->staging_base, staging);
  if (e == cudaSuccess)
    e = cudaHostAlloc((void**)&m->nnz_slots, kCountSlots * sizeof(uint32_t), cudaHostAllocPortable | cudaHostAllocMapped);
  if (e == cudaSuccess) e = cudaMalloc((void**)&m->nnz_dev, kCountSlots * sizeof(uint32_t));
  if (e != cudaSuccess) {
    csw_status st = cuda_fail(e);
    csw_mgr_destroy(m);
    return st;
  }
  m->pinned.init(m->pinned_base, pinned);
  m->staging.init(m->staging_base, staging);
  for (int i = kCountSlots - 1; i >= 0; i--) m->free_slots.push_back(i);
  *out = m;
  return CSW_OK;
}

csw_status csw_mgr_destroy(csw_mgr* m) {
  if (!m) return CSW_ERR_ARG;
  DeviceGuard g(m->device);
  if (m->s_codec) cudaStreamSynchronize(m->s_codec);
  if (m->s_d2h) cudaStreamSynchronize(m->s_d2h);
  if (m->s_h2d) cudaStreamSynchronize(m->s_h2d);
  // every ticket still alive, released or not: the streams are idle now, so all of it can go
  // (handles the caller still holds are invalid once the manager is gone)
  while (!m->all.empty()) destroy_ticket(m, m->all.back());
  m->zombies.clear();
  m->live.clear();
  for (cudaEvent_t ev : m->free_events) cudaEventDestroy(ev);
  if (m->s_codec) cudaStreamDestroy(m->s_codec);
  if (m->s_d2h) cudaStreamDestroy(m->s_d2h);
  if (m->s_h2d) cudaStreamDestroy(m->s_h2d);
  if (m->pinned_base) cudaFreeHost(m->pinned_base);
  if (m->staging_base) cudaFree(m->staging_base);
  if (m->nnz_slots) cudaFreeHost(m->nnz_slots);
  if (m->nnz_dev) cudaFree(m->nnz_dev);
  delete m;
  return CSW_OK;
}

csw_status csw_mgr_set_zfp_maxbits(csw_mgr* m, unsigned maxbits) {
  if (!m) return CSW_ERR_ARG;
  size_t b;
  if (csw_zfp_max_bytes(32, 32, 4, maxbits, &b) != CSW_OK) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  m->maxbits = maxbits;
  return CSW_OK;
}

csw_status csw_mgr_keep_staged(csw_mgr* m, int keep) {
  if (!m) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  m->keep_staged = keep != 0;
  if (!m->keep_staged)
    while (!m->cache.empty()) free_stage(m, m->cache.front());
  return CSW_OK;
}

csw_status csw_mgr_get_streams(csw_mgr* m, csw_stream_t* codec, csw_stream_t* d2h, csw_stream_t* h2d) {
  if (!m) return CSW_ERR_ARG;
  if (codec) *codec = m->s_codec;
  if (d2h) *d2h = m->s_d2h;
  if (h2d) *h2d = m->s_h2d;
  return CSW_OK;
}

csw_status csw_swap_out(csw_mgr* m, const float* d_ptr, size_t numel, int policy, csw_stream_t compute,
                        csw_ticket** ticket) {
  if (!m || !d_ptr || !numel || !ticket) return CSW_ERR_ARG;
  if (policy != CSW_POLICY_RAW && policy != CSW_POLICY_SPARSE && policy != CSW_POLICY_ZFP) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (!g.ok) return CSW_ERR_ARG;
  poll(m);

  size_t nz = 0, zstream = 0, zbytes = 0;  // slabs, stream bytes, stream + raw tail
  if (policy == CSW_POLICY_ZFP && zfp_geometry(numel, m->maxbits, &nz, &zstream, &zbytes) != CSW_OK)
    policy = CSW_POLICY_RAW;
  csw_sparse_layout L{};
  if (policy == CSW_POLICY_SPARSE && (csw_sparse_layout_of(numel, &L) != CSW_OK || m->free_slots.empty()))
    policy = CSW_POLICY_RAW;

  csw_ticket* t = new (std::nothrow) csw_ticket;
  if (!t) return CSW_ERR_NOMEM;
  t->policy = policy;
  t->numel = numel;
  t->maxbits = m->maxbits;
  const size_t raw = numel * sizeof(float);
  const size_t host_need = policy == CSW_POLICY_RAW ? raw : policy == CSW_POLICY_ZFP ? zbytes : L.bound;
  const size_t stage_need = policy == CSW_POLICY_RAW ? 0 : host_need;

  auto fail = [&](csw_status st) {
    // codec or copy work may already be queued on the manager's streams: let it finish
    // before the memory it touches goes back to the pools
    cudaStreamSynchronize(m->s_codec);
    cudaStreamSynchronize(m->s_d2h);
    cudaGetLastError();
    if (t->host) m->pinned.release(t->host, t->host_cap);
    free_stage(m, t);
    if (t->nnz_slot >= 0) m->free_slots.push_back(t->nnz_slot);
    put_event(m, t->ev_read);
    put_event(m, t->ev_d2h);
    delete t;
    return st;
  };

  t->host = pool_alloc(m, m->pinned, host_need, &t->host_cap);
  if (!t->host) return fail(CSW_ERR_NOMEM);
  if (stage_need) {
    t->stage = pool_alloc(m, m->staging, stage_need, &t->stage_cap);
    if (!t->stage) return fail(CSW_ERR_NOMEM);
  }
  cudaError_t e = get_event(m, &t->ev_read);
  if (e == cudaSuccess) e = get_event(m, &t->ev_d2h);
  if (e != cudaSuccess) return fail(cuda_fail(e));

  // the producer's work on `compute` must be visible to our streams
  cudaEvent_t ev_ready = nullptr;
  e = get_event(m, &ev_ready);
  if (e == cudaSuccess) e = cudaEventRecord(ev_ready, compute);
  if (e == cudaSuccess && policy != CSW_POLICY_RAW) e = cudaStreamWaitEvent(m->s_codec, ev_ready, 0);
  if (policy != CSW_POLICY_RAW || e != cudaSuccess) put_event(m, ev_ready);
  if (e != cudaSuccess) return fail(cuda_fail(e));

  csw_status st = CSW_OK;
  if (policy == CSW_POLICY_RAW) {
    // queued; pump_raw hands it to the copy stream when fewer than kRawInFlight are on it
    t->ev_ready = ev_ready;
    t->src = d_ptr;
    t->queued = true;
    t->moved = raw;
    t->moved_final = true;
    m->raw_queue.push_back(t);
    pump_raw(m);
  } else if (policy == CSW_POLICY_ZFP) {
    st = csw_zfp_compress(d_ptr, 32, 32, nz, m->maxbits, t->stage, t->stage_cap, nullptr, m->s_codec);
    if (st == CSW_OK && zbytes > zstream)  // the values past the last whole slab
      e = cudaMemcpyAsync(static_cast<char*>(t->stage) + zstream, d_ptr + nz * 1024, zbytes - zstream,
                          cudaMemcpyDeviceToDevice, m->s_codec);
    if (st == CSW_OK && e == cudaSuccess) {
      e = cudaEventRecord(t->ev_read, m->s_codec);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(m->s_d2h, t->ev_read, 0);
      if (e == cudaSuccess) e = cudaMemcpyAsync(t->host, t->stage, zbytes, cudaMemcpyDeviceToHost, m->s_d2h);
      if (e == cudaSuccess) e = cudaEventRecord(t->ev_d2h, m->s_d2h);
    }
    t->moved = zbytes;
    t->moved_final = true;
  } else {
    t->nnz_slot = m->free_slots.back();
    m->free_slots.pop_back();
    t->nnz_host = m->nnz_slots + t->nnz_slot;
    uint32_t* nnz_dev = m->nnz_dev + t->nnz_slot;
    st = csw_sparse_compress_onepass(d_ptr, numel, t->stage, t->stage_cap, nnz_dev, m->s_codec);
    if (st == CSW_OK) {
      e = cudaEventRecord(t->ev_read, m->s_codec);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(m->s_d2h, t->ev_read, 0);
      if (e == cudaSuccess) {
        sparse_to_host_kernel<<<32, 256, 0, m->s_d2h>>>(reinterpret_cast<const uint4*>(t->stage),
                                                        reinterpret_cast<uint4*>(t->host), nnz_dev, t->nnz_host,
                                                        L.values);
        e = cudaGetLastError();
      }
      if (e == cudaSuccess) e = cudaEventRecord(t->ev_d2h, m->s_d2h);
    }
    t->moved = L.bound;  // upper bound until the count lands
  }
  if (st != CSW_OK) return fail(st);
  if (e != cudaSuccess) return fail(cuda_fail(e));

  m->stats.swap_outs++;
  m->stats.raw_bytes_out += raw;
  if (t->moved_final && policy != CSW_POLICY_RAW) m->stats.moved_bytes_out += t->moved;  // raw: when its copy is issued
  m->live.push_back(t);
  t->in_live = true;
  m->all.push_back(t);
  *ticket = t;
  return CSW_OK;
}

csw_status csw_swap_out_done(csw_mgr* m, csw_ticket* t, int* done) {
  if (!m || !t || !done) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  pump_raw(m);
  if (t->queued) {  // its copy has not even been issued
    *done = 0;
    return CSW_OK;
  }
  cudaError_t e = cudaEventQuery(t->ev_read);
  if (e != cudaSuccess && e != cudaErrorNotReady) return cuda_fail(e);
  cudaGetLastError();
  *done = e == cudaSuccess;
  return CSW_OK;
}

csw_status csw_swap_out_sync(csw_mgr* m, csw_ticket* t) {
  if (!m || !t) return CSW_ERR_ARG;
  cudaEvent_t ev;
  {
    std::lock_guard<std::mutex> lk(m->mu);
    if (t->state == T_DEAD) return CSW_ERR_STATE;
    DeviceGuard g0(m->device);
    submit_raw_through(m, t);
    ev = t->ev_read;
  }
  DeviceGuard g(m->device);
  cudaError_t e = cudaEventSynchronize(ev);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

csw_status csw_swap_out_wait(csw_mgr* m, csw_ticket* t, csw_stream_t stream) {
  if (!m || !t) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  submit_raw_through(m, t);
  cudaError_t e = cudaStreamWaitEvent(stream, t->ev_read, 0);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

// Brings the payload of a codec ticket back into device staging (no-op for raw).
static csw_status load_stage(csw_mgr* m, csw_ticket* t) {
  if (t->policy == CSW_POLICY_RAW || t->stage_loaded) return CSW_OK;
  cudaError_t e;
  if (t->state == T_OUT) {
    // still going out: the staging copy is intact once the codec has written it
    if (!t->moved_final) {
      e = cudaEventSynchronize(t->ev_d2h);
      if (e != cudaSuccess) return cuda_fail(e);
      finalize_moved(m, t);
    }
    if (t->stage) {
      t->stage_loaded = true;
      if (!t->ev_h2d) {
        e = get_event(m, &t->ev_h2d);
        if (e != cudaSuccess) return cuda_fail(e);
      }
      // nothing to wait for but the codec that wrote it, which the decoder's own stream
      // has behind it already; the copy out goes on reading the staged payload meanwhile
      // (poll() keeps it until both have finished)
      e = cudaEventRecord(t->ev_h2d, m->s_codec);
      return e == cudaSuccess ? CSW_OK : cuda_fail(e);
    }
  }
  if (t->stage && t->cached) {
    // on the host and still staged: nothing crosses the link
    uncache(m, t);
    t->stage_loaded = true;
    if (!t->ev_h2d) {
      e = get_event(m, &t->ev_h2d);
      if (e != cudaSuccess) return cuda_fail(e);
    }
    e = cudaEventRecord(t->ev_h2d, m->s_codec);
    return e == cudaSuccess ? CSW_OK : cuda_fail(e);
  }
  if (!t->moved_final) {
    e = cudaEventSynchronize(t->ev_d2h);
    if (e != cudaSuccess) return cuda_fail(e);
    finalize_moved(m, t);
  }
  if (!t->stage) {
    t->stage = pool_alloc(m, m->staging, t->moved, &t->stage_cap);
    if (!t->stage) return CSW_ERR_NOMEM;
  }
  if (!t->ev_h2d) {
    e = get_event(m, &t->ev_h2d);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  e = t->ev_d2h ? cudaStreamWaitEvent(m->s_h2d, t->ev_d2h, 0) : cudaSuccess;  // imported tickets have no copy out
  if (e == cudaSuccess) e = cudaMemcpyAsync(t->stage, t->host, t->moved, cudaMemcpyHostToDevice, m->s_h2d);
  if (e == cudaSuccess) e = cudaEventRecord(t->ev_h2d, m->s_h2d);
  if (e != cudaSuccess) return cuda_fail(e);
  t->stage_loaded = true;
  m->stats.moved_bytes_in += t->moved;
  return CSW_OK;
}

csw_status csw_prefetch(csw_mgr* m, csw_ticket* t) {
  if (!m || !t) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (t->state == T_DEAD) return CSW_ERR_STATE;
  poll(m);
  return load_stage(m, t);
}

csw_status csw_swap_in(csw_mgr* m, csw_ticket* t, float* d_dst, csw_stream_t compute) {
  csw_status st = csw_swap_in_start(m, t, d_dst, compute);
  return st == CSW_OK ? csw_swap_in_wait(m, t, compute) : st;
}

csw_status csw_swap_in_wait(csw_mgr* m, csw_ticket* t, csw_stream_t compute) {
  if (!m || !t) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (t->state == T_DEAD || !t->ev_done) return CSW_ERR_STATE;  // no csw_swap_in_start before it
  cudaError_t e = cudaStreamWaitEvent(compute, t->ev_done, 0);
  return e == cudaSuccess ? CSW_OK : cuda_fail(e);
}

csw_status csw_swap_in_start(csw_mgr* m, csw_ticket* t, float* d_dst, csw_stream_t compute) {
  if (!m || !t || !d_dst) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (t->state == T_DEAD) return CSW_ERR_STATE;
  poll(m);
  cudaError_t e = cudaSuccess;
  if (!t->ev_done) {
    e = get_event(m, &t->ev_done);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  // the destination may still be in use by earlier work on `compute`
  cudaEvent_t ev_free = nullptr;
  e = get_event(m, &ev_free);
  if (e == cudaSuccess) e = cudaEventRecord(ev_free, compute);
  cudaStream_t worker = t->policy == CSW_POLICY_RAW ? m->s_h2d : m->s_codec;
  if (e == cudaSuccess) e = cudaStreamWaitEvent(worker, ev_free, 0);
  put_event(m, ev_free);
  if (e != cudaSuccess) return cuda_fail(e);

  const size_t raw = t->numel * sizeof(float);
  csw_status st = CSW_OK;
  if (t->policy == CSW_POLICY_RAW) {
    submit_raw_through(m, t);
    e = t->ev_d2h ? cudaStreamWaitEvent(m->s_h2d, t->ev_d2h, 0) : cudaSuccess;
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_dst, t->host, raw, cudaMemcpyHostToDevice, m->s_h2d);
    if (e == cudaSuccess) e = cudaEventRecord(t->ev_done, m->s_h2d);
  } else {
    st = load_stage(m, t);
    if (st != CSW_OK) return st;
    e = cudaStreamWaitEvent(m->s_codec, t->ev_h2d, 0);
    if (e != cudaSuccess) return cuda_fail(e);
    if (t->policy == CSW_POLICY_ZFP) {
      const size_t nz = t->numel / 1024, tail = (t->numel % 1024) * sizeof(float);
      st = csw_zfp_decompress(t->stage, t->moved - tail, 32, 32, nz, t->maxbits, d_dst, m->s_codec);
      if (st == CSW_OK && tail) {
        e = cudaMemcpyAsync(d_dst + nz * 1024, static_cast<const char*>(t->stage) + (t->moved - tail), tail,
                            cudaMemcpyDeviceToDevice, m->s_codec);
        if (e != cudaSuccess) return cuda_fail(e);
      }
    } else {
      st = csw_sparse_decompress(t->stage, t->numel, d_dst, m->s_codec);
    }
    if (st != CSW_OK) return st;
    e = cudaEventRecord(t->ev_done, m->s_codec);
  }
  if (e != cudaSuccess) return cuda_fail(e);
  t->state = T_IN;
  if (!t->in_live) {
    m->live.push_back(t);
    t->in_live = true;
  }
  m->stats.swap_ins++;
  m->stats.raw_bytes_in += raw;
  if (t->policy == CSW_POLICY_RAW) m->stats.moved_bytes_in += raw;  // codec tickets count in load_stage, when they cross
  return CSW_OK;
}

csw_status csw_ticket_release(csw_mgr* m, csw_ticket* t) {
  if (!m || !t) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (t->state == T_DEAD) return CSW_ERR_STATE;
  // Never blocks: memory goes back to the pools now if nothing in flight
  // touches it, otherwise as soon as a later call finds its copies finished.
  // a raw ticket whose copy has not been issued is never copied at all (taken out of the queue
  // before anything below can pump it onto the copy stream)
  const bool never_copied = t->queued;
  if (never_copied) forget_raw(m, t);
  const bool idle = never_copied || (event_done(t->ev_d2h) && event_done(t->ev_h2d) && event_done(t->ev_done));
  cudaGetLastError();
  if (idle && t->policy == CSW_POLICY_SPARSE && !t->moved_final) finalize_moved(m, t);
  t->state = T_DEAD;
  drop_from_live(m, t);
  poll(m);
  if (idle) destroy_ticket(m, t);
  else m->zombies.push_back(t);
  return CSW_OK;
}

csw_status csw_swap_out_cancel(csw_mgr* m, csw_ticket* t, int* cancelled) {
  if (!m || !t || !cancelled) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (t->state == T_DEAD) return CSW_ERR_STATE;
  *cancelled = t->queued ? 1 : 0;
  if (t->queued) {
    forget_raw(m, t);
    t->state = T_DEAD;
    drop_from_live(m, t);
    destroy_ticket(m, t);
  }
  return CSW_OK;
}

csw_status csw_ticket_query(csw_mgr* m, csw_ticket* t, csw_ticket_info* info) {
  if (!m || !t || !info) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  poll(m);
  info->policy = t->policy;
  info->numel = t->numel;
  info->raw_bytes = t->numel * sizeof(float);
  info->moved_bytes = t->moved;
  info->complete = t->moved_final ? 1 : 0;
  return CSW_OK;
}

// ---- self-describing blobs ---------------------------------------------------------
static_assert(sizeof(csw_blob_header) == 64, "blob header layout");

static inline int popcount32(uint32_t v) { return __builtin_popcount(v); }

csw_status csw_blob_info(const void* blob, size_t bytes, csw_blob_header* header) {
  if (!blob || !header) return CSW_ERR_ARG;
  if (bytes < sizeof(csw_blob_header)) return CSW_ERR_SIZE;
  csw_blob_header h;
  std::memcpy(&h, blob, sizeof h);
  if (h.magic != CSW_BLOB_MAGIC || h.version != CSW_BLOB_VERSION || h.numel == 0) return CSW_ERR_ARG;
  // element counts beyond 2^40 (4 TiB of floats) cannot be real and would let the size arithmetic below wrap
  if (h.numel > ((uint64_t)1 << 40)) return CSW_ERR_ARG;
  if (bytes - sizeof h < h.payload_bytes) return CSW_ERR_SIZE;
  const unsigned char* payload = static_cast<const unsigned char*>(blob) + sizeof h;
  if (h.policy == CSW_POLICY_RAW) {
    if (h.payload_bytes != h.numel * sizeof(float) || h.nnz != 0 || h.zfp_maxbits != 0) return CSW_ERR_ARG;
  } else if (h.policy == CSW_POLICY_ZFP) {
    size_t nz = 0, zstream = 0, zbytes = 0;
    if (zfp_geometry(h.numel, h.zfp_maxbits, &nz, &zstream, &zbytes) != CSW_OK || h.payload_bytes != zbytes ||
        h.nnz != 0)
      return CSW_ERR_ARG;
  } else if (h.policy == CSW_POLICY_SPARSE) {
    csw_sparse_layout L;
    if (csw_sparse_layout_of(h.numel, &L) != CSW_OK || h.zfp_maxbits != 0 || h.nnz > h.numel ||
        h.payload_bytes != L.values + 4 * h.nnz)
      return CSW_ERR_ARG;
    // every tile's segment must lie inside the packed values: the unpack kernel
    // trusts tile_off, so a damaged blob is turned away here, on the host
    const size_t tiles = (h.numel + SPARSE_TILE - 1) / SPARSE_TILE, words = (h.numel + 31) / 32;
    uint64_t total = 0;
    for (size_t t = 0; t < tiles; t++) {
      uint32_t off;
      std::memcpy(&off, payload + L.tile_off + 4 * t, 4);
      const size_t w0 = t * (SPARSE_TILE / 32), w1 = w0 + SPARSE_TILE / 32 < words ? w0 + SPARSE_TILE / 32 : words;
      uint32_t cnt = 0;
      for (size_t w = w0; w < w1; w++) {
        uint32_t bits;
        std::memcpy(&bits, payload + L.bitmap + 4 * w, 4);
        if (w == words - 1 && (h.numel & 31)) bits &= (1u << (h.numel & 31)) - 1u;
        cnt += (uint32_t)popcount32(bits);
      }
      if ((uint64_t)off + cnt > h.nnz) return CSW_ERR_ARG;
      total += cnt;
    }
    if (total != h.nnz) return CSW_ERR_ARG;
  } else {
    return CSW_ERR_ARG;
  }
  *header = h;
  return CSW_OK;
}

csw_status csw_ticket_export(csw_mgr* m, csw_ticket* t, void* dst, size_t cap, size_t* bytes) {
  if (!m || !t || !bytes) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (t->state == T_DEAD) return CSW_ERR_STATE;
  submit_raw_through(m, t);
  if (t->ev_d2h) {
    cudaError_t e = cudaEventSynchronize(t->ev_d2h);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  if (!t->moved_final) finalize_moved(m, t);
  const size_t total = sizeof(csw_blob_header) + t->moved;
  *bytes = total;
  if (!dst) return CSW_OK;
  if (cap < total) return CSW_ERR_SIZE;
  csw_blob_header h{};
  h.magic = CSW_BLOB_MAGIC;
  h.version = CSW_BLOB_VERSION;
  h.policy = (uint32_t)t->policy;
  h.zfp_maxbits = t->policy == CSW_POLICY_ZFP ? t->maxbits : 0u;
  h.numel = t->numel;
  h.payload_bytes = t->moved;
  if (t->policy == CSW_POLICY_SPARSE) {
    csw_sparse_layout L;
    csw_sparse_layout_of(t->numel, &L);
    h.nnz = (t->moved - L.values) / 4;
  }
  std::memcpy(dst, &h, sizeof h);
  std::memcpy(static_cast<char*>(dst) + sizeof h, t->host, t->moved);
  return CSW_OK;
}

csw_status csw_blob_import(csw_mgr* m, const void* blob, size_t bytes, csw_ticket** ticket) {
  if (!m || !ticket) return CSW_ERR_ARG;
  csw_blob_header h;
  csw_status st = csw_blob_info(blob, bytes, &h);
  if (st != CSW_OK) return st;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (!g.ok) return CSW_ERR_ARG;
  poll(m);
  csw_ticket* t = new (std::nothrow) csw_ticket;
  if (!t) return CSW_ERR_NOMEM;
  t->policy = (int)h.policy;
  t->numel = (size_t)h.numel;
  t->maxbits = h.zfp_maxbits;
  t->state = T_HOST;
  t->moved = (size_t)h.payload_bytes;
  t->moved_final = true;
  t->host = pool_alloc(m, m->pinned, t->moved, &t->host_cap);
  if (!t->host) {
    delete t;
    return CSW_ERR_NOMEM;
  }
  std::memcpy(t->host, static_cast<const char*>(blob) + sizeof h, t->moved);
  m->all.push_back(t);
  *ticket = t;
  return CSW_OK;
}

csw_status csw_mgr_get_stats(csw_mgr* m, csw_mgr_stats* s) {
  if (!m || !s) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  poll(m);
  *s = m->stats;
  s->pinned_in_use = m->pinned.in_use();
  s->pinned_high_water = m->pinned.high_water();
  s->staging_in_use = m->staging.in_use();
  s->staging_high_water = m->staging.high_water();
  return CSW_OK;
}

csw_status csw_mgr_reset_stats(csw_mgr* m) {
  if (!m) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  m->stats = csw_mgr_stats{};
  return CSW_OK;
}

csw_status csw_mgr_sync(csw_mgr* m) {
  if (!m) return CSW_ERR_ARG;
  std::lock_guard<std::mutex> lk(m->mu);
  DeviceGuard g(m->device);
  if (!m->raw_queue.empty()) submit_raw_through(m, m->raw_queue.back());
  cudaError_t e = cudaStreamSynchronize(m->s_codec);
  if (e == cudaSuccess) e = cudaStreamSynchronize(m->s_d2h);
  if (e == cudaSuccess) e = cudaStreamSynchronize(m->s_h2d);
  if (e != cudaSuccess) return cuda_fail(e);
  poll(m);
  // "everything is on the host": the staged copies kept for a quick return go as well
  while (!m->cache.empty()) free_stage(m, m->cache.front());
  return CSW_OK;
}

}  // extern "C"
