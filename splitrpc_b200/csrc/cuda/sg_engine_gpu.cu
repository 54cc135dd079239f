// GPU scatter-gather engine: turns the fragment lists of a batch of requests into
// one copy-list submission on the serving GPU.
//
// Submission modes follow P2P_RPC_GPU_COPY_TYPE of reference
// src/transport/g_copy_ng.cu:194-216 and src/p2p_rpc_sg_engine.h:185-308:
//   0  copy-engine DMA: one cudaMemcpyAsync per coalesced run
//   1  resident kernel behind a doorbell in mapped host memory (re-armed by the
//      host whenever it has left after its idle limit)
//   2  one kernel launch per submission (SIMT vector copies)
//   3  one kernel launch per submission (cp.async.bulk pipeline)
// Every call returns only when the bytes are visible (bounded wait); the status
// is 0 or negative.
#include <cuda_runtime.h>

#include <chrono>
#include <thread>

#include "../host/p2p_rpc_sg_engine.h"
#include "gemm_tcgen05.h"
#include "sg_kernels.cuh"

namespace {

class P2pRpcSgGpuEngine : public P2pRpcSgEngine {
  int copy_type_;
  // Blocks per copy kernel.  A list whose sources sit in host memory is bound by the PCIe link and needs only enough
  // loads in flight to cover its latency.  When the model's persistent kernels leave r SMs out of their grids
  // (srpc_gemm_reserve_sms), the copy runs as r blocks of 1024 threads (written -r): twelve reach the link rate, and
  // the model beside it runs as fast as alone (measured: ResNet-50 graph 1.68 ms with the copy, 1.63 ms alone, against
  // 1.98 ms when the copy's 48 blocks of 256 threads each hold an SM that a persistent kernel counts on).  Lists
  // that read device memory get four blocks of 256 threads per SM.  P2P_RPC_SG_BLOCKS overrides both
  // (negative = 1024-thread blocks).
  int n_blocks_ = readEnvInfo<int>("P2P_RPC_SG_BLOCKS", 0);
  int blocks_for(const SgItem& first) const {
    if (n_blocks_ != 0) return n_blocks_;
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, (const void*)first.src) != cudaSuccess) {
      (void)cudaGetLastError();
      return 0;
    }
    if (a.type != cudaMemoryTypeHost) return 0;
    const int r = srpc_gemm_reserved_sms();
    return r > 0 ? -r : 48;
  }
  cudaStream_t stream_ = nullptr;

  // Submission slots.  A synchronous call uses slot 0 and waits; calls that finish by themselves (gather_batch_notify)
  // rotate through all of them, so the host builds list k+1 while the kernel of list k still runs.  Per slot: the copy
  // list and the doorbell addresses in pinned host memory, their device copies, and the arrival counter of the launch.
  static constexpr int kSlots = 4;
  static constexpr uint32_t kMaxBells = 1024;
  struct Slot {
    SgItem* h_items = nullptr;
    uint64_t* h_bells = nullptr;
    SgItem* d_items = nullptr;
    uint64_t* d_bells = nullptr;
    uint32_t* d_counter = nullptr;
    uint32_t ticket = 0;  // last submission that used this slot
  } slots_[kSlots];
  SgItem* h_items_ = nullptr;  // = slots_[cur_].h_items while a list is being built
  int cur_ = 0;
  volatile uint32_t* h_done_ = nullptr;  // mapped: sequence number of the newest finished asynchronous submission
  uint32_t* d_done_ = nullptr;
  uint32_t ticket_ = 0;

  SgCtrl* h_ctrl_ = nullptr;   // persistent mode control block (mapped)
  SgCtrl* d_ctrl_ = nullptr;
  uint32_t* d_counter_ = nullptr;
  bool resident_ = false;
  uint32_t seq_ = 0;
  int persistent_blocks_ = 16;
  uint64_t wait_budget_ns_ = 2000000000ull;

  // ---- resident kernel (copy type 1)
  // Stops the resident kernel: asks every block to leave, waits (bounded) until all have, and only then lets the
  // stream drain.  The doorbell is never moved backwards; a sequence number that was rung but not served stays
  // consumed, and the list is submitted again under a new one.
  bool stop_resident() {
    if (!resident_) return true;
    __atomic_store_n(&h_ctrl_->exit_flag, 1u, __ATOMIC_RELEASE);
    uint64_t t0 = getCurNs();
    while (__atomic_load_n(&h_ctrl_->exited, __ATOMIC_ACQUIRE) < (uint32_t)persistent_blocks_) {
      if (getCurNs() - t0 > wait_budget_ns_) return false;
      std::this_thread::yield();
    }
    cudaStreamSynchronize(stream_);
    resident_ = false;
    return true;
  }

  bool ensure_resident() {
    if (resident_ && __atomic_load_n(&h_ctrl_->exited, __ATOMIC_ACQUIRE) == 0) return true;
    if (!stop_resident()) return false;  // some blocks have left after their idle limit: collect the rest, then re-arm
    h_ctrl_->exited = 0;
    h_ctrl_->exit_flag = 0;
    h_ctrl_->error = 0;
    h_ctrl_->done = seq_;
    h_ctrl_->doorbell = seq_;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    // every block has left: the arrival counter of a half-served submission can be cleared safely
    cudaMemsetAsync(d_counter_, 0, sizeof(uint32_t), stream_);
    if (sg_launch_persistent(d_ctrl_, d_counter_, persistent_blocks_, stream_) != cudaSuccess) return false;
    resident_ = true;
    return true;
  }

  int submit_persistent(const SgItem* items, uint32_t n) {
    for (uint32_t off = 0; off < n; off += SG_PERSISTENT_ITEMS) {
      uint32_t m = n - off < SG_PERSISTENT_ITEMS ? n - off : SG_PERSISTENT_ITEMS;
      bool served = false;
      for (int attempt = 0; attempt < 2 && !served; attempt++) {
        if (!ensure_resident()) return -2;
        SgItem* dst = const_cast<SgItem*>(h_ctrl_->items);
        std::memcpy(dst, items + off, m * sizeof(SgItem));
        h_ctrl_->n_items = m;
        h_ctrl_->n_chunks = sg_assign_chunks(dst, m);
        std::atomic_thread_fence(std::memory_order_release);
        const uint32_t s = ++seq_;
        __atomic_store_n(&h_ctrl_->doorbell, s, __ATOMIC_RELEASE);
        uint64_t t0 = getCurNs();
        bool gone = false;
        for (;;) {
          if (__atomic_load_n(&h_ctrl_->done, __ATOMIC_ACQUIRE) == s) {
            served = true;
            break;
          }
          if (__atomic_load_n(&h_ctrl_->exited, __ATOMIC_ACQUIRE) != 0) {
            gone = true;
            break;
          }
          if (getCurNs() - t0 > wait_budget_ns_) break;
        }
        if (served) break;
        // Blocks left between the residency check and the doorbell (idle limit), or the wait ran out.  Either way the
        // kernel is stopped completely before anything else happens; the copies it may have made are idempotent.
        if (!stop_resident()) return -2;
        if (!gone) {
          counters.timeouts++;
          return -1;
        }
      }
      if (!served) {
        counters.timeouts++;
        return -1;
      }
    }
    return 0;
  }

  // Optional transform applied by gathers (not by scatters): see set_gather_transform.
  bool has_transform_ = false;
  SgStemS2d transform_{};

  static bool reached(uint32_t done, uint32_t ticket) { return (int32_t)(done - ticket) >= 0; }

  // Makes slot `k` safe to overwrite: the asynchronous submission that used it last has finished.
  bool wait_slot_free(int k) {
    const uint32_t t = slots_[k].ticket;
    if (t == 0) return true;
    uint64_t t0 = getCurNs();
    while (!reached(__atomic_load_n(h_done_, __ATOMIC_ACQUIRE), t)) {
      if (getCurNs() - t0 > wait_budget_ns_) return false;
    }
    return true;
  }
  bool begin_list() {
    if (!wait_slot_free(cur_)) return false;
    h_items_ = slots_[cur_].h_items;
    return true;
  }

  // Launches the list built in the current slot.  notify == nullptr: waits for it (synchronous calls).
  int submit(uint32_t n, bool gather, const SgNotify* notify) {
    if (n == 0 && !notify) return 0;
    Slot& sl = slots_[cur_];
    counters.items += n;
    for (uint32_t i = 0; i < n; i++) counters.bytes += h_items_[i].len;
    cudaError_t e = cudaSuccess;
    if (copy_type_ == 0 && !notify) {
      for (uint32_t i = 0; i < n && e == cudaSuccess; i++)
        e = cudaMemcpyAsync((void*)h_items_[i].dst, (const void*)h_items_[i].src, h_items_[i].len, cudaMemcpyDefault, stream_);
      if (e == cudaSuccess) e = cudaStreamSynchronize(stream_);
    } else if (copy_type_ == 1 && !notify) {
      return submit_persistent(h_items_, n);
    } else {
      uint32_t chunks = sg_assign_chunks(h_items_, n);
      e = cudaMemcpyAsync(sl.d_items, h_items_, n * sizeof(SgItem), cudaMemcpyHostToDevice, stream_);
      if (e == cudaSuccess) {
        const int impl = (copy_type_ == 3 && !notify) ? SG_IMPL_BULK : SG_IMPL_SIMT;
        if (gather && has_transform_)
          e = sg_launch_stem_s2d(sl.d_items, n, chunks, transform_, blocks_for(h_items_[0]), stream_, notify);
        else
          e = sg_launch_copy(sl.d_items, n, chunks, impl, blocks_for(h_items_[0]), stream_, notify);
      }
      if (e == cudaSuccess && !notify) e = cudaStreamSynchronize(stream_);
    }
    if (e != cudaSuccess) {
      srpc_log(SRPC_LOG_ERROR, "GPU scatter-gather failed: %s", cudaGetErrorString(e));
      return -3;
    }
    return 0;
  }

  // Appends the coalesced runs of one request to the staging list.
  bool append(const p2p_sk_buf* skb, uint32_t* n) {
    for (size_t i = 0; i < skb->num_items; i++) {
      if (*n >= SG_MAX_ITEMS) return false;
      h_items_[*n].src = skb->i_buf[i];
      h_items_[*n].dst = skb->o_buf[i];
      h_items_[*n].len = (uint32_t)skb->len[i];
      h_items_[*n].first_chunk = 0;
      (*n)++;
    }
    return true;
  }

 public:
  P2pRpcSgGpuEngine(int dev, int copy_type) : copy_type_(copy_type) {
    device_id = dev;
    cudaSetDevice(dev);
    sg_preload_kernels();
    cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking);
    for (Slot& sl : slots_) {
      cudaHostAlloc(&sl.h_items, sizeof(SgItem) * SG_MAX_ITEMS, cudaHostAllocDefault);
      cudaHostAlloc(&sl.h_bells, sizeof(uint64_t) * kMaxBells, cudaHostAllocDefault);
      cudaMalloc(&sl.d_items, sizeof(SgItem) * SG_MAX_ITEMS);
      cudaMalloc(&sl.d_bells, sizeof(uint64_t) * kMaxBells);
      cudaMalloc(&sl.d_counter, sizeof(uint32_t));
      cudaMemset(sl.d_counter, 0, sizeof(uint32_t));
    }
    h_items_ = slots_[0].h_items;
    void* h = nullptr;
    cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable);
    std::memset(h, 0, 64);
    h_done_ = (volatile uint32_t*)h;
    cudaHostGetDevicePointer((void**)&d_done_, h, 0);
    if (copy_type_ == 1) {
      cudaHostAlloc(&h_ctrl_, sizeof(SgCtrl), cudaHostAllocMapped | cudaHostAllocPortable);
      std::memset(h_ctrl_, 0, sizeof(SgCtrl));
      cudaHostGetDevicePointer((void**)&d_ctrl_, h_ctrl_, 0);
      h_ctrl_->idle_limit_ns = (uint64_t)readEnvInfo<uint64_t>("P2P_RPC_SG_IDLE_MS", 200) * 1000000ull;
      cudaMalloc(&d_counter_, sizeof(uint32_t));
      cudaMemset(d_counter_, 0, sizeof(uint32_t));
    }
  }
  ~P2pRpcSgGpuEngine() override {
    cudaSetDevice(device_id);
    stop_resident();
    cudaStreamSynchronize(stream_);
    if (h_ctrl_) cudaFreeHost(h_ctrl_);
    if (d_counter_) cudaFree(d_counter_);
    for (Slot& sl : slots_) {
      cudaFree(sl.d_items);
      cudaFree(sl.d_bells);
      cudaFree(sl.d_counter);
      cudaFreeHost(sl.h_items);
      cudaFreeHost(sl.h_bells);
    }
    cudaFreeHost((void*)h_done_);
    cudaStreamDestroy(stream_);
  }

  using P2pRpcSgEngine::gather;
  using P2pRpcSgEngine::scatter;
  int gather(P2pRpcRr* rr, g_params* stub) override { return gather_batch(&rr, &stub, 1); }
  int scatter(P2pRpcRr* rr, g_params* stub) override { return scatter_batch(&rr, &stub, 1); }

  int gather_batch(P2pRpcRr** rrs, g_params** stubs, int n) override {
    PROF_START(Gather);
    cudaSetDevice(device_id);
    if (!begin_list()) return -1;
    uint32_t ni = 0;
    int rc = 0;
    for (int i = 0; i < n; i++) {
      gather_skbs(rrs[i]->payload_sk_bufs, rrs[i]->payload_bufs, stubs[i]->req);
      if (!append(rrs[i]->payload_sk_bufs, &ni)) {
        rc |= submit(ni, true, nullptr);
        ni = 0;
        append(rrs[i]->payload_sk_bufs, &ni);
      }
    }
    rc |= submit(ni, true, nullptr);
    counters.gathers += (uint64_t)n;
    PROF_STOP(Gather);
    return rc;
  }

  // Gather that finishes by itself: one launch (per SG_MAX_ITEMS items) whose last block stores `state_value` into the
  // d_states words and then publishes the ticket.  Nothing here waits for the GPU, except for a submission slot to
  // come free when kSlots submissions are already in flight.
  int64_t gather_batch_notify(P2pRpcRr** rrs, g_params** stubs, volatile uint32_t** h_states, volatile uint32_t** d_states,
                              int n, uint32_t state_value) override {
    // Only the launch-per-submission mode has a doorbell epilogue; DMA copies, the resident kernel and the bulk
    // pipeline keep their own way of submitting and complete the slots from the host.
    if (copy_type_ != 2) return P2pRpcSgEngine::gather_batch_notify(rrs, stubs, h_states, d_states, n, state_value);
    if (n <= 0 || (uint32_t)n > kMaxBells) return -4;
    PROF_START(Gather);
    cudaSetDevice(device_id);
    int rc = 0;
    int first = 0;
    uint32_t ticket = 0;
    while (first < n && rc == 0) {
      cur_ = (cur_ + 1) % kSlots;
      if (!begin_list()) {
        counters.timeouts++;
        return -1;
      }
      Slot& sl = slots_[cur_];
      uint32_t ni = 0;
      int i = first;
      for (; i < n; i++) {
        gather_skbs(rrs[i]->payload_sk_bufs, rrs[i]->payload_bufs, stubs[i]->req);
        const uint32_t before = ni;
        if (!append(rrs[i]->payload_sk_bufs, &ni)) {
          ni = before;  // this request goes into the next launch
          if (i == first) return -4;  // a single request with more runs than a launch can hold
          break;
        }
        sl.h_bells[i - first] = (uint64_t)(uintptr_t)d_states[i];
      }
      const uint32_t nb = (uint32_t)(i - first);
      ticket = ++ticket_;
      if (ticket == 0) ticket = ++ticket_;  // 0 means "slot never used"
      sl.ticket = ticket;
      cudaError_t e = cudaMemcpyAsync(sl.d_bells, sl.h_bells, nb * sizeof(uint64_t), cudaMemcpyHostToDevice, stream_);
      if (e != cudaSuccess) return -3;
      SgNotify nt;
      nt.counter = sl.d_counter;
      nt.bells = sl.d_bells;
      nt.n_bells = nb;
      nt.bell_value = state_value;
      nt.done_word = d_done_;
      nt.done_value = ticket;
      if (d_states_base_ && d_stamps_base_) {
        nt.states_base = (uint64_t)(uintptr_t)d_states_base_;
        nt.stamps_base = (uint64_t)(uintptr_t)d_stamps_base_;
      }
      rc = submit(ni, true, &nt);
      first = i;
    }
    counters.gathers += (uint64_t)n;
    PROF_STOP(Gather);
    return rc == 0 ? (int64_t)ticket : (int64_t)rc;
  }
  bool ticket_done(int64_t ticket) override {
    return ticket <= 0 || reached(__atomic_load_n(h_done_, __ATOMIC_ACQUIRE), (uint32_t)ticket);
  }

  int scatter_batch(P2pRpcRr** rrs, g_params** stubs, int n) override {
    PROF_START(Scatter);
    cudaSetDevice(device_id);
    if (!begin_list()) return -1;
    uint32_t ni = 0;
    int rc = 0;
    for (int i = 0; i < n; i++) {
      if (rrs[i]->payload_bufs->num_items == 0) continue;
      scatter_skbs(rrs[i]->payload_sk_bufs, rrs[i]->payload_bufs, stubs[i]->resp);
      if (!append(rrs[i]->payload_sk_bufs, &ni)) {
        rc |= submit(ni, false, nullptr);
        ni = 0;
        append(rrs[i]->payload_sk_bufs, &ni);
      }
    }
    rc |= submit(ni, false, nullptr);
    counters.scatters += (uint64_t)n;
    PROF_STOP(Scatter);
    return rc;
  }
  int copy_list(const p2p_sk_buf* skb) override {
    cudaSetDevice(device_id);
    if (!begin_list()) return -1;
    uint32_t ni = 0;
    if (!append(skb, &ni)) return -4;
    return submit(ni, false, nullptr);
  }
  int set_gather_transform(int kind, uint64_t ring_base, uint32_t slot_bytes, const float* params) override {
    if (kind == 0) {
      has_transform_ = false;
      return 0;
    }
    if (kind != SG_TRANSFORM_STEM_S2D || copy_type_ != 2 || !params) return -1;
    transform_.ring_base = ring_base;
    transform_.slot_bytes = slot_bytes;
    for (int i = 0; i < 3; i++) {
      transform_.mean[i] = params[i];
      transform_.inv_std[i] = params[3 + i];
    }
    has_transform_ = true;
    return 0;
  }
  const char* name() const override { return "gpu"; }
};

}  // namespace

extern "C" P2pRpcSgEngine* srpc_make_gpu_sg_engine(int device_id, int copy_type) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device_id >= n) return nullptr;
  return new P2pRpcSgGpuEngine(device_id, copy_type);
}

// ------------------------------------------------------------------ list helpers for the bindings
#include "ops_api.h"

struct SgListHandle {
  SgItem* d_items = nullptr;
  uint64_t* d_bells = nullptr;  // optional: addresses of the doorbell words that a launch rings when it has finished
  uint32_t* d_counter = nullptr;
  uint32_t n = 0, chunks = 0, n_bells = 0;
};

static std::vector<SgItem> to_items(const std::vector<SgTuple>& in, uint32_t* chunks) {
  std::vector<SgItem> v(in.size());
  for (size_t i = 0; i < in.size(); i++) {
    v[i].src = std::get<0>(in[i]);
    v[i].dst = std::get<1>(in[i]);
    v[i].len = std::get<2>(in[i]);
  }
  *chunks = sg_assign_chunks(v.data(), (uint32_t)v.size());
  return v;
}

uintptr_t srpc_sg_list_create(const std::vector<SgTuple>& items, const std::vector<uint64_t>& bells) {
  auto* h = new SgListHandle;
  std::vector<SgItem> v = to_items(items, &h->chunks);
  h->n = (uint32_t)v.size();
  h->n_bells = (uint32_t)bells.size();
  bool ok = cudaMalloc(&h->d_items, sizeof(SgItem) * (v.size() + 1)) == cudaSuccess &&
            cudaMemcpy(h->d_items, v.data(), sizeof(SgItem) * v.size(), cudaMemcpyHostToDevice) == cudaSuccess;
  if (ok && !bells.empty()) {
    ok = cudaMalloc(&h->d_bells, sizeof(uint64_t) * bells.size()) == cudaSuccess &&
         cudaMemcpy(h->d_bells, bells.data(), sizeof(uint64_t) * bells.size(), cudaMemcpyHostToDevice) == cudaSuccess &&
         cudaMalloc(&h->d_counter, sizeof(uint32_t)) == cudaSuccess && cudaMemset(h->d_counter, 0, sizeof(uint32_t)) == cudaSuccess;
  }
  if (!ok) {
    srpc_sg_list_destroy((uintptr_t)h);
    return 0;
  }
  return (uintptr_t)h;
}
void srpc_sg_list_destroy(uintptr_t handle) {
  auto* h = reinterpret_cast<SgListHandle*>(handle);
  if (!h) return;
  cudaFree(h->d_items);
  if (h->d_bells) cudaFree(h->d_bells);
  if (h->d_counter) cudaFree(h->d_counter);
  delete h;
}
// bell_value != 0 on a list created with bells: the launch's last block stores bell_value into every bell, then
// done_value into *done_word (when given); see SgNotify.
static SgNotify list_notify(const SgListHandle* h, uint32_t bell_value, uintptr_t done_word, uint32_t done_value) {
  SgNotify nt;
  if (h->d_bells && bell_value != 0) {
    nt.counter = h->d_counter;
    nt.bells = h->d_bells;
    nt.n_bells = h->n_bells;
    nt.bell_value = bell_value;
    nt.done_word = reinterpret_cast<uint32_t*>(done_word);
    nt.done_value = done_value;
  }
  return nt;
}
cudaError_t srpc_sg_list_launch(uintptr_t handle, int impl, int n_blocks, cudaStream_t stream, uint32_t bell_value,
                                uintptr_t done_word, uint32_t done_value) {
  auto* h = reinterpret_cast<SgListHandle*>(handle);
  if (!h) return cudaErrorInvalidValue;
  const SgNotify nt = list_notify(h, bell_value, done_word, done_value);
  return sg_launch_copy(h->d_items, h->n, h->chunks, impl, n_blocks, stream, nt.counter ? &nt : nullptr);
}
cudaError_t srpc_sg_list_launch_stem_s2d(uintptr_t handle, uint64_t ring_base, uint32_t slot_bytes, const float mean[3],
                                         const float inv_std[3], int n_blocks, cudaStream_t stream, uint32_t bell_value,
                                         uintptr_t done_word, uint32_t done_value) {
  auto* h = reinterpret_cast<SgListHandle*>(handle);
  if (!h) return cudaErrorInvalidValue;
  SgStemS2d tr{ring_base, slot_bytes, {mean[0], mean[1], mean[2]}, {inv_std[0], inv_std[1], inv_std[2]}};
  const SgNotify nt = list_notify(h, bell_value, done_word, done_value);
  return sg_launch_stem_s2d(h->d_items, h->n, h->chunks, tr, n_blocks, stream, nt.counter ? &nt : nullptr);
}
cudaError_t srpc_sg_copy_list(const std::vector<SgTuple>& items, int impl, int n_blocks, cudaStream_t stream) {
  uintptr_t h = srpc_sg_list_create(items, {});
  if (!h) return cudaErrorMemoryAllocation;
  cudaError_t e = srpc_sg_list_launch(h, impl, n_blocks, stream, 0, 0, 0);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  srpc_sg_list_destroy(h);
  return e;
}
cudaError_t srpc_sg_cast_list(const std::vector<SgTuple>& items, float scale, float shift, int n_blocks, cudaStream_t stream) {
  uintptr_t hh = srpc_sg_list_create(items, {});
  if (!hh) return cudaErrorMemoryAllocation;
  auto* h = reinterpret_cast<SgListHandle*>(hh);
  cudaError_t e = sg_launch_cast_bf16(h->d_items, h->n, h->chunks, scale, shift, n_blocks, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  srpc_sg_list_destroy(hh);
  return e;
}
