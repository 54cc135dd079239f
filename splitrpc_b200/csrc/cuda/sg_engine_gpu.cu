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
  SgItem* h_items_ = nullptr;  // pinned staging of the copy list
  SgItem* d_items_ = nullptr;
  SgCtrl* h_ctrl_ = nullptr;   // persistent mode control block (mapped)
  SgCtrl* d_ctrl_ = nullptr;
  uint32_t* d_counter_ = nullptr;
  bool resident_ = false;
  uint32_t seq_ = 0;
  int persistent_blocks_ = 16;
  uint64_t wait_budget_ns_ = 2000000000ull;

  bool ensure_resident() {
    if (resident_ && h_ctrl_->exited == 0) return true;
    if (resident_) {
      // Some blocks have left after their idle limit; wait for the rest, then re-arm.
      uint64_t t0 = getCurNs();
      while (h_ctrl_->exited < (uint32_t)persistent_blocks_) {
        if (getCurNs() - t0 > wait_budget_ns_) return false;
        std::this_thread::yield();
      }
      cudaStreamSynchronize(stream_);
    }
    h_ctrl_->exited = 0;
    h_ctrl_->exit_flag = 0;
    h_ctrl_->error = 0;
    h_ctrl_->done = seq_;
    h_ctrl_->doorbell = seq_;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    cudaMemsetAsync(d_counter_, 0, sizeof(uint32_t), stream_);
    if (sg_launch_persistent(d_ctrl_, d_counter_, persistent_blocks_, stream_) != cudaSuccess) return false;
    resident_ = true;
    return true;
  }

  int submit_persistent(const SgItem* items, uint32_t n) {
    for (uint32_t off = 0; off < n; off += SG_PERSISTENT_ITEMS) {
      uint32_t m = n - off < SG_PERSISTENT_ITEMS ? n - off : SG_PERSISTENT_ITEMS;
      for (int attempt = 0; attempt < 2; attempt++) {
        if (!ensure_resident()) return -2;
        SgItem* dst = const_cast<SgItem*>(h_ctrl_->items);
        std::memcpy(dst, items + off, m * sizeof(SgItem));
        h_ctrl_->n_items = m;
        h_ctrl_->n_chunks = sg_assign_chunks(dst, m);
        std::atomic_thread_fence(std::memory_order_release);
        uint32_t s = seq_ + 1;
        __atomic_store_n(&h_ctrl_->doorbell, s, __ATOMIC_RELEASE);
        uint64_t t0 = getCurNs();
        bool done = false, gone = false;
        while (!(done = (__atomic_load_n(&h_ctrl_->done, __ATOMIC_ACQUIRE) == s))) {
          if (h_ctrl_->exited != 0) {
            gone = true;
            break;
          }
          if (getCurNs() - t0 > wait_budget_ns_) break;
        }
        if (done) {
          seq_ = s;
          break;
        }
        // The kernel left between the residency check and the doorbell (or the
        // wait ran out): take the doorbell back and try once more on a fresh launch.
        __atomic_store_n(&h_ctrl_->doorbell, seq_, __ATOMIC_RELEASE);
        if (!gone || attempt == 1) {
          counters.timeouts++;
          return -1;
        }
      }
    }
    return 0;
  }

  // Optional transform applied by gathers (not by scatters): see set_gather_transform.
  bool has_transform_ = false;
  SgStemS2d transform_{};

  int submit(uint32_t n, bool gather = false) {
    if (n == 0) return 0;
    counters.items += n;
    for (uint32_t i = 0; i < n; i++) counters.bytes += h_items_[i].len;
    cudaError_t e = cudaSuccess;
    switch (copy_type_) {
      case 0:
        for (uint32_t i = 0; i < n && e == cudaSuccess; i++)
          e = cudaMemcpyAsync((void*)h_items_[i].dst, (const void*)h_items_[i].src, h_items_[i].len, cudaMemcpyDefault,
                              stream_);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream_);
        break;
      case 1:
        return submit_persistent(h_items_, n);
      default: {
        uint32_t chunks = sg_assign_chunks(h_items_, n);
        e = cudaMemcpyAsync(d_items_, h_items_, n * sizeof(SgItem), cudaMemcpyHostToDevice, stream_);
        if (e == cudaSuccess) {
          if (gather && has_transform_)
            e = sg_launch_stem_s2d(d_items_, n, chunks, transform_, blocks_for(h_items_[0]), stream_);
          else
            e = sg_launch_copy(d_items_, n, chunks, copy_type_ == 3 ? SG_IMPL_BULK : SG_IMPL_SIMT, blocks_for(h_items_[0]), stream_);
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream_);
      }
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
    cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking);
    cudaHostAlloc(&h_items_, sizeof(SgItem) * SG_MAX_ITEMS, cudaHostAllocDefault);
    cudaMalloc(&d_items_, sizeof(SgItem) * SG_MAX_ITEMS);
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
    if (resident_) {
      __atomic_store_n(&h_ctrl_->exit_flag, 1u, __ATOMIC_RELEASE);
      cudaStreamSynchronize(stream_);
    }
    if (h_ctrl_) cudaFreeHost(h_ctrl_);
    if (d_counter_) cudaFree(d_counter_);
    cudaFree(d_items_);
    cudaFreeHost(h_items_);
    cudaStreamDestroy(stream_);
  }

  using P2pRpcSgEngine::gather;
  using P2pRpcSgEngine::scatter;
  int gather(P2pRpcRr* rr, g_params* stub) override { return gather_batch(&rr, &stub, 1); }
  int scatter(P2pRpcRr* rr, g_params* stub) override { return scatter_batch(&rr, &stub, 1); }

  int gather_batch(P2pRpcRr** rrs, g_params** stubs, int n) override {
    PROF_START(Gather);
    cudaSetDevice(device_id);
    uint32_t ni = 0;
    int rc = 0;
    for (int i = 0; i < n; i++) {
      gather_skbs(rrs[i]->payload_sk_bufs, rrs[i]->payload_bufs, stubs[i]->req);
      if (!append(rrs[i]->payload_sk_bufs, &ni)) {
        rc |= submit(ni, true);
        ni = 0;
        append(rrs[i]->payload_sk_bufs, &ni);
      }
    }
    rc |= submit(ni, true);
    counters.gathers += (uint64_t)n;
    PROF_STOP(Gather);
    return rc;
  }

  int scatter_batch(P2pRpcRr** rrs, g_params** stubs, int n) override {
    PROF_START(Scatter);
    cudaSetDevice(device_id);
    uint32_t ni = 0;
    int rc = 0;
    for (int i = 0; i < n; i++) {
      if (rrs[i]->payload_bufs->num_items == 0) continue;
      scatter_skbs(rrs[i]->payload_sk_bufs, rrs[i]->payload_bufs, stubs[i]->resp);
      if (!append(rrs[i]->payload_sk_bufs, &ni)) {
        rc |= submit(ni);
        ni = 0;
        append(rrs[i]->payload_sk_bufs, &ni);
      }
    }
    rc |= submit(ni);
    counters.scatters += (uint64_t)n;
    PROF_STOP(Scatter);
    return rc;
  }
  int copy_list(const p2p_sk_buf* skb) override {
    cudaSetDevice(device_id);
    uint32_t ni = 0;
    if (!append(skb, &ni)) return -4;
    return submit(ni);
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
  uint32_t n = 0, chunks = 0;
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

uintptr_t srpc_sg_list_create(const std::vector<SgTuple>& items) {
  auto* h = new SgListHandle;
  std::vector<SgItem> v = to_items(items, &h->chunks);
  h->n = (uint32_t)v.size();
  if (cudaMalloc(&h->d_items, sizeof(SgItem) * (v.size() + 1)) != cudaSuccess ||
      cudaMemcpy(h->d_items, v.data(), sizeof(SgItem) * v.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
    delete h;
    return 0;
  }
  return (uintptr_t)h;
}
void srpc_sg_list_destroy(uintptr_t handle) {
  auto* h = reinterpret_cast<SgListHandle*>(handle);
  if (!h) return;
  cudaFree(h->d_items);
  delete h;
}
cudaError_t srpc_sg_list_launch(uintptr_t handle, int impl, int n_blocks, cudaStream_t stream) {
  auto* h = reinterpret_cast<SgListHandle*>(handle);
  if (!h) return cudaErrorInvalidValue;
  return sg_launch_copy(h->d_items, h->n, h->chunks, impl, n_blocks, stream);
}
cudaError_t srpc_sg_list_launch_stem_s2d(uintptr_t handle, uint64_t ring_base, uint32_t slot_bytes, const float mean[3],
                                         const float inv_std[3], int n_blocks, cudaStream_t stream) {
  auto* h = reinterpret_cast<SgListHandle*>(handle);
  if (!h) return cudaErrorInvalidValue;
  SgStemS2d tr{ring_base, slot_bytes, {mean[0], mean[1], mean[2]}, {inv_std[0], inv_std[1], inv_std[2]}};
  return sg_launch_stem_s2d(h->d_items, h->n, h->chunks, tr, n_blocks, stream);
}
cudaError_t srpc_sg_copy_list(const std::vector<SgTuple>& items, int impl, int n_blocks, cudaStream_t stream) {
  uintptr_t h = srpc_sg_list_create(items);
  if (!h) return cudaErrorMemoryAllocation;
  cudaError_t e = srpc_sg_list_launch(h, impl, n_blocks, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  srpc_sg_list_destroy(h);
  return e;
}
cudaError_t srpc_sg_cast_list(const std::vector<SgTuple>& items, float scale, float shift, int n_blocks, cudaStream_t stream) {
  uintptr_t hh = srpc_sg_list_create(items);
  if (!hh) return cudaErrorMemoryAllocation;
  auto* h = reinterpret_cast<SgListHandle*>(hh);
  cudaError_t e = sg_launch_cast_bf16(h->d_items, h->n, h->chunks, scale, shift, n_blocks, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  srpc_sg_list_destroy(hh);
  return e;
}
