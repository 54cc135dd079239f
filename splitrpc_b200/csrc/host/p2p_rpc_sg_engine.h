// Scatter-gather engines: move a request's fragments into its ring slot (gather)
// and a response out of its slot into transmit buffers (scatter).
//
// API and behaviour follow reference src/p2p_rpc_sg_engine.h:19-308: the list
// builders merge fragments that are adjacent in memory into one copy; the
// zero-copy engine only hands pointers over; the CPU engine copies with memcpy;
// the GPU engine (declared here, implemented in the CUDA half) drives copy
// kernels on the serving GPU.  Added: batch entry points, so that one kernel
// launch or doorbell round trip serves many requests, and a status code from
// every call because all waits are bounded.
#pragma once

#include <atomic>

#include "p2p_rpc_app.h"
#include "p2p_rpc_rr.h"

// Builds the copy list fragment -> contiguous app buffer.
static inline void gather_skbs(p2p_sk_buf* skb, const p2p_bufs* frags, uint8_t* app_buf) {
  uintptr_t dst = (uintptr_t)app_buf;
  size_t n = 0;
  uintptr_t run_end = 0;
  for (size_t i = 0; i < frags->num_items; i++) {
    uintptr_t src = frags->burst_items[i];
    size_t len = frags->item_size[i];
    if (n > 0 && src == run_end) {
      skb->len[n - 1] += len;
    } else {
      skb->i_buf[n] = src;
      skb->o_buf[n] = dst;
      skb->len[n] = len;
      n++;
    }
    run_end = src + len;
    dst += len;
  }
  skb->num_items = n;
}

// Builds the copy list contiguous app buffer -> fragments.
static inline void scatter_skbs(p2p_sk_buf* skb, const p2p_bufs* frags, uint8_t* app_buf) {
  uintptr_t src = (uintptr_t)app_buf;
  size_t n = 0;
  uintptr_t run_end = 0;
  for (size_t i = 0; i < frags->num_items; i++) {
    uintptr_t dst = frags->burst_items[i];
    size_t len = frags->item_size[i];
    if (n > 0 && dst == run_end) {
      skb->len[n - 1] += len;
    } else {
      skb->i_buf[n] = src;
      skb->o_buf[n] = dst;
      skb->len[n] = len;
      n++;
    }
    run_end = dst + len;
    src += len;
  }
  skb->num_items = n;
}

// Multi-tensor gather list.  A request is the concatenation of n_tensors tensors of sizes
// stub->input_tensor_size[k]; request number `batch_index` of a batch must land at
// stub->inputs[k] + batch_index * size[k], so that every input tensor of the batch is contiguous by itself
// (the layout g_params_v2 describes, reference src/p2p_rpc_app_stub.h:7-20, which the original never fills in:
// it batches by treating consecutive ring slots as one tensor, which is only right for single-input models).
// Fragments and tensor boundaries are walked together; adjacent pieces are merged.
static inline void gather_skbs_v2(p2p_sk_buf* skb, const p2p_bufs* frags, const g_params_v2* stub, int n_tensors,
                                  int batch_index) {
  size_t n = 0;
  int k = 0;
  size_t t_off = 0;  // bytes of tensor k already placed
  uintptr_t run_src_end = 0, run_dst_end = 0;
  for (size_t i = 0; i < frags->num_items && k < n_tensors; i++) {
    uintptr_t src = frags->burst_items[i];
    size_t left = frags->item_size[i];
    while (left > 0 && k < n_tensors) {
      size_t tsz = stub->input_tensor_size[k];
      size_t take = tsz - t_off < left ? tsz - t_off : left;
      uintptr_t dst = stub->inputs[k] + (uintptr_t)batch_index * tsz + t_off;
      if (take > 0) {
        if (n > 0 && src == run_src_end && dst == run_dst_end) {
          skb->len[n - 1] += take;
        } else if (n < MAX_BI_SIZE) {
          skb->i_buf[n] = src;
          skb->o_buf[n] = dst;
          skb->len[n] = take;
          n++;
        }
        run_src_end = src + take;
        run_dst_end = dst + take;
      }
      src += take;
      left -= take;
      t_off += take;
      if (t_off == tsz) {
        k++;
        t_off = 0;
      }
    }
  }
  skb->num_items = n;
}

struct SgCounters {
  uint64_t gathers = 0, scatters = 0, items = 0, bytes = 0, timeouts = 0;
};

enum { SG_TRANSFORM_NONE = 0, SG_TRANSFORM_STEM_S2D = 1 };

class P2pRpcSgEngine {
 public:
  int num_instances = 1;
  int device_id = -1;
  uint16_t app_queue_length = 0;
  SgCounters counters;
  int64_t sync_ticket_ = 0;
  volatile uint32_t *h_states_base_ = nullptr, *d_states_base_ = nullptr;
  volatile uint64_t *h_stamps_base_ = nullptr, *d_stamps_base_ = nullptr;
  PROF_DECL(Gather);
  PROF_DECL(Scatter);

  virtual ~P2pRpcSgEngine() {
    PROF_PRINT("Gather", Gather);
    PROF_PRINT("Scatter", Scatter);
  }
  // Return 0 on success, negative when a bounded wait ran out or the device failed.
  virtual int gather(P2pRpcRr* rr, g_params* stub) = 0;
  virtual int scatter(P2pRpcRr* rr, g_params* stub) = 0;
  // Raw-pointer forms kept for API parity; they treat the pointer as stub->req/resp.
  virtual int gather(P2pRpcRr* rr, uint8_t* req_buf) {
    g_params p{req_buf, nullptr};
    return gather(rr, &p);
  }
  virtual int scatter(P2pRpcRr* rr, uint8_t* resp_buf) {
    g_params p{nullptr, resp_buf};
    return scatter(rr, &p);
  }
  // Batch forms: default implementation loops; the GPU engine overrides them
  // with a single submission.
  virtual int gather_batch(P2pRpcRr** rrs, g_params** stubs, int n) {
    int rc = 0;
    for (int i = 0; i < n; i++) rc |= gather(rrs[i], stubs[i]);
    return rc;
  }
  virtual int scatter_batch(P2pRpcRr** rrs, g_params** stubs, int n) {
    int rc = 0;
    for (int i = 0; i < n; i++) rc |= scatter(rrs[i], stubs[i]);
    return rc;
  }
  // Gather that completes the slots by itself: once every byte of the n requests is in place, `state_value` is stored
  // (release) into each request's slot state, and the returned ticket (> 0) turns "done" (ticket_done).  The caller
  // must keep the fragments alive until then.  The GPU engine does all of this in one kernel launch without waiting
  // (d_states: the state words as the engine's GPU addresses them); this default does it synchronously on the calling
  // thread (h_states).  Negative return: failure, no state was stored.
  virtual int64_t gather_batch_notify(P2pRpcRr** rrs, g_params** stubs, volatile uint32_t** h_states,
                                      volatile uint32_t** d_states, int n, uint32_t state_value) {
    (void)d_states;
    int rc = gather_batch(rrs, stubs, n);
    if (rc != 0) return rc < 0 ? rc : -1;
    const uint64_t now = getCurNs();
    for (int i = 0; i < n; i++) {
      if (h_states_base_ && h_stamps_base_) h_stamps_base_[2 * (h_states[i] - h_states_base_)] = now;
      __atomic_store_n(h_states[i], state_value, __ATOMIC_RELEASE);
    }
    return ++sync_ticket_;
  }
  // Tells the engine where the slot ring it fills keeps its state words and its time stamps (host view and the view of
  // the engine's device), so that a gather can record when it rang each doorbell.  Optional.
  virtual void set_stamp_layout(volatile uint32_t* h_states_base, volatile uint64_t* h_stamps_base, volatile uint32_t* d_states_base,
                                volatile uint64_t* d_stamps_base) {
    h_states_base_ = h_states_base;
    h_stamps_base_ = h_stamps_base;
    d_states_base_ = d_states_base;
    d_stamps_base_ = d_stamps_base;
  }
  virtual bool ticket_done(int64_t ticket) {
    (void)ticket;
    return true;
  }
  // Makes gathers transform the payload on the way into the ring instead of copying it (GPU engine, copy type 2).
  // kind 0 = plain copy; SG_TRANSFORM_STEM_S2D = fp32 CHW image -> normalised bf16 space-to-depth tensor, params =
  // {mean[3], inv_std[3]}.  ring_base / slot_bytes describe the request ring.  Returns 0 when the engine supports it.
  virtual int set_gather_transform(int kind, uint64_t ring_base, uint32_t slot_bytes, const float* params) {
    (void)kind;
    (void)ring_base;
    (void)slot_bytes;
    (void)params;
    return -1;
  }
  // Executes an already built copy list.  Engines that cannot copy (zero copy) return -1.
  virtual int copy_list(const p2p_sk_buf* skb) {
    (void)skb;
    return -1;
  }
  // Multi-tensor gather of one request into slot `batch_index` of the per-tensor batch buffers.
  int gather_v2(P2pRpcRr* rr, const g_params_v2* stub, int n_tensors, int batch_index) {
    gather_skbs_v2(rr->payload_sk_bufs, rr->payload_bufs, stub, n_tensors, batch_index);
    counters.gathers++;
    return copy_list(rr->payload_sk_bufs);
  }
  virtual const char* name() const = 0;
};

// Zero copy: the app works directly on the first fragment's buffer and answers in
// place.  Only valid for single-fragment requests.
class P2pRpcSgZcEngine : public P2pRpcSgEngine {
 public:
  using P2pRpcSgEngine::gather;
  using P2pRpcSgEngine::scatter;
  int gather(P2pRpcRr* rr, g_params* stub) override {
    PROF_START(Gather);
    stub->req = (uint8_t*)rr->payload_bufs->burst_items[0];
    stub->resp = (uint8_t*)rr->payload_bufs->burst_items[0];
    std::atomic_thread_fence(std::memory_order_release);
    counters.gathers++;
    PROF_STOP(Gather);
    return 0;
  }
  int scatter(P2pRpcRr*, g_params*) override {
    counters.scatters++;
    return 0;
  }
  const char* name() const override { return "zc"; }
};

// CPU copies; the oracle for the GPU engines and the engine of the CPU device.
class P2pRpcSgCpuEngine : public P2pRpcSgEngine {
  int run(const p2p_sk_buf* skb) {
    for (size_t i = 0; i < skb->num_items; i++) {
      std::memcpy((void*)skb->o_buf[i], (const void*)skb->i_buf[i], skb->len[i]);
      counters.bytes += skb->len[i];
    }
    counters.items += skb->num_items;
    return 0;
  }

 public:
  using P2pRpcSgEngine::gather;
  using P2pRpcSgEngine::scatter;
  int gather(P2pRpcRr* rr, g_params* stub) override {
    PROF_START(Gather);
    gather_skbs(rr->payload_sk_bufs, rr->payload_bufs, stub->req);
    int rc = run(rr->payload_sk_bufs);
    std::atomic_thread_fence(std::memory_order_release);
    counters.gathers++;
    PROF_STOP(Gather);
    return rc;
  }
  int scatter(P2pRpcRr* rr, g_params* stub) override {
    PROF_START(Scatter);
    scatter_skbs(rr->payload_sk_bufs, rr->payload_bufs, stub->resp);
    int rc = run(rr->payload_sk_bufs);
    std::atomic_thread_fence(std::memory_order_release);
    counters.scatters++;
    PROF_STOP(Scatter);
    return rc;
  }
  int copy_list(const p2p_sk_buf* skb) override { return run(skb); }
  // the original's name and return convention (1 = done; reference src/p2p_rpc_sg_engine.h:139-145)
  int sg_on_cpu(p2p_sk_buf* skb) { return run(skb) == 0 ? 1 : 0; }
  const char* name() const override { return "cpu"; }
};

// Stand-alone helpers on flat buffers (reference src/p2p_rpc_sg_engine.h:315-361).
static inline void gather_payload_on_cpu(const p2p_bufs* frags, uint8_t* dst) {
  for (size_t i = 0; i < frags->num_items; i++) {
    std::memcpy(dst, (const void*)frags->burst_items[i], frags->item_size[i]);
    dst += frags->item_size[i];
  }
}
static inline void scatter_payload_on_cpu(const p2p_bufs* frags, const uint8_t* src) {
  for (size_t i = 0; i < frags->num_items; i++) {
    std::memcpy((void*)frags->burst_items[i], src, frags->item_size[i]);
    src += frags->item_size[i];
  }
}

// GPU engine factory, implemented by the CUDA half.  copy_type follows
// P2P_RPC_GPU_COPY_TYPE: 0 copy-engine DMA per run, 1 persistent kernel behind a
// doorbell, 2 one kernel launch per submission.
extern "C" P2pRpcSgEngine* srpc_make_gpu_sg_engine(int device_id, int copy_type);
