// Device side of "the serving GPU answers by itself": where a response goes and how its slot is completed.
//
// A kernel that produces the response of request `row` of the running batch asks resp_push_target() for the
// destination (the producer's transmit arena when the producer named an offset for the slot, otherwise the response
// ring) and, after all its stores, has ONE thread call resp_push_complete(), which publishes WORK_COMPLETE in the
// slot's state word with a system-scope release store.  The arena may be pinned host memory of another process or a
// peer GPU's memory; the fence before the store makes the bytes visible there before the state is.
// In the original this hand-off takes a host thread, a SEND_WITH_IMM and an RDMA READ per response (reference
// src/splitrpc_rdma_transport/gpu_rdma_batched_server.cc:441-458, gpu_dpdk_rdma_proxy_handler.cc:249-296).
#pragma once

#include "../host/p2p_rpc_app.h"
#include "ptx.cuh"

struct RespPushTarget {
  uint8_t* dst;
  volatile uint32_t* state;  // nullptr: completion is left to the host
  volatile uint64_t* stamp;  // where the completion time goes (may be nullptr)
};

// The push block, the slots' destinations and their state words live in host memory that several processes map: a
// read costs a PCIe round trip.  Call this from ONE thread per response and hand the result to the others through
// shared memory (resp_push_target_block does that); thousands of threads reading it at once cost more than the
// softmax they belong to.
__device__ __forceinline__ RespPushTarget resp_push_target(const RespPushCtx* ctx_, uint32_t row, uint8_t* ring_dst) {
  // volatile: a resident kernel looks at the block once per batch and must see what the host wrote since the last one
  const volatile RespPushCtx* ctx = ctx_;
  RespPushTarget t{ring_dst, nullptr, nullptr};
  if (!ctx || ctx->enabled == 0 || ctx->pool_size == 0) return t;
  const uint32_t slot = (ctx->first_slot + row) % ctx->pool_size;
  const uint64_t* win = ctx->tx_window;
  const uint64_t off = win ? win[row] : ctx->tx_off[slot];
  if (ctx->tx_base && off != ~0ull && off + ctx->resp_size <= ctx->tx_bytes) t.dst = reinterpret_cast<uint8_t*>(ctx->tx_base + off);
  t.state = ctx->states + slot;
  t.stamp = ctx->stamps ? ctx->stamps + 2 * slot + 1 : nullptr;
  return t;
}

// Block-wide form: thread 0 looks the target up, everybody gets it.  Contains __syncthreads(): call it from all
// threads of the block, outside divergent code.
__device__ __forceinline__ RespPushTarget resp_push_target_block(const RespPushCtx* ctx, uint32_t row, uint8_t* ring_dst) {
  __shared__ RespPushTarget s_target;
  if (threadIdx.x == 0) s_target = resp_push_target(ctx, row, ring_dst);
  __syncthreads();
  return s_target;
}

// Call from one thread, after a __syncthreads() that follows every store of the response by the block.
__device__ __forceinline__ void resp_push_complete(const RespPushTarget& t) {
  if (!t.state) return;
  if (t.stamp) *t.stamp = ptx::globaltimer_ns();
  __threadfence_system();
  ptx::st_release_sys(t.state, (uint32_t)APP_RR_STATUS::WORK_COMPLETE);
}

// Stores the `batch` responses that one block has just produced at resp (resp_size apart) and completes their slots,
// one after the other.  For kernels that serve a whole batch with one block (resident apps).  Call from all threads.
__device__ __forceinline__ void resp_push_rows_block(const RespPushCtx* ctx, uint8_t* resp, uint32_t resp_size, int batch) {
  if (!ctx) return;
  for (int r = 0; r < batch; r++) {
    uint8_t* src = resp + (size_t)r * resp_size;
    const RespPushTarget t = resp_push_target_block(ctx, (uint32_t)r, src);
    if (t.dst != src)
      for (uint32_t i = threadIdx.x; i < resp_size; i += blockDim.x) t.dst[i] = src[i];
    __syncthreads();
    if (threadIdx.x == 0) resp_push_complete(t);
    __syncthreads();
  }
}
