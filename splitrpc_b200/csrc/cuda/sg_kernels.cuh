// Scatter-gather copy kernels and their launch API.
//
// A copy list is an array of SgItem {src, dst, len}; the list is cut into chunks
// of SG_CHUNK bytes and chunks are spread over thread blocks, so one launch moves
// every fragment run of a whole batch of requests.  Sources and destinations may
// be local HBM, mapped pinned host memory (the receive/transmit arenas) or a peer
// GPU's memory reached over NVLink.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

static constexpr uint32_t SG_CHUNK = 16384;
static constexpr uint32_t SG_MAX_ITEMS = 8192;        // per launch
static constexpr uint32_t SG_PERSISTENT_ITEMS = 1024;  // per doorbell ring of the resident engine

struct SgItem {
  uint64_t src;
  uint64_t dst;
  uint32_t len;
  uint32_t first_chunk;  // index of this item's first chunk in the launch-wide chunk numbering
};

// Control block of the persistent engine; lives in mapped pinned host memory.
struct SgCtrl {
  volatile uint32_t doorbell;   // host: sequence number of the newest submission
  volatile uint32_t done;       // device: sequence number of the newest finished submission
  volatile uint32_t exit_flag;  // host: 1 asks the kernel to leave
  volatile uint32_t exited;     // device: number of thread blocks that have left
  volatile uint32_t n_items;
  volatile uint32_t n_chunks;
  volatile uint32_t error;      // device: non-zero when a bounded wait ran out
  uint32_t _pad;
  uint64_t idle_limit_ns;       // a block leaves after this long without new work
  SgItem items[SG_PERSISTENT_ITEMS];
};

enum SgImpl { SG_IMPL_SIMT = 0, SG_IMPL_BULK = 1 };

// Optional epilogue of a copy launch: when the last block has finished (arrival counter), it stores `bell_value` into
// each of the n_bells 32-bit words whose addresses are listed in `bells`, then `done_value` into `done_word`, all with
// system-scope release stores that follow a system-scope fence.  The words may live in mapped host memory or in
// another GPU's memory: this is how a gather rings the doorbells of the slots it filled (payload first, doorbell
// second, the order the original gets from chaining an RDMA WRITE of the payload with one of the doorbell, reference
// src/splitrpc_rdma_transport/p2p_rpc_bf_rr_pool.h:107-152) without a host thread in between.  counter == nullptr: no
// epilogue.  The counter must be zero at launch; the last block leaves it at zero.
struct SgNotify {
  uint32_t* counter = nullptr;
  const uint64_t* bells = nullptr;  // device-readable list of addresses
  uint32_t n_bells = 0;
  uint32_t bell_value = 0;
  uint32_t* done_word = nullptr;
  uint32_t done_value = 0;
  // When set: the bells are the state words of one slot ring that starts at states_base, and the time at which they
  // are rung (this GPU's nanosecond timer) goes into stamps_base[2 * slot] for each of them.
  uint64_t states_base = 0;
  uint64_t stamps_base = 0;
};

// One launch over a copy list that the device can read (device or mapped memory).
cudaError_t sg_launch_copy(const SgItem* d_items, uint32_t n_items, uint32_t n_chunks, int impl, int n_blocks,
                           cudaStream_t stream, const SgNotify* notify = nullptr);
// Stores the responses of a batch where the producer asked for them and completes their slots (see resp_push.cuh):
// one block per response.  d_stub / d_push are the device views of the app's stub and RespPushCtx.
cudaError_t sg_launch_resp_push(const void* d_stub, const void* d_push, int n, cudaStream_t stream);
// See SrpcDeviceOps::window_params.
struct g_params;
struct RespPushCtx;
cudaError_t sg_launch_window_params(void* block, const g_params* stub, const RespPushCtx* ctx, const uint64_t* offsets, int n,
                                    const uint32_t* live_enabled, cudaStream_t stream);
// fp32 -> bf16 gather: every item copies len/4 floats to len/4 bf16 values,
// computing (x - shift) * scale on the way.
cudaError_t sg_launch_cast_bf16(const SgItem* d_items, uint32_t n_items, uint32_t n_chunks, float scale, float shift,
                                int n_blocks, cudaStream_t stream);
// Gather fused with the ResNet stem's deserialisation (fp32 CHW fragments -> normalised bf16 space-to-depth tensor in
// the ring slot).  ring_base / slot_bytes describe the request ring that the items' destinations point into.
struct SgStemS2d {
  uint64_t ring_base;
  uint32_t slot_bytes;
  float mean[3];
  float inv_std[3];
};
cudaError_t sg_launch_stem_s2d(const SgItem* d_items, uint32_t n_items, uint32_t n_chunks, const SgStemS2d& tr, int n_blocks,
                               cudaStream_t stream, const SgNotify* notify = nullptr);
// Loads this file's kernels on the current device (idempotent).  Call it before any stream of the device may be parked
// on a doorbell: a kernel's first launch can otherwise block behind that stream (lazy module loading).
void sg_preload_kernels();
// Persistent engine: `counter` is a zero-initialised device word.
cudaError_t sg_launch_persistent(SgCtrl* d_ctrl, uint32_t* d_counter, int n_blocks, cudaStream_t stream);

// Host helper: fills first_chunk and returns the chunk count.
static inline uint32_t sg_assign_chunks(SgItem* items, uint32_t n) {
  uint32_t c = 0;
  for (uint32_t i = 0; i < n; i++) {
    items[i].first_chunk = c;
    c += (items[i].len + SG_CHUNK - 1) / SG_CHUNK;
  }
  return c;
}
static_assert(sizeof(SgItem) == 24, "three 8-byte words");
