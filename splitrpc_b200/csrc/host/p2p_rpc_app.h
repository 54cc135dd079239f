// App-side runtime: stub, device abstraction, ring memory, request slots, app context.
//
// What an app sees of a call is a g_params stub {req, resp} that points into the
// request and response rings (reference src/p2p_rpc_app_stub.h:11-29).  The rings
// are mapped twice back to back in virtual memory, so a batch of consecutive
// slots is contiguous even when it crosses the end of the ring (reference
// src/p2p_rpc_app_rr_mem_pool.h:213-339).  Each slot has a 32-bit state word
// (FREE -> RX_COMPLETE -> WORK_COMPLETE -> TX_COMPLETE) that doubles as the
// doorbell a GPU stream can wait on.
//
// The host core never calls CUDA directly: everything device-specific goes
// through the SrpcDeviceOps table, which the CUDA half of the library fills in.
// device_id < 0 selects the CPU "device" (memfd double mapping, synchronous
// execution), which is what the GPU-less plumbing configuration runs on.
#pragma once

#include <sys/mman.h>
#include <unistd.h>

#include <climits>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <vector>

#include "config_utils.h"

typedef struct CUstream_st* cudaStream_t;
typedef struct CUevent_st* cudaEvent_t;
typedef struct CUgraph_st* cudaGraph_t;
typedef struct CUgraphExec_st* cudaGraphExec_t;

// ------------------------------------------------------------------ stubs
#define MAX_NUM_TENSORS 4
// Multi-tensor form: each input tensor of a batch is contiguous by itself.
struct g_params_v2 {
  uintptr_t inputs[MAX_NUM_TENSORS];
  uintptr_t outputs[MAX_NUM_TENSORS];
  size_t input_tensor_size[MAX_NUM_TENSORS];
  size_t output_tensor_size[MAX_NUM_TENSORS];
} __attribute__((packed));

struct g_params {
  uint8_t* req;
  uint8_t* resp;
} __attribute__((packed));

static constexpr uint32_t APP_DOORBELL_START = 0x40000000u;
static constexpr uint32_t APP_DOORBELL_IDLE = 0xFFFFFFFFu;
static constexpr uint32_t APP_DOORBELL_RUN_DONE = 1u;   // written from the stream after a run
static constexpr uint32_t APP_DOORBELL_PT_DONE = 2u;    // written by a resident kernel after a batch
static constexpr uint32_t APP_DOORBELL_EXIT = 3u;       // asks a resident kernel to leave

// RX_DESCRIBED: the slot's request has not been moved yet; its fragment list sits in the slot's descriptor block and
// the serving side fetches the bytes itself (over its own link to host memory), then marks the slot RX_COMPLETE.
enum APP_RR_STATUS : uint32_t { FREE = 0, RX_COMPLETE = 1, WORK_COMPLETE = 2, TX_COMPLETE = 3, RX_DESCRIBED = 4 };

// Where the fragments of a described request are: `where` = region index << 56 | byte offset inside that region (the
// regions are the host memory ranges that the producer shared at ALLOC time: its receive arena and the buffers that
// senders hand over by reference); the bytes go to request offset dst_off.
struct SrpcFragDesc {
  uint64_t where;
  uint32_t len;
  uint32_t dst_off;
};
struct SrpcSlotDesc {
  uint32_t n_frags;
  uint32_t pad_[3];
  SrpcFragDesc frag[1];  // desc_per_slot entries follow
};
static inline uint32_t srpc_desc_per_slot(size_t req_size) {
  size_t n = req_size / 1024 + 3;
  return (uint32_t)(n > 1024 ? 1024 : n);
}
static inline size_t srpc_desc_stride(size_t req_size) { return 16 + (size_t)srpc_desc_per_slot(req_size) * sizeof(SrpcFragDesc); }

// What the serving side needs to answer a slot by itself: for the batch whose first slot is `first_slot`, request r
// belongs to slot (first_slot + r) % pool_size; its response goes to tx_base + tx_off[slot] (unless tx_off is
// kNoTxOffset: then it stays in the response ring) and states[slot] becomes WORK_COMPLETE with a system-scope release
// store once the bytes are written.  The block sits in memory that kernels read when they run (mapped pinned memory),
// so graphs captured before the transmit arena is known pick the values up later.  enabled == 0: kernels leave
// completion to the host.  This replaces the original's "host sends SEND_WITH_IMM(slot), proxy RDMA-READs the
// response" exchange (reference src/splitrpc_rdma_transport/gpu_rdma_batched_server.cc:441-458) by stores from the
// GPU that computed the response.
struct RespPushCtx {
  uint64_t tx_base;                 // device-side address of the ingress transmit arena in the serving process
  uint64_t tx_bytes;
  const volatile uint64_t* tx_off;  // per slot, device view
  volatile uint32_t* states;        // per slot, device view
  volatile uint64_t* stamps;        // per slot {doorbell rung, response stored} device timer values (ns), device view
  uint32_t pool_size;
  uint32_t resp_size;
  uint32_t enabled;
  uint32_t first_slot;              // written by the worker with the stub, before every run
  // Optional: the transmit offsets of the running batch, request r at tx_window[r], already looked up and placed in
  // the serving GPU's own memory (see SrpcDeviceOps::window_params).  nullptr: kernels read tx_off[slot].
  const uint64_t* tx_window;
};

// A GPU app's kernels take the stub and the push block from a small block in the GPU's own memory, laid out as
// below and rewritten in stream order before every batch.  (A read of mapped host memory by a kernel crosses PCIe;
// a kernel whose every block does a dozen of them spends longer on that than on its work.)
static constexpr size_t APP_PARAM_BLOCK_BYTES = 4096;
static constexpr size_t APP_PARAM_PUSH_OFFSET = 64;     // RespPushCtx
static constexpr size_t APP_PARAM_WINDOW_OFFSET = 256;  // tx_window[]
static constexpr int APP_PARAM_WINDOW_MAX = (int)((APP_PARAM_BLOCK_BYTES - APP_PARAM_WINDOW_OFFSET) / 8);
static constexpr int APP_PARAM_INLINE_MAX = 112;        // offsets that fit the kernel's argument space

// ------------------------------------------------------------------ tring
// Bump-pointer address generator over a ring-shaped address range (reference
// src/p2p_rpc_tring.h:10-34): get_next(n) returns the current address and
// advances by n modulo the capacity.
class P2pRpcTring {
  uintptr_t base_;
  size_t capacity_;
  size_t offset_ = 0;

 public:
  P2pRpcTring(void* base, size_t capacity) : base_((uintptr_t)base), capacity_(capacity) {}
  void* get_next(size_t size) {
    void* ret = (void*)(base_ + offset_);
    offset_ = (offset_ + size) % capacity_;
    return ret;
  }
  size_t offset() const { return offset_; }
  size_t capacity() const { return capacity_; }
  void* base() const { return (void*)base_; }
  void reset() { offset_ = 0; }
};

// ------------------------------------------------------------------ device ops
struct SrpcRingMem {
  void* base = nullptr;      // start of the (double) mapping
  size_t capacity = 0;       // bytes of physical ring (mapping covers 2x when double_mapped)
  bool double_mapped = false;
  void* impl = nullptr;      // backend bookkeeping
  int fd = -1;               // host rings: the memfd behind the mapping (kept open so the ring can be exported)
};

// Host memory that several processes map (a memfd) and that, on a GPU build, every one of them registers with CUDA, so
// that the CPU threads and the GPUs of all those processes address the same words: slot doorbells, response
// destinations, transmit arenas.  `dev` is this process's device-side address of `host`.
struct SrpcSharedMem {
  void* host = nullptr;
  void* dev = nullptr;
  size_t bytes = 0;
  int fd = -1;
  bool registered = false;
};

struct SrpcDeviceOps {
  int (*device_count)();
  int (*set_device)(int dev);
  int (*stream_create)(int dev, cudaStream_t* s);
  int (*stream_destroy)(cudaStream_t s);
  int (*stream_sync)(cudaStream_t s);
  int (*stream_query)(cudaStream_t s);  // 0 = idle, 1 = busy, <0 error
  int (*stream_wait_value32)(cudaStream_t s, volatile uint32_t* d_addr, uint32_t value);
  int (*stream_write_value32)(cudaStream_t s, volatile uint32_t* d_addr, uint32_t value);
  int (*event_create)(cudaEvent_t* e);
  int (*event_destroy)(cudaEvent_t e);
  // Capacity = min_bytes rounded up to a multiple of both the allocation granularity and slot_bytes, so that the
  // ring's address generator wraps on a slot boundary and every slot starts at a multiple of slot_bytes.
  int (*ring_alloc)(int dev, size_t min_bytes, size_t slot_bytes, bool peer_access, SrpcRingMem* out);
  int (*ring_free)(SrpcRingMem* m);
  int (*host_alloc_mapped)(size_t bytes, void** host_ptr, void** dev_ptr);
  int (*host_free)(void* host_ptr);
  int (*dev_alloc)(int dev, size_t bytes, void** p);
  int (*dev_free)(void* p);
  int (*memcpy_async)(void* dst, const void* src, size_t n, cudaStream_t s);
  int (*memset_async)(void* dst, int v, size_t n, cudaStream_t s);
  int (*graph_launch)(cudaGraphExec_t g, cudaStream_t s);
  const char* (*last_error)();
  // Sharing with another process on the same machine.  ring_export returns a file descriptor for the physical
  // allocation of a ring made by ring_alloc (the caller closes it); ring_import maps such an allocation (twice, like
  // its owner does) into this process and gives `dev` read/write access to it.  host_register pins an existing host
  // mapping (a memfd that the peer process maps too) and returns its device-side address.
  int (*ring_export)(const SrpcRingMem* m, int* fd);
  int (*ring_import)(int dev, int fd, size_t capacity, SrpcRingMem* out);
  int (*host_register)(void* p, size_t bytes, void** dptr);
  int (*host_unregister)(void* p);
  // Queues, on `s`, the kernel that stores the `n` responses of the window at *d_stub where *d_push says and marks
  // their slots WORK_COMPLETE (see RespPushCtx).
  int (*resp_push)(const void* d_stub, const void* d_push, int n, cudaStream_t s);
  // Device `dev`'s nanosecond timer (what its kernels stamp slots with) minus this machine's steady clock, measured
  // now.  The timers of two GPUs differ by an arbitrary amount; a latency that starts on one GPU and ends on another
  // is the difference of the stamps minus the difference of these offsets.
  int (*timer_offset_ns)(int dev, int64_t* offset);
  // Queues, on `s`, a one-block kernel that rewrites the parameter block `block` (device memory, see
  // APP_PARAM_BLOCK_BYTES) with *stub, *ctx and the transmit offsets of a batch of `n` requests: `offsets[0..n)` when
  // `offsets` is given (n <= APP_PARAM_INLINE_MAX; the values travel in the launch), otherwise read from
  // ctx->tx_off[(first_slot + r) % pool_size] when the kernel runs (n <= APP_PARAM_WINDOW_MAX).  `live_enabled`
  // (optional, device view of a host word): a zero found there when the kernel runs switches the push off.
  int (*window_params)(void* block, const g_params* stub, const RespPushCtx* ctx, const uint64_t* offsets, int n,
                       const uint32_t* live_enabled, cudaStream_t s);
};

// Implemented by the CUDA half; returns nullptr when the library was built
// without it.
extern "C" const SrpcDeviceOps* srpc_cuda_ops();

static inline const SrpcDeviceOps* srpc_require_cuda(const char* what) {
  const SrpcDeviceOps* ops = srpc_cuda_ops();
  if (!ops) {
    srpc_log(SRPC_LOG_ERROR, "%s needs the CUDA half of the library, which is not available", what);
    std::abort();
  }
  return ops;
}

// ------------------------------------------------------------------ ring memory
static inline size_t find_lcm(size_t a, size_t b) { return a / std::gcd(a, b) * b; }

// Host ring mapped twice back to back with memfd + MAP_FIXED.
// Ring capacity: min_bytes rounded up to a multiple of lcm(granularity, slot_bytes).  A ring that wrapped in the
// middle of a slot would still give contiguous windows (double mapping), but slots would stop being aligned to
// slot_bytes after the first lap, and kernels that address the ring by slot index would read the wrong bytes.
static inline size_t srpc_ring_capacity(size_t min_bytes, size_t slot_bytes, size_t gran) {
  size_t unit = slot_bytes ? find_lcm(gran, slot_bytes) : gran;
  if (unit > ((size_t)4 << 30)) unit = gran;  // pathological slot size: keep the plain rounding
  size_t cap = (min_bytes + unit - 1) / unit * unit;
  return cap ? cap : unit;
}

static inline bool srpc_host_ring_alloc(size_t min_bytes, size_t slot_bytes, SrpcRingMem* out) {
  size_t page = (size_t)sysconf(_SC_PAGESIZE);
  size_t cap = srpc_ring_capacity(min_bytes, slot_bytes, page);
  int fd = memfd_create("splitrpc_ring", 0);
  if (fd < 0) return false;
  if (ftruncate(fd, (off_t)cap) != 0) {
    close(fd);
    return false;
  }
  void* va = mmap(nullptr, 2 * cap, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (va == MAP_FAILED) {
    close(fd);
    return false;
  }
  void* a = mmap(va, cap, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0);
  void* b = mmap((uint8_t*)va + cap, cap, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0);
  if (a == MAP_FAILED || b == MAP_FAILED) {
    close(fd);
    munmap(va, 2 * cap);
    return false;
  }
  out->base = va;
  out->capacity = cap;
  out->double_mapped = true;
  out->impl = nullptr;
  out->fd = fd;
  return true;
}
// Maps a host ring that another process created (its memfd arrived over a control channel).  Takes ownership of fd.
static inline bool srpc_host_ring_import(int fd, size_t cap, SrpcRingMem* out) {
  void* va = mmap(nullptr, 2 * cap, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (va == MAP_FAILED) return false;
  void* a = mmap(va, cap, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0);
  void* b = mmap((uint8_t*)va + cap, cap, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0);
  if (a == MAP_FAILED || b == MAP_FAILED) {
    munmap(va, 2 * cap);
    return false;
  }
  out->base = va;
  out->capacity = cap;
  out->double_mapped = true;
  out->impl = nullptr;
  out->fd = fd;
  return true;
}
static inline void srpc_host_ring_free(SrpcRingMem* m) {
  if (m->base) munmap(m->base, 2 * m->capacity);
  if (m->fd >= 0) close(m->fd);
  m->base = nullptr;
  m->fd = -1;
}

// Shared host memory: create (memfd) or import (an fd that arrived from the creator), then optionally register it
// with CUDA.  `with_cuda` needs the CUDA half of the library.
static inline bool srpc_shm_map(int fd, size_t bytes, bool with_cuda, SrpcSharedMem* out) {
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) return false;
  out->host = out->dev = p;
  out->bytes = bytes;
  out->fd = fd;
  out->registered = false;
  if (with_cuda) {
    const SrpcDeviceOps* ops = srpc_cuda_ops();
    void* d = nullptr;
    if (!ops || ops->host_register(p, bytes, &d) != 0) {
      munmap(p, bytes);
      out->host = out->dev = nullptr;
      return false;
    }
    out->dev = d;
    out->registered = true;
  }
  return true;
}
static inline bool srpc_shm_create(size_t min_bytes, bool with_cuda, SrpcSharedMem* out) {
  size_t page = (size_t)sysconf(_SC_PAGESIZE);
  size_t bytes = (min_bytes + page - 1) / page * page;
  int fd = memfd_create("splitrpc_shm", 0);
  if (fd < 0) return false;
  if (ftruncate(fd, (off_t)bytes) != 0 || !srpc_shm_map(fd, bytes, with_cuda, out)) {
    close(fd);
    return false;
  }
  return true;
}
// Takes ownership of fd on success.
static inline bool srpc_shm_import(int fd, size_t bytes, bool with_cuda, SrpcSharedMem* out) {
  return srpc_shm_map(fd, bytes, with_cuda, out);
}
static inline void srpc_shm_free(SrpcSharedMem* m) {
  if (!m->host) return;
  if (m->registered)
    if (const SrpcDeviceOps* ops = srpc_cuda_ops()) ops->host_unregister(m->host);
  munmap(m->host, m->bytes);
  if (m->fd >= 0) close(m->fd);
  *m = SrpcSharedMem{};
}

// What one process tells another about the rings of an app so that the other can produce into them: three file
// descriptors (request ring, response ring, control block) and the geometry.  This is the NVLink-era form of the three
// remotely writable memory regions {address, length, key} that the original's batched server registers and hands to
// its SmartNIC proxy (reference src/splitrpc_rdma_transport/gpu_rdma_batched_server.cc:326-352).
struct AppRrPoolExport {
  int req_fd = -1, resp_fd = -1, ctl_fd = -1;
  uint64_t req_capacity = 0, resp_capacity = 0, ctl_bytes = 0;
  uint32_t pool_size = 0;
  int32_t owner_device = -1;
  uint64_t req_size = 0, resp_size = 0;
};

// Request ring, response ring and per-slot control words of one app.
// On a GPU the rings are CUDA virtual-memory allocations mapped twice (and made
// accessible to every peer GPU when `peer_access` is set); the control block lives
// in mapped pinned host memory so that the host can poll it and a GPU stream
// (or a peer GPU) can wait on or write it.  The control block holds, per slot, the
// 32-bit state word (the doorbell) and a 64-bit response destination: the offset
// in the ingress transmit arena where the serving side stores the slot's response
// (kNoTxOffset = the response stays in the response ring).
// A pool is either the owner of its memory or a mirror of a pool that another
// process owns (import constructor): the mirror maps the same rings and the same
// control block, which is what lets a producer in another process fill slots and
// ring doorbells without the owner's CPU.
class P2pRpcAppRrMemPool {
  int device_id_;
  SrpcRingMem req_{}, resp_{};
  SrpcSharedMem ctl_{};
  volatile uint32_t* h_doorbells_ = nullptr;
  volatile uint32_t* d_doorbells_ = nullptr;
  volatile uint64_t* h_tx_off_ = nullptr;
  volatile uint64_t* d_tx_off_ = nullptr;
  volatile uint64_t* h_stamps_ = nullptr;  // per slot: [0] when the gather rang the doorbell, [1] when the response was stored
  volatile uint64_t* d_stamps_ = nullptr;
  size_t n_doorbells_ = 0;
  bool mirror_ = false;
  bool ctl_plain_ = false;  // control block from host_alloc_mapped / posix_memalign instead of a memfd
  size_t req_size_ = 0;
  uint8_t* h_desc_ = nullptr;  // per slot: SrpcSlotDesc (host view; only the hosts of both sides touch it)

  // states | transmit offsets | stamps | fragment descriptors
  static size_t ctl_layout(size_t n, size_t req_size, size_t* tx_off_at, size_t* stamps_at = nullptr, size_t* desc_at = nullptr) {
    size_t a = (n * sizeof(uint32_t) + 63) / 64 * 64;
    *tx_off_at = a;
    size_t b = a + n * sizeof(uint64_t);
    if (stamps_at) *stamps_at = b;
    size_t c = (b + 2 * n * sizeof(uint64_t) + 63) / 64 * 64;
    if (desc_at) *desc_at = c;
    return c + n * srpc_desc_stride(req_size);
  }
  void bind_ctl(void* h, void* d) {
    size_t at = 0, st = 0, ds = 0;
    ctl_layout(n_doorbells_, req_size_, &at, &st, &ds);
    h_desc_ = (uint8_t*)h + ds;
    h_doorbells_ = (volatile uint32_t*)h;
    d_doorbells_ = (volatile uint32_t*)d;
    h_tx_off_ = (volatile uint64_t*)((uint8_t*)h + at);
    d_tx_off_ = (volatile uint64_t*)((uint8_t*)d + at);
    h_stamps_ = (volatile uint64_t*)((uint8_t*)h + st);
    d_stamps_ = (volatile uint64_t*)((uint8_t*)d + st);
  }

 public:
  static constexpr uint64_t kNoTxOffset = ~0ull;

  P2pRpcAppRrMemPool(int pool_size, int device_id, size_t req_size, size_t resp_size, bool peer_access = true)
      : device_id_(device_id), n_doorbells_((size_t)pool_size), req_size_(req_size) {
    size_t req_bytes = (size_t)pool_size * req_size, resp_bytes = (size_t)pool_size * resp_size;
    size_t at = 0, ctl_bytes = ctl_layout(n_doorbells_, req_size_, &at);
    if (device_id < 0) {
      if (!srpc_host_ring_alloc(req_bytes, req_size, &req_) || !srpc_host_ring_alloc(resp_bytes, resp_size, &resp_)) {
        srpc_log(SRPC_LOG_ERROR, "host ring allocation failed (%zu + %zu bytes)", req_bytes, resp_bytes);
        std::abort();
      }
      if (!srpc_shm_create(ctl_bytes, false, &ctl_)) std::abort();
    } else {
      const SrpcDeviceOps* ops = srpc_require_cuda("a GPU request ring");
      if (ops->ring_alloc(device_id, req_bytes, req_size, peer_access, &req_) != 0 ||
          ops->ring_alloc(device_id, resp_bytes, resp_size, peer_access, &resp_) != 0) {
        srpc_log(SRPC_LOG_ERROR, "GPU ring allocation failed: %s", ops->last_error());
        std::abort();
      }
      ops->set_device(device_id);
      if (!srpc_shm_create(ctl_bytes, true, &ctl_)) {
        // No memfd or no registration of foreign mappings: a private pinned block (the pool cannot be exported).
        void *h = nullptr, *d = nullptr;
        if (ops->host_alloc_mapped(ctl_bytes, &h, &d) != 0) std::abort();
        ctl_.host = h;
        ctl_.dev = d;
        ctl_.bytes = ctl_bytes;
        ctl_plain_ = true;
      }
    }
    bind_ctl(ctl_.host, ctl_.dev);
    for (size_t i = 0; i < n_doorbells_; i++) {
      h_doorbells_[i] = APP_RR_STATUS::FREE;
      h_tx_off_[i] = kNoTxOffset;
      h_stamps_[2 * i] = h_stamps_[2 * i + 1] = 0;
    }
  }

  // Mirror of a pool owned by another process.  `device_id` is the device whose kernels will write the rings (the
  // ingress GPU), or -1 when the CPU does.  Takes ownership of the descriptors in `ex`.
  P2pRpcAppRrMemPool(const AppRrPoolExport& ex, int device_id)
      : device_id_(device_id), n_doorbells_(ex.pool_size), mirror_(true), req_size_(ex.req_size) {
    bool ok;
    {
      size_t at = 0;
      if (ctl_layout(n_doorbells_, req_size_, &at) > ex.ctl_bytes) {  // the owner's mapping is rounded up to pages
        srpc_log(SRPC_LOG_ERROR, "control block of a remote app is smaller than its layout");
        ::close(ex.req_fd);
        ::close(ex.resp_fd);
        ::close(ex.ctl_fd);
        n_doorbells_ = 0;
        return;
      }
    }
    if (ex.owner_device < 0) {
      ok = srpc_host_ring_import(ex.req_fd, ex.req_capacity, &req_) && srpc_host_ring_import(ex.resp_fd, ex.resp_capacity, &resp_);
    } else {
      const SrpcDeviceOps* ops = srpc_require_cuda("importing a GPU request ring");
      ok = device_id >= 0 && ops->ring_import(device_id, ex.req_fd, ex.req_capacity, &req_) == 0 &&
           ops->ring_import(device_id, ex.resp_fd, ex.resp_capacity, &resp_) == 0;
      if (!ok) srpc_log(SRPC_LOG_ERROR, "ring import failed: %s", ops->last_error());
    }
    if (ok && device_id >= 0) srpc_require_cuda("importing a control block")->set_device(device_id);
    ok = ok && srpc_shm_import(ex.ctl_fd, ex.ctl_bytes, device_id >= 0, &ctl_);
    if (!ok) {
      srpc_log(SRPC_LOG_ERROR, "could not map the rings of a remote app");
      n_doorbells_ = 0;
      return;
    }
    bind_ctl(ctl_.host, ctl_.dev);
  }

  ~P2pRpcAppRrMemPool() {
    const SrpcDeviceOps* ops = srpc_cuda_ops();
    bool gpu_rings = mirror_ ? (req_.impl != nullptr) : device_id_ >= 0;
    if (!gpu_rings) {
      srpc_host_ring_free(&req_);
      srpc_host_ring_free(&resp_);
    } else if (ops) {
      ops->ring_free(&req_);
      ops->ring_free(&resp_);
    }
    if (ctl_plain_) {
      if (ops) ops->host_free(ctl_.host);
    } else {
      srpc_shm_free(&ctl_);
    }
  }
  P2pRpcAppRrMemPool(const P2pRpcAppRrMemPool&) = delete;

  bool ok() const { return n_doorbells_ > 0 && req_.base && resp_.base; }
  bool is_mirror() const { return mirror_; }
  bool exportable() const { return !mirror_ && !ctl_plain_ && ctl_.fd >= 0; }
  // Fills `ex` with freshly duplicated descriptors (the caller sends and closes them).  false when this pool cannot
  // be shared (no memfd-backed control block, or the driver refused to export the rings).
  bool export_to(AppRrPoolExport* ex, size_t req_size, size_t resp_size) const {
    if (!exportable()) return false;
    ex->ctl_fd = dup(ctl_.fd);
    ex->ctl_bytes = ctl_.bytes;
    if (device_id_ < 0) {
      ex->req_fd = dup(req_.fd);
      ex->resp_fd = dup(resp_.fd);
    } else {
      const SrpcDeviceOps* ops = srpc_require_cuda("ring export");
      if (ops->ring_export(&req_, &ex->req_fd) != 0 || ops->ring_export(&resp_, &ex->resp_fd) != 0) {
        srpc_log(SRPC_LOG_ERROR, "ring export failed: %s", ops->last_error());
        return false;
      }
    }
    ex->req_capacity = req_.capacity;
    ex->resp_capacity = resp_.capacity;
    ex->pool_size = (uint32_t)n_doorbells_;
    ex->owner_device = device_id_;
    ex->req_size = req_size;
    ex->resp_size = resp_size;
    return ex->ctl_fd >= 0 && ex->req_fd >= 0 && ex->resp_fd >= 0;
  }

  void* get_req_addr_range() const { return req_.base; }
  void* get_resp_addr_range() const { return resp_.base; }
  size_t get_req_addr_pool_size() const { return req_.capacity; }
  size_t get_resp_addr_pool_size() const { return resp_.capacity; }
  bool is_double_mapped() const { return req_.double_mapped && resp_.double_mapped; }
  volatile uint32_t* get_doorbells_host() const { return h_doorbells_; }
  void* get_state_addr_range() const { return (void*)h_doorbells_; }  // the original's name for the same range
  volatile uint32_t* get_doorbells_device() const { return d_doorbells_; }
  SrpcSlotDesc* get_slot_desc(int slot) const { return (SrpcSlotDesc*)(h_desc_ + (size_t)slot * srpc_desc_stride(req_size_)); }
  uint32_t desc_per_slot() const { return srpc_desc_per_slot(req_size_); }
  volatile uint64_t* get_tx_offsets_host() const { return h_tx_off_; }
  volatile uint64_t* get_tx_offsets_device() const { return d_tx_off_; }
  volatile uint64_t* get_stamps_host() const { return h_stamps_; }
  volatile uint64_t* get_stamps_device() const { return d_stamps_; }
};

// ------------------------------------------------------------------ app slots
class P2pRpcAppRr {
 public:
  g_params* h_stub = nullptr;
  g_params* d_stub = nullptr;
  volatile uint32_t* h_state = nullptr;
  volatile uint32_t* d_state = nullptr;
  volatile uint64_t* h_tx_off = nullptr;  // where the serving side stores this slot's response (offset in the transmit arena)
  volatile uint64_t* h_stamps = nullptr;  // [0] doorbell rung, [1] response stored: timer values of whoever did it (ns)
  size_t req_size = 0, resp_size = 0;
  void* rpc_rr = nullptr;  // transport-side record this slot currently serves
  int rr_idx = 0;

  void print_app_rr_info() const {
    std::printf("app_rr %p idx=%d req=%p resp=%p state=%u\n", (const void*)this, rr_idx, (void*)h_stub->req,
                (void*)h_stub->resp, h_state ? *h_state : 0u);
  }

  // Debugging aids with the original's names (reference src/p2p_rpc_app_rr.h:49-79): fill the slot's request with
  // 32-bit ones / its response with zeros, and print the first words of either as floats and as integers.  The
  // buffers may be device memory: the bytes travel through a host staging copy on the default stream.
  int device_id = -1;  // set by the pool; < 0: the rings are host memory
  void set_dummy_input_on_gpu() { fill_words(h_stub->req, req_size, 1u); }
  void set_dummy_output_on_gpu() { fill_words(h_stub->resp, resp_size, 0u); }
  void dump_input_on_gpu(size_t max_words = 16) const { dump_words("Input", h_stub->req, req_size, max_words); }
  void dump_output_on_gpu(size_t max_words = 16) const { dump_words("Output", h_stub->resp, resp_size, max_words); }

 private:
  void fill_words(uint8_t* p, size_t bytes, uint32_t value) {
    std::vector<uint32_t> host(bytes / 4, value);
    copy_bytes(p, host.data(), host.size() * 4, true);
  }
  void dump_words(const char* what, const uint8_t* p, size_t bytes, size_t max_words) const {
    const size_t n = bytes / 4 < max_words ? bytes / 4 : max_words;
    std::vector<uint32_t> host(n);
    const_cast<P2pRpcAppRr*>(this)->copy_bytes(host.data(), p, n * 4, false);
    std::printf("%s: app_rr %p idx=%d at %p:", what, (const void*)this, rr_idx, (const void*)p);
    for (size_t i = 0; i < n; i++) {
      float f;
      std::memcpy(&f, &host[i], 4);
      std::printf(" %g(%u)", f, host[i]);
    }
    std::printf("\n");
  }
  // to_slot: host -> slot memory, else slot memory -> host
  void copy_bytes(void* dst, const void* src, size_t n, bool to_slot) {
    (void)to_slot;
    if (device_id < 0) {
      std::memcpy(dst, src, n);
      return;
    }
    const SrpcDeviceOps* ops = srpc_require_cuda("slot dump");
    ops->set_device(device_id);
    ops->memcpy_async(dst, src, n, nullptr);
    ops->stream_sync(nullptr);
  }
};

// N slots over the two rings.  get_next() hands the producer the next slot and
// binds it to the next req/resp addresses of the rings (reference
// src/p2p_rpc_app_rr.h:82-191).
class P2pRpcAppRrPool {
  int pool_size_;
  int device_id_;
  g_params* h_stubs_ = nullptr;
  g_params* d_stubs_ = nullptr;
  P2pRpcTring *req_pool_ = nullptr, *resp_pool_ = nullptr;
  size_t pi_idx_ = 0;
  bool stubs_mapped_ = false;

 public:
  size_t req_size, resp_size;
  P2pRpcAppRr* rr_pool = nullptr;
  P2pRpcAppRrMemPool* rr_mem_pool = nullptr;

  P2pRpcAppRrPool(int pool_size, int device_id, size_t _req_size, size_t _resp_size)
      : pool_size_(pool_size), device_id_(device_id), req_size(_req_size), resp_size(_resp_size) {
    rr_mem_pool = new P2pRpcAppRrMemPool(pool_size, device_id, req_size, resp_size);
    bind();
  }
  // Producer-side mirror of a pool that another process owns: same slots, same ring arithmetic, the addresses are this
  // process's mappings of the owner's rings (the original's SmartNIC-side pool mirrors the host's ring addresses the
  // same way, reference src/splitrpc_rdma_transport/p2p_rpc_bf_rr_pool.h:13-60).
  P2pRpcAppRrPool(const AppRrPoolExport& ex, int device_id)
      : pool_size_((int)ex.pool_size), device_id_(device_id), req_size(ex.req_size), resp_size(ex.resp_size) {
    rr_mem_pool = new P2pRpcAppRrMemPool(ex, device_id);
    if (rr_mem_pool->ok()) bind();
  }
  bool ok() const { return rr_mem_pool && rr_mem_pool->ok() && rr_pool; }

 private:
  void bind() {
    const int pool_size = pool_size_;
    const int device_id = device_id_;
    rr_pool = new P2pRpcAppRr[pool_size];
    req_pool_ = new P2pRpcTring(rr_mem_pool->get_req_addr_range(), rr_mem_pool->get_req_addr_pool_size());
    resp_pool_ = new P2pRpcTring(rr_mem_pool->get_resp_addr_range(), rr_mem_pool->get_resp_addr_pool_size());
    if (device_id >= 0) {
      // Slot stubs in mapped pinned memory: kernels that read the stub indirectly
      // (graph replay, persistent kernels) see host updates without a copy.
      void *h = nullptr, *d = nullptr;
      if (srpc_require_cuda("slot stubs")->host_alloc_mapped(sizeof(g_params) * pool_size, &h, &d) != 0) std::abort();
      h_stubs_ = (g_params*)h;
      d_stubs_ = (g_params*)d;
      stubs_mapped_ = true;
    } else {
      h_stubs_ = d_stubs_ = new g_params[pool_size];
    }
    volatile uint32_t* hs = rr_mem_pool->get_doorbells_host();
    volatile uint32_t* ds = rr_mem_pool->get_doorbells_device();
    for (int i = 0; i < pool_size; i++) {
      P2pRpcAppRr& r = rr_pool[i];
      r.req_size = req_size;
      r.resp_size = resp_size;
      r.h_stub = &h_stubs_[i];
      r.d_stub = &d_stubs_[i];
      r.h_state = &hs[i];
      r.d_state = &ds[i];
      r.h_tx_off = &rr_mem_pool->get_tx_offsets_host()[i];
      r.h_stamps = &rr_mem_pool->get_stamps_host()[2 * i];
      r.h_stub->req = nullptr;
      r.h_stub->resp = nullptr;
      r.rr_idx = i;
      r.device_id = device_id_;
    }
  }

 public:
  ~P2pRpcAppRrPool() {
    delete req_pool_;
    delete resp_pool_;
    if (stubs_mapped_) {
      if (const SrpcDeviceOps* ops = srpc_cuda_ops()) ops->host_free(h_stubs_);
    } else {
      delete[] h_stubs_;
    }
    delete rr_mem_pool;
    delete[] rr_pool;
  }

  int get_pool_size() const { return pool_size_; }
  int get_device_id() const { return device_id_; }
  P2pRpcAppRr* get_app_rr_pool() { return rr_pool; }
  P2pRpcAppRr* get_app_rr(int idx) { return (idx >= 0 && idx < pool_size_) ? &rr_pool[idx] : nullptr; }
  // Start of a serving session: the rings rewind and every slot is FREE with no transmit offset and no stamps
  // (whatever an earlier session left behind, e.g. a window that was armed when its server stopped).
  void init_pool() {
    pi_idx_ = 0;
    req_pool_->reset();
    resp_pool_->reset();
    for (int i = 0; i < pool_size_; i++) {
      P2pRpcAppRr* r = &rr_pool[i];
      if (r->h_stamps) r->h_stamps[0] = r->h_stamps[1] = 0;
      if (r->h_tx_off) __atomic_store_n(r->h_tx_off, P2pRpcAppRrMemPool::kNoTxOffset, __ATOMIC_RELAXED);
      if (r->h_state) __atomic_store_n(r->h_state, (uint32_t)APP_RR_STATUS::FREE, __ATOMIC_RELEASE);
    }
  }
  size_t producer_index() const { return pi_idx_; }

  P2pRpcAppRr* get_next() {
    P2pRpcAppRr* r = &rr_pool[pi_idx_];
    r->h_stub->req = (uint8_t*)req_pool_->get_next(req_size);
    r->h_stub->resp = (uint8_t*)resp_pool_->get_next(resp_size);
    pi_idx_ = (pi_idx_ + 1) % (size_t)pool_size_;
    return r;
  }

  // Ring addresses of the seq-th slot handed out since init_pool().  The rings
  // advance by a fixed size per slot, so the addresses of a window are known
  // before its producer has bound it; a consumer that arms work ahead of arrival
  // (the stream-armed worker) uses this instead of the slot's own stub.
  g_params window_stub(uint64_t seq) const {
    g_params p;
    p.req = (uint8_t*)req_pool_->base() + (size_t)((seq * (uint64_t)req_size) % req_pool_->capacity());
    p.resp = (uint8_t*)resp_pool_->base() + (size_t)((seq * (uint64_t)resp_size) % resp_pool_->capacity());
    return p;
  }
};

// ------------------------------------------------------------------ app context
// Execution context handed to the four app callbacks (reference
// src/p2p_rpc_app_ctx.h:24-112).  The doorbell is one word shared by host and
// device: UINT_MAX = armed/idle, 1 = run finished (written from the stream),
// 2 = persistent kernel finished, batch size = start signal for a persistent app.
template <class T>
class MetaAppCtx {
 public:
  T* h_stub = nullptr;
  T* d_stub = nullptr;
  uint32_t* door_bell = nullptr;
  uint32_t* d_door_bell = nullptr;
  void* app_ctx_internal = nullptr;
  int curr_batch_size = 1;
  int next_batch_size = 1;
  cudaStream_t work_stream = nullptr;
  cudaEvent_t work_complete = nullptr;
  void* curr_rr = nullptr;
  uint8_t launch_type = 1;  // 0 none, 1 kernel, 2 device-side launch, 3 persistent kernel, 4 CUDA graph
  int device_id = -1;
  bool graphCreated = false;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t instance = nullptr;
  uint64_t wait_budget_ns = 2000000000ull;  // bound on every host-side spin
  int last_status = 0;                      // 0 ok, -1 a bounded wait ran out
  RespPushCtx* h_push = nullptr;            // response-push block (host view / device view), see RespPushCtx
  RespPushCtx* d_push = nullptr;
  // On a GPU, d_stub and d_push point into a parameter block in the GPU's own memory that P2pRpcAppInfo::stage_window
  // rewrites in stream order before every batch; the mapped host copies below are what resident kernels poll.
  T* d_stub_mapped = nullptr;
  RespPushCtx* d_push_mapped = nullptr;
  uint8_t* param_block = nullptr;
  bool self_push = false;                   // the app's own kernels store responses and completions (fused epilogue)

  // Makes the work stream wait until *d_state == value.
  void AppRrRunNotify(volatile uint32_t* d_state, int value) {
    if (device_id >= 0) {
      const SrpcDeviceOps* ops = srpc_require_cuda("stream wait");
      ops->set_device(device_id);  // driver-level memops need this thread bound to the device's context
      if (ops->stream_wait_value32(work_stream, d_state, (uint32_t)value) != 0) {
        srpc_log(SRPC_LOG_ERROR, "stream wait failed: %s", ops->last_error());
        last_status = -2;
      }
    } else {
      last_status = spin_until(d_state, (uint32_t)value) ? 0 : -1;
    }
  }
  void AppRunNotify(int value) { AppRrRunNotify((volatile uint32_t*)d_door_bell, value); }

  // Writes `value` into the doorbell once everything queued so far has finished.
  void AppCompleteNotify(uint32_t value = 2) {
    if (device_id >= 0) {
      const SrpcDeviceOps* ops = srpc_require_cuda("stream write");
      ops->set_device(device_id);
      if (ops->stream_write_value32(work_stream, (volatile uint32_t*)d_door_bell, value) != 0) {
        srpc_log(SRPC_LOG_ERROR, "stream write failed: %s", ops->last_error());
        last_status = -2;
      }
    } else {
      __atomic_store_n(door_bell, value, __ATOMIC_RELEASE);
    }
  }
  // Start signal for a resident app kernel: the batch size with the start bit set
  // (so that batch sizes 1..3 cannot be mistaken for the status values).
  void NotifyAppRunStart() {
    __atomic_store_n(door_bell, APP_DOORBELL_START | (uint32_t)curr_batch_size, __ATOMIC_SEQ_CST);
  }
  bool IsAppRunComplete() const { return __atomic_load_n(door_bell, __ATOMIC_ACQUIRE) == 1u; }
  void ResetAppRunStatus() { __atomic_store_n(door_bell, (uint32_t)UINT_MAX, __ATOMIC_SEQ_CST); }

  // Returns false when the bounded wait ran out.
  bool WaitForAppRunComplete() {
    if (launch_type == 3) return spin_until((volatile uint32_t*)door_bell, 2u);
    if (device_id >= 0) return srpc_require_cuda("stream sync")->stream_sync(work_stream) == 0;
    return true;
  }

 private:
  bool spin_until(volatile uint32_t* p, uint32_t v) const {
    uint64_t t0 = getCurNs();
    uint32_t spins = 0;
    while (__atomic_load_n(p, __ATOMIC_ACQUIRE) != v) {
      if ((++spins & 0x3FF) == 0 && getCurNs() - t0 > wait_budget_ns) return false;
    }
    return true;
  }
};

typedef MetaAppCtx<g_params> AppCtx;
using AppInitCB = int (*)(AppCtx*);
using AppRunCB = int (*)(AppCtx*);
using AppCleanupCB = int (*)(AppCtx*);
using AppRunAsyncCB = int (*)(AppCtx*);
using AppRunWaitCB = int (*)(AppCtx*);
using AppCompleteCB = int (*)(AppCtx*);
