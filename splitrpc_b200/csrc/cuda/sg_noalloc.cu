// Allocation-free variant of the scatter-gather copy (see sg_noalloc.h for who
// needs it and the rules of use).  Same kernel as the regular path
// (sg_launch_copy in sg_kernels.cu); only the home of the copy list differs: a
// file-scope device array instead of a cudaMalloc'd buffer.
#include "sg_noalloc.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <mutex>

#include "sg_kernels.cuh"

namespace {

// The copy list of the most recent call on this device.  In host code this name
// is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) SgItem g_noalloc_items[SRPC_NOALLOC_MAX_ITEMS];

constexpr int kMaxDevices = 64;
std::atomic<SgItem*> g_dev_list[kMaxDevices];  // device address of g_noalloc_items per device, filled on first use
std::mutex g_setup_mu;

// Set-up, once per device, with that device current.  After the first call a device costs one atomic load here: the
// threads this entry point is for must not queue up behind a lock on every copy.
SgItem* list_address(int dev) {
  if (SgItem* p = g_dev_list[dev].load(std::memory_order_acquire)) return p;
  std::lock_guard<std::mutex> g(g_setup_mu);
  if (SgItem* p = g_dev_list[dev].load(std::memory_order_acquire)) return p;
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_items);
  if (e != cudaSuccess || !p) {
    std::fprintf(stderr, "srpc_sg_copy_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
    return nullptr;
  }
  g_dev_list[dev].store(static_cast<SgItem*>(p), std::memory_order_release);
  return static_cast<SgItem*>(p);
}

}  // namespace

extern "C" int srpc_sg_copy_noalloc(const uint64_t* src, const uint64_t* dst, const uint64_t* len, uint32_t n, void* stream) {
  if (n == 0) return 0;
  if (n > SRPC_NOALLOC_MAX_ITEMS) {
    std::fprintf(stderr, "srpc_sg_copy_noalloc: %u items exceed the built-in list of %d; split the list\n", n,
                 SRPC_NOALLOC_MAX_ITEMS);
    return -1;
  }
  if (!src || !dst || !len) return -2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
    (void)cudaGetLastError();
    return -4;
  }
  if (cap != cudaStreamCaptureStatusNone) return -5;  // a captured upload would read this stack frame at replay time
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -3;
  SgItem* d_list = list_address(dev);
  if (!d_list) return -3;
  // The list is assembled on this thread's stack and uploaded over the previous call's list.
  SgItem items[SRPC_NOALLOC_MAX_ITEMS];
  for (uint32_t i = 0; i < n; i++) {
    if (len[i] == 0 || len[i] > 0xFFFFFFFFull) return -2;
    items[i].src = src[i];
    items[i].dst = dst[i];
    items[i].len = (uint32_t)len[i];
    items[i].first_chunk = 0;
  }
  const uint32_t chunks = sg_assign_chunks(items, n);
  // Pageable source: the runtime stages it before returning, so `items` may leave scope.
  if (cudaMemcpyAsync(d_list, items, sizeof(SgItem) * n, cudaMemcpyHostToDevice, st) != cudaSuccess) return -4;
  if (sg_launch_copy(d_list, n, chunks, SG_IMPL_SIMT, 0, st) != cudaSuccess) return -4;
  return 0;
}
