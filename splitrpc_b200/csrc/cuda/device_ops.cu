// CUDA implementation of the device-operation table used by the host core.
//
// Ring memory is a CUDA virtual-memory-management allocation mapped twice back to
// back in one reserved address range, so a window of consecutive slots that runs
// past the end of the ring is still contiguous (same idea as reference
// src/p2p_rpc_app_rr_mem_pool.h:213-339), with read/write access granted to every
// GPU that can reach the owner over NVLink.  Doorbell words are mapped pinned
// host memory.  Stream-ordered doorbell waits and writes use the driver's stream
// memory operations (reference src/utils/g_utils.cu:42-53).  Driver entry points
// are resolved at run time, so the library loads on machines without a driver.
#include <cuda.h>
#include <cuda_runtime.h>

#include <unistd.h>

#include <mutex>
#include <string>
#include <vector>

#include "../host/p2p_rpc_app.h"
#include "driver_api.h"
#include "sg_kernels.cuh"

static thread_local std::string g_last_error;

static int fail(const char* what, cudaError_t e) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return -1;
}
static int fail_drv(const char* what, CUresult r) {
  g_last_error = std::string(what) + ": CUresult " + std::to_string((int)r);
  return -1;
}
#define RT(call)                                   \
  do {                                             \
    cudaError_t _e = (call);                       \
    if (_e != cudaSuccess) return fail(#call, _e); \
  } while (0)
#define DRV(call)                                        \
  do {                                                   \
    CUresult _r = (call);                                \
    if (_r != CUDA_SUCCESS) return fail_drv(#call, _r);  \
  } while (0)

const SrpcDriverApi* srpc_driver_api() {
  static SrpcDriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char* name, void** fn) {
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
        *fn = nullptr;
    };
    get("cuMemCreate", (void**)&api.MemCreate);
    get("cuMemRelease", (void**)&api.MemRelease);
    get("cuMemAddressReserve", (void**)&api.MemAddressReserve);
    get("cuMemAddressFree", (void**)&api.MemAddressFree);
    get("cuMemMap", (void**)&api.MemMap);
    get("cuMemUnmap", (void**)&api.MemUnmap);
    get("cuMemSetAccess", (void**)&api.MemSetAccess);
    get("cuMemGetAllocationGranularity", (void**)&api.MemGetAllocationGranularity);
    get("cuStreamWaitValue32", (void**)&api.StreamWaitValue32);
    get("cuStreamWriteValue32", (void**)&api.StreamWriteValue32);
    get("cuStreamWriteValue64", (void**)&api.StreamWriteValue64);
    get("cuTensorMapEncodeTiled", (void**)&api.TensorMapEncodeTiled);
    get("cuDeviceGetAttribute", (void**)&api.DeviceGetAttribute);
    get("cuMemExportToShareableHandle", (void**)&api.MemExportToShareableHandle);
    get("cuMemImportFromShareableHandle", (void**)&api.MemImportFromShareableHandle);
    api.ok = api.MemCreate && api.MemMap && api.StreamWaitValue32 && api.TensorMapEncodeTiled;
  });
  return &api;
}

struct RingImpl {
  CUmemGenericAllocationHandle handle;
  CUdeviceptr va;
  size_t cap;
  bool vmm;
  bool shareable;  // created with a POSIX file descriptor handle type, so it can be exported
};

// Maps `handle` twice back to back and grants access to `owner` and (optionally) to every device that can reach it.
static int map_ring_twice(const SrpcDriverApi* d, RingImpl* impl, size_t cap, size_t gran, int owner, bool peer_access,
                          int only_dev) {
  CUresult r = d->MemAddressReserve(&impl->va, 2 * cap, gran, 0, 0);
  if (r != CUDA_SUCCESS) return fail_drv("cuMemAddressReserve", r);
  DRV(d->MemMap(impl->va, cap, 0, impl->handle, 0));
  DRV(d->MemMap(impl->va + cap, cap, 0, impl->handle, 0));
  std::vector<CUmemAccessDesc> acc;
  int ndev = 0;
  cudaGetDeviceCount(&ndev);
  for (int p = 0; p < ndev; p++) {
    int can = (p == owner);
    if (only_dev >= 0) can = (p == only_dev);
    else if (p != owner && peer_access) cudaDeviceCanAccessPeer(&can, p, owner);
    if (!can) continue;
    CUmemAccessDesc a = {};
    a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    a.location.id = p;
    a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    acc.push_back(a);
  }
  DRV(d->MemSetAccess(impl->va, 2 * cap, acc.data(), acc.size()));
  impl->cap = cap;
  impl->vmm = true;
  return 0;
}

static int d_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}
__global__ void timer_probe_kernel(volatile unsigned long long* out);
struct TimerProbe;
static TimerProbe* timer_probe_for(int dev);
static void preload_own_kernels() {
  cudaFuncAttributes fa;
  (void)cudaFuncGetAttributes(&fa, timer_probe_kernel);
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) (void)timer_probe_for(dev);
  (void)cudaGetLastError();
}
static int d_set_device(int dev) {
  RT(cudaSetDevice(dev));
  return 0;
}
static int d_stream_create(int dev, cudaStream_t* s) {
  RT(cudaSetDevice(dev));
  sg_preload_kernels();  // every GPU app context passes here before its stream can be armed on a doorbell
  preload_own_kernels();
  RT(cudaStreamCreateWithFlags(s, cudaStreamNonBlocking));
  return 0;
}
static int d_stream_destroy(cudaStream_t s) {
  RT(cudaStreamDestroy(s));
  return 0;
}
static int d_stream_sync(cudaStream_t s) {
  RT(cudaStreamSynchronize(s));
  return 0;
}
static int d_stream_query(cudaStream_t s) {
  cudaError_t e = cudaStreamQuery(s);
  if (e == cudaSuccess) return 0;
  if (e == cudaErrorNotReady) return 1;
  return fail("cudaStreamQuery", e);
}
static int d_wait32(cudaStream_t s, volatile uint32_t* addr, uint32_t v) {
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->StreamWaitValue32) return fail_drv("cuStreamWaitValue32 unavailable", CUDA_ERROR_NOT_SUPPORTED);
  DRV(d->StreamWaitValue32((CUstream)s, (CUdeviceptr)(uintptr_t)addr, v, CU_STREAM_WAIT_VALUE_EQ));
  return 0;
}
static int d_write32(cudaStream_t s, volatile uint32_t* addr, uint32_t v) {
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->StreamWriteValue32) return fail_drv("cuStreamWriteValue32 unavailable", CUDA_ERROR_NOT_SUPPORTED);
  DRV(d->StreamWriteValue32((CUstream)s, (CUdeviceptr)(uintptr_t)addr, v, CU_STREAM_WRITE_VALUE_DEFAULT));
  return 0;
}
// Stream-ordered wait until (int32)(*addr - v) >= 0, for sequence-number doorbells that may have moved on.
extern "C" int srpc_stream_wait32_geq(cudaStream_t s, uint32_t* addr, uint32_t v) {
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->StreamWaitValue32) return fail_drv("cuStreamWaitValue32 unavailable", CUDA_ERROR_NOT_SUPPORTED);
  DRV(d->StreamWaitValue32((CUstream)s, (CUdeviceptr)(uintptr_t)addr, v, CU_STREAM_WAIT_VALUE_GEQ));
  return 0;
}
extern "C" int srpc_stream_write64(cudaStream_t s, uint64_t* addr, uint64_t v) {
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->StreamWriteValue64) return fail_drv("cuStreamWriteValue64 unavailable", CUDA_ERROR_NOT_SUPPORTED);
  DRV(d->StreamWriteValue64((CUstream)s, (CUdeviceptr)(uintptr_t)addr, v, CU_STREAM_WRITE_VALUE_DEFAULT));
  return 0;
}
static int d_event_create(cudaEvent_t* e) {
  RT(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
  return 0;
}
static int d_event_destroy(cudaEvent_t e) {
  RT(cudaEventDestroy(e));
  return 0;
}

static int d_ring_alloc(int dev, size_t min_bytes, size_t slot_bytes, bool peer_access, SrpcRingMem* out) {
  RT(cudaSetDevice(dev));
  RT(cudaFree(0));  // make sure the primary context exists before driver calls
  const SrpcDriverApi* d = srpc_driver_api();
  RingImpl* impl = new RingImpl{};
  if (d->ok) {
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    size_t gran = 0;
    DRV(d->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM));
    size_t cap = srpc_ring_capacity(min_bytes, slot_bytes, gran);
    // Ask for an allocation that can be handed to another process as a file descriptor; fall back to a private one.
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    impl->shareable = true;
    if (d->MemCreate(&impl->handle, cap, &prop, 0) != CUDA_SUCCESS) {
      prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_NONE;
      impl->shareable = false;
      DRV(d->MemCreate(&impl->handle, cap, &prop, 0));
    }
    if (map_ring_twice(d, impl, cap, gran, dev, peer_access, -1) != 0) {
      d->MemRelease(impl->handle);
      delete impl;
      return -1;
    }
    out->base = (void*)impl->va;
    out->capacity = cap;
    out->double_mapped = true;
  } else {
    // No virtual memory management: plain allocation, windows must not wrap.
    void* p = nullptr;
    RT(cudaMalloc(&p, min_bytes));
    impl->va = (CUdeviceptr)(uintptr_t)p;
    impl->cap = min_bytes;
    impl->vmm = false;
    out->base = p;
    out->capacity = min_bytes;
    out->double_mapped = false;
  }
  out->impl = impl;
  return 0;
}

static int d_ring_free(SrpcRingMem* m) {
  RingImpl* impl = static_cast<RingImpl*>(m->impl);
  if (!impl) return 0;
  const SrpcDriverApi* d = srpc_driver_api();
  if (impl->vmm) {
    d->MemUnmap(impl->va, 2 * impl->cap);
    d->MemAddressFree(impl->va, 2 * impl->cap);
    d->MemRelease(impl->handle);
  } else {
    cudaFree((void*)(uintptr_t)impl->va);
  }
  delete impl;
  m->impl = nullptr;
  m->base = nullptr;
  return 0;
}

static int d_ring_export(const SrpcRingMem* m, int* fd) {
  const RingImpl* impl = static_cast<const RingImpl*>(m->impl);
  const SrpcDriverApi* d = srpc_driver_api();
  if (!impl || !impl->vmm || !impl->shareable || !d->MemExportToShareableHandle)
    return fail_drv("ring is not shareable", CUDA_ERROR_NOT_SUPPORTED);
  int out = -1;
  DRV(d->MemExportToShareableHandle(&out, impl->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd = out;
  return 0;
}

// The physical memory stays on the exporting process's GPU; this process maps it and lets `dev` address it over
// NVLink.  The descriptor is closed here: the mapping keeps the allocation alive.
static int d_ring_import(int dev, int fd, size_t cap, SrpcRingMem* out) {
  RT(cudaSetDevice(dev));
  RT(cudaFree(0));
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->ok || !d->MemImportFromShareableHandle) return fail_drv("cuMemImportFromShareableHandle unavailable", CUDA_ERROR_NOT_SUPPORTED);
  RingImpl* impl = new RingImpl{};
  CUresult r = d->MemImportFromShareableHandle(&impl->handle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  if (r != CUDA_SUCCESS) {
    delete impl;
    return fail_drv("cuMemImportFromShareableHandle", r);
  }
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  size_t gran = 0;
  DRV(d->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM));
  if (map_ring_twice(d, impl, cap, gran, dev, false, dev) != 0) {
    d->MemRelease(impl->handle);
    delete impl;
    return -1;
  }
  impl->shareable = false;
  out->base = (void*)impl->va;
  out->capacity = cap;
  out->double_mapped = true;
  out->impl = impl;
  out->fd = -1;
  return 0;
}

static int d_host_register(void* p, size_t bytes, void** dptr) {
  RT(cudaHostRegister(p, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable));
  RT(cudaHostGetDevicePointer(dptr, p, 0));
  return 0;
}
static int d_host_unregister(void* p) {
  RT(cudaHostUnregister(p));
  return 0;
}

static int d_host_alloc_mapped(size_t bytes, void** h, void** dptr) {
  RT(cudaHostAlloc(h, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
  RT(cudaHostGetDevicePointer(dptr, *h, 0));
  memset(*h, 0, bytes);
  return 0;
}
static int d_host_free(void* h) {
  RT(cudaFreeHost(h));
  return 0;
}
static int d_dev_alloc(int dev, size_t bytes, void** p) {
  RT(cudaSetDevice(dev));
  RT(cudaMalloc(p, bytes));
  return 0;
}
static int d_dev_free(void* p) {
  RT(cudaFree(p));
  return 0;
}
static int d_memcpy_async(void* dst, const void* src, size_t n, cudaStream_t s) {
  RT(cudaMemcpyAsync(dst, src, n, cudaMemcpyDefault, s));
  return 0;
}
static int d_memset_async(void* dst, int v, size_t n, cudaStream_t s) {
  RT(cudaMemsetAsync(dst, v, n, s));
  return 0;
}
static int d_graph_launch(cudaGraphExec_t g, cudaStream_t s) {
  RT(cudaGraphLaunch(g, s));
  return 0;
}
static int d_resp_push(const void* d_stub, const void* d_push, int n, cudaStream_t s) {
  RT(sg_launch_resp_push(d_stub, d_push, n, s));
  return 0;
}
static int d_window_params(void* block, const g_params* stub, const RespPushCtx* ctx, const uint64_t* offsets, int n,
                           const uint32_t* live_enabled, cudaStream_t s) {
  RT(sg_launch_window_params(block, stub, ctx, offsets, n, live_enabled, s));
  return 0;
}
// One thread writes the device timer into a mapped host word; the host notes its own clock the moment the word
// arrives (the write takes about a microsecond to cross PCIe).  The smallest of a few tries is the least delayed.
__global__ void timer_probe_kernel(volatile unsigned long long* out) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *out = t;
  __threadfence_system();
}
// The probe's mapped word and stream are made once per device, when the device's first app context is set up:
// allocating or freeing pinned memory synchronises the device, and a device whose work stream is parked on a doorbell
// (or that runs a collective that waits for the very process that asked for this measurement) never gets there.
struct TimerProbe {
  volatile unsigned long long* w = nullptr;
  unsigned long long* dw = nullptr;
  cudaStream_t s = nullptr;
};
static TimerProbe* timer_probe_for(int dev) {
  static std::mutex mu;
  static TimerProbe probes[64];
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> g(mu);
  TimerProbe& p = probes[dev];
  if (!p.w) {
    void* h = nullptr;
    if (cudaHostAlloc(&h, 64, cudaHostAllocMapped) != cudaSuccess) return nullptr;
    if (cudaHostGetDevicePointer((void**)&p.dw, h, 0) != cudaSuccess || cudaStreamCreateWithFlags(&p.s, cudaStreamNonBlocking) != cudaSuccess) {
      cudaFreeHost(h);
      return nullptr;
    }
    p.w = (volatile unsigned long long*)h;
  }
  return &p;
}
static int d_timer_offset_ns(int dev, int64_t* offset) {
  int prev = 0;
  RT(cudaGetDevice(&prev));
  RT(cudaSetDevice(dev));
  TimerProbe* p = timer_probe_for(dev);
  int rc = p ? 0 : -1;
  int64_t best = 0;
  uint64_t best_wait = ~0ull;
  for (int i = 0; rc == 0 && i < 6; i++) {
    *p->w = 0;
    const uint64_t t0 = getCurNs();
    timer_probe_kernel<<<1, 1, 0, p->s>>>(p->dw);
    if (cudaGetLastError() != cudaSuccess) {
      rc = -1;
      break;
    }
    uint64_t t1 = t0;
    while (*p->w == 0 && (t1 = getCurNs()) - t0 < 500000000ull) {
    }
    if (*p->w == 0) {
      rc = -1;
      break;
    }
    t1 = getCurNs();
    // the first try includes start-up costs; a short host wait means the stamp is fresh
    if (i >= 1 && t1 - t0 < best_wait) {
      best_wait = t1 - t0;
      best = (int64_t)*p->w - (int64_t)t1;
    }
  }
  cudaSetDevice(prev);
  if (rc != 0) {
    g_last_error = "timer_offset_ns: probe failed";
    return rc;
  }
  *offset = best;
  return 0;
}
static const char* d_last_error() { return g_last_error.c_str(); }

extern "C" const SrpcDeviceOps* srpc_cuda_ops() {
  static const SrpcDeviceOps ops = {
      d_device_count, d_set_device,  d_stream_create, d_stream_destroy,    d_stream_sync, d_stream_query, d_wait32,
      d_write32,      d_event_create, d_event_destroy, d_ring_alloc,        d_ring_free,   d_host_alloc_mapped,
      d_host_free,    d_dev_alloc,    d_dev_free,      d_memcpy_async,      d_memset_async, d_graph_launch, d_last_error,
      d_ring_export,  d_ring_import,  d_host_register, d_host_unregister,   d_resp_push,
      d_timer_offset_ns, d_window_params};
  return &ops;
}

// Capability report in the spirit of reference src/splitrpc_server/device_test.cu:8-41.
extern "C" int srpc_device_caps(int dev, int* vmm, int* stream_memops, int* gdr_with_vmm, int* sm_major, int* sm_minor,
                                int* n_sm) {
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->DeviceGetAttribute) return -1;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) return -1;
  *sm_major = p.major;
  *sm_minor = p.minor;
  *n_sm = p.multiProcessorCount;
  d->DeviceGetAttribute(vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
  *stream_memops = 1;  // stream memory operations are always on since CUDA 12
  d->DeviceGetAttribute(gdr_with_vmm, CU_DEVICE_ATTRIBUTE_GPU_DIRECT_RDMA_WITH_CUDA_VMM_SUPPORTED, dev);
  return 0;
}
