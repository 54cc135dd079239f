// C entry points around the ORIGINAL scatter-gather code, for the reference arm of bench.py.
//
// Nothing of the data path is re-implemented here: the copy lists are built by the original's gather_skbs /
// scatter_skbs (src/p2p_rpc_sg_engine.h:19-73) and executed by the original's sg_on_gpu (src/transport/g_copy_ng.cu:
// 185-223) on a CopyCtx, followed by the original's WaitForAppRunComplete (src/p2p_rpc_app_ctx.h:65-74), one request
// at a time, which is how its shunter thread drives the engine (src/splitrpc_server/p2p_rpc_dpdk_server.cc:117-136).
// Copy types: 0 = one cudaMemcpyAsync per buffer, 2 = CopyKernel (one thread block per buffer).  Type 1 (the resident
// single-block kernel, whose doorbell spin has no bound) and type 3 (device-side memcpy) are refused.
// This file only allocates the context and exposes plain C symbols.  The original keeps the engine's stub in GPU memory
// that the CPU writes through a gdrcopy BAR mapping (src/p2p_rpc_sg_engine.h:262-266, BufItemPool with a device id), so
// its copy kernel reads the buffer list out of local HBM.  gdrcopy does not exist here; the same placement is obtained
// by giving the context a device-memory d_stub and uploading the list with one cudaMemcpyAsync on the engine's stream
// right before sg_on_gpu (whose own memcpy then lands in a pinned host staging copy that nothing reads).  A stub in
// mapped host memory would make every thread of CopyKernel fetch its three list entries over PCIe, which the original
// never does.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <fstream>  // the original's stats_utils.h uses std::ofstream without including it

// same include order as src/splitrpc_server/p2p_rpc_dpdk_server.cc:14-19
#include "p2p_rpc_rr_ng.h"
#include "p2p_rpc_sg_engine.h"

namespace {

struct RefEngine {
  CopyCtx* gather_ctx = nullptr;
  CopyCtx* scatter_ctx = nullptr;
  p2p_bufs* bufs = nullptr;
  p2p_sk_buf* skb = nullptr;
  int device = 0;
};

CopyCtx* make_ctx(int device, int copy_type) {
  CopyCtx* c = new CopyCtx;
  c->launch_type = (uint8_t)copy_type;
  c->device_id = device;
  if (cudaStreamCreateWithFlags(&c->work_stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
  if (cudaEventCreateWithFlags(&c->work_complete, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  void* h = nullptr;
  if (cudaHostAlloc(&h, sizeof(g_copy_params) + 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return nullptr;
  std::memset(h, 0, sizeof(g_copy_params) + 64);
  c->h_stub = (g_copy_params*)h;
  void* d = nullptr;
  if (cudaMalloc(&d, sizeof(g_copy_params)) != cudaSuccess) return nullptr;
  c->d_stub = (g_copy_params*)d;
  void* db = nullptr;
  if (cudaHostGetDevicePointer(&db, h, 0) != cudaSuccess) return nullptr;
  c->door_bell = (uint32_t*)((uint8_t*)h + sizeof(g_copy_params));
  c->d_door_bell = (uint32_t*)((uint8_t*)db + sizeof(g_copy_params));
  return c;
}

// Stands in for the CPU's write of the list through the BAR mapping: the list reaches the device copy of the stub in
// stream order, ahead of the kernel that sg_on_gpu launches on the same stream.
bool upload_stub(CopyCtx* c, const p2p_sk_buf* skb) {
  if (c->launch_type != 2) return true;
  return cudaMemcpyAsync(c->d_stub, skb, sizeof(g_copy_params), cudaMemcpyHostToDevice, c->work_stream) == cudaSuccess;
}

}  // namespace

extern "C" {

void* ref_engine_create(int device, int copy_type) {
  if (copy_type != 0 && copy_type != 2) return nullptr;
  if (cudaSetDevice(device) != cudaSuccess) return nullptr;
  RefEngine* e = new RefEngine;
  e->device = device;
  e->gather_ctx = make_ctx(device, copy_type);
  e->scatter_ctx = make_ctx(device, copy_type);
  e->bufs = new p2p_bufs;
  if (cudaHostAlloc((void**)&e->skb, sizeof(p2p_sk_buf), cudaHostAllocDefault) != cudaSuccess) return nullptr;  // pinned: the upload is a true async copy
  if (!e->gather_ctx || !e->scatter_ctx) return nullptr;
  return e;
}

// Gathers `n_req` requests, each made of `frags_per_req` fragments of `frag_len` bytes (the last one `last_len`) that
// sit `frag_stride` bytes apart starting at src + r * req_stride, into dst + r * req_size: per request the original's
// list builder, launch and wait.  Returns 0, or the 1-based request that failed.
int ref_gather_batch(void* engine, uint64_t src, uint64_t req_stride, uint64_t frag_stride, uint32_t frag_len, uint32_t last_len,
                     int frags_per_req, uint64_t dst, uint64_t req_size, int n_req) {
  RefEngine* e = (RefEngine*)engine;
  cudaSetDevice(e->device);
  for (int r = 0; r < n_req; r++) {
    e->bufs->num_items = (uint16_t)frags_per_req;
    for (int f = 0; f < frags_per_req; f++) {
      e->bufs->burst_items[f] = (uintptr_t)(src + (uint64_t)r * req_stride + (uint64_t)f * frag_stride);
      e->bufs->item_size[f] = f == frags_per_req - 1 ? last_len : frag_len;
    }
    gather_skbs(e->skb, e->bufs, (uint8_t*)(uintptr_t)(dst + (uint64_t)r * req_size));
    if (!upload_stub(e->gather_ctx, e->skb) || sg_on_gpu(e->gather_ctx, e->skb) != 1) return r + 1;
    e->gather_ctx->WaitForAppRunComplete();
  }
  return 0;
}

// Scatters `n_req` responses of `resp_size` bytes from src + r * resp_size into one transmit buffer each at
// dst + r * dst_stride (responses here fit one fragment).
int ref_scatter_batch(void* engine, uint64_t src, uint64_t resp_size, uint64_t dst, uint64_t dst_stride, int n_req) {
  RefEngine* e = (RefEngine*)engine;
  cudaSetDevice(e->device);
  for (int r = 0; r < n_req; r++) {
    e->bufs->num_items = 1;
    e->bufs->burst_items[0] = (uintptr_t)(dst + (uint64_t)r * dst_stride);
    e->bufs->item_size[0] = resp_size;
    scatter_skbs(e->skb, e->bufs, (uint8_t*)(uintptr_t)(src + (uint64_t)r * resp_size));
    if (!upload_stub(e->scatter_ctx, e->skb) || sg_on_gpu(e->scatter_ctx, e->skb) != 1) return r + 1;
    e->scatter_ctx->WaitForAppRunComplete();
  }
  return 0;
}

// Scatters `n_req` multi-fragment responses: response r (resp_size bytes at src + r * resp_size) goes into
// `frags_per_resp` transmit buffers of `frag_len` bytes (the last one `last_len`) that sit `frag_stride` bytes apart
// from dst + r * resp_stride on.
int ref_scatter_batch_frags(void* engine, uint64_t src, uint64_t resp_size, uint64_t dst, uint64_t resp_stride, uint64_t frag_stride,
                            uint32_t frag_len, uint32_t last_len, int frags_per_resp, int n_req) {
  RefEngine* e = (RefEngine*)engine;
  cudaSetDevice(e->device);
  for (int r = 0; r < n_req; r++) {
    e->bufs->num_items = (uint16_t)frags_per_resp;
    for (int f = 0; f < frags_per_resp; f++) {
      e->bufs->burst_items[f] = (uintptr_t)(dst + (uint64_t)r * resp_stride + (uint64_t)f * frag_stride);
      e->bufs->item_size[f] = f == frags_per_resp - 1 ? last_len : frag_len;
    }
    scatter_skbs(e->skb, e->bufs, (uint8_t*)(uintptr_t)(src + (uint64_t)r * resp_size));
    if (!upload_stub(e->scatter_ctx, e->skb) || sg_on_gpu(e->scatter_ctx, e->skb) != 1) return r + 1;
    e->scatter_ctx->WaitForAppRunComplete();
  }
  return 0;
}

// Number of copy items the original's list builder makes of one such request (shows whether fragments coalesced).
int ref_items_per_request(void* engine, uint64_t src, uint64_t frag_stride, uint32_t frag_len, uint32_t last_len, int frags_per_req) {
  RefEngine* e = (RefEngine*)engine;
  e->bufs->num_items = (uint16_t)frags_per_req;
  for (int f = 0; f < frags_per_req; f++) {
    e->bufs->burst_items[f] = (uintptr_t)(src + (uint64_t)f * frag_stride);
    e->bufs->item_size[f] = f == frags_per_req - 1 ? last_len : frag_len;
  }
  gather_skbs(e->skb, e->bufs, (uint8_t*)0x1000);
  return (int)e->skb->num_items;
}

void ref_engine_destroy(void* engine) {
  RefEngine* e = (RefEngine*)engine;
  if (!e) return;
  cudaSetDevice(e->device);
  for (CopyCtx* c : {e->gather_ctx, e->scatter_ctx}) {
    if (!c) continue;
    cudaStreamSynchronize(c->work_stream);
    cudaStreamDestroy(c->work_stream);
    cudaEventDestroy(c->work_complete);
    cudaFreeHost(c->h_stub);
    cudaFree(c->d_stub);
    delete c;
  }
  delete e->bufs;
  cudaFreeHost(e->skb);
  delete e;
}

}  // extern "C"
