// C entry points around the ORIGINAL LeNet (src/apps/lenet/lenet_vanilla.cu, compiled unmodified): its cuda_init()
// loads data/lenet/data{0,1,2,3}.dat below the directory that P2P_DATA_SET_PATH names, its kernel_entry() runs one
// inference (twelve kernel launches) on the work stream of an AppCtx whose stub names a 784-byte image and a 40-byte
// response in device memory.  Nothing of the model is re-implemented here.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <string>

#include "lenet_vanilla.cuh"

namespace {
AppCtx* g_ctx = nullptr;
uint8_t* g_in = nullptr;
float* g_out = nullptr;
}  // namespace

extern "C" {

// `base` holds data/lenet/*.dat.  Returns 0 on success.  (A missing file makes the original exit the process.)
int ref_lenet_init(const char* base, int device) {
  if (g_ctx) return 0;
  if (cudaSetDevice(device) != cudaSuccess) return -1;
  std::string b(base);
  if (!b.empty() && b.back() != '/') b += '/';
  setenv("P2P_DATA_SET_PATH", b.c_str(), 1);
  cuda_init();
  if (cudaMalloc(&g_in, 1024) != cudaSuccess || cudaMalloc(&g_out, 64) != cudaSuccess) return -2;
  g_ctx = new AppCtx;
  g_ctx->h_stub = new g_params;
  g_ctx->h_stub->req = g_in;
  g_ctx->h_stub->resp = (uint8_t*)g_out;
  g_ctx->d_stub = nullptr;
  g_ctx->door_bell = new uint32_t(0);
  g_ctx->launch_type = 1;
  g_ctx->device_id = device;
  if (cudaStreamCreateWithFlags(&g_ctx->work_stream, cudaStreamNonBlocking) != cudaSuccess) return -3;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : -4;
}

// One inference: 784 bytes in, 10 floats out (host memory).
int ref_lenet_forward(const unsigned char* in, float* out) {
  if (!g_ctx) return -1;
  if (cudaMemcpyAsync(g_in, in, 784, cudaMemcpyHostToDevice, g_ctx->work_stream) != cudaSuccess) return -2;
  kernel_entry(g_ctx);
  if (cudaMemcpyAsync(out, g_out, 40, cudaMemcpyDeviceToHost, g_ctx->work_stream) != cudaSuccess) return -3;
  return cudaStreamSynchronize(g_ctx->work_stream) == cudaSuccess ? 0 : -4;
}

// Milliseconds per inference over `iters` back-to-back inferences (CUDA events), negative on failure.
float ref_lenet_time(int warmup, int iters) {
  if (!g_ctx || iters <= 0) return -1.f;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -2.f;
  for (int i = 0; i < warmup; i++) kernel_entry(g_ctx);
  cudaEventRecord(e0, g_ctx->work_stream);
  for (int i = 0; i < iters; i++) kernel_entry(g_ctx);
  cudaEventRecord(e1, g_ctx->work_stream);
  if (cudaStreamSynchronize(g_ctx->work_stream) != cudaSuccess) return -3.f;
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return ms / iters;
}

}  // extern "C"
