// C entry points around the ORIGINAL generated LSTM runtime (src/apps/nnfusion_lstm/nnfusion_rt.cu, compiled
// unmodified): its cuda_init() loads ./Constant/Constant_<id>_0.bin and its kernel_entry() runs one inference on the
// work stream of an AppCtx whose stub names the input and output in device memory.  Nothing of the model is
// re-implemented here; the file only builds the context, copies the request in and the response out, and times the
// launches with CUDA events.
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdio>
#include <exception>

#include "nnfusion_rt.h"

namespace {
AppCtx* g_ctx = nullptr;
float *g_in = nullptr, *g_out = nullptr;
constexpr size_t kReqBytes = 8 * 256 * 4, kRespBytes = 256 * 4;  // 8 time steps x hidden 256 in, last hidden state out
}  // namespace

extern "C" {

// `dir` holds the Constant/ directory.  Returns 0 on success.
int ref_lstm_init(const char* dir, int device) {
  if (g_ctx) return 0;
  if (cudaSetDevice(device) != cudaSuccess) return -1;
  char cwd[4096];
  if (!getcwd(cwd, sizeof(cwd))) return -2;
  if (chdir(dir) != 0) return -3;
  int rc = 0;
  try {
    cuda_init();  // reads ./Constant/...; exits the process when a file is missing
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ref_lstm_init: %s\n", e.what());
    rc = -4;
  }
  if (chdir(cwd) != 0) rc = rc ? rc : -5;
  if (rc) return rc;
  if (cudaMalloc(&g_in, kReqBytes) != cudaSuccess || cudaMalloc(&g_out, kRespBytes) != cudaSuccess) return -6;
  g_ctx = new AppCtx;
  g_ctx->h_stub = new g_params;
  g_ctx->h_stub->req = (uint8_t*)g_in;
  g_ctx->h_stub->resp = (uint8_t*)g_out;
  g_ctx->d_stub = nullptr;
  g_ctx->launch_type = 1;
  g_ctx->device_id = device;
  if (cudaStreamCreateWithFlags(&g_ctx->work_stream, cudaStreamNonBlocking) != cudaSuccess) return -7;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : -8;
}

// One inference: 2048 floats in, 256 floats out (host memory).  Returns 0 on success.
int ref_lstm_forward(const float* in, float* out) {
  if (!g_ctx) return -1;
  if (cudaMemcpyAsync(g_in, in, kReqBytes, cudaMemcpyHostToDevice, g_ctx->work_stream) != cudaSuccess) return -2;
  kernel_entry(g_ctx);
  if (cudaMemcpyAsync(out, g_out, kRespBytes, cudaMemcpyDeviceToHost, g_ctx->work_stream) != cudaSuccess) return -3;
  return cudaStreamSynchronize(g_ctx->work_stream) == cudaSuccess ? 0 : -4;
}

// `iters` back-to-back inferences on the input that is already on the device; returns milliseconds per inference
// (CUDA events on the work stream), negative on failure.
float ref_lstm_time(int warmup, int iters) {
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
