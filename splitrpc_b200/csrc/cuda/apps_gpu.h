// Factories for the built-in GPU apps (echo, vec_add, matmul, lenet5) and for the
// graph app that serves models captured into CUDA graphs.
#pragma once

#include <vector>

#include "../host/p2p_rpc_app.h"

struct GpuAppHandle {
  void* internal = nullptr;  // goes into app_ctx->app_ctx_internal; freed by cleanup
  AppInitCB init = nullptr;
  AppRunCB run = nullptr;
  AppCleanupCB cleanup = nullptr;
  AppCompleteCB complete = nullptr;
};

// Returns a handle with null callbacks when the name is unknown or no GPU is present.
GpuAppHandle srpc_make_gpu_app(const char* name, int device_id, size_t req_size, size_t resp_size,
                               const std::vector<std::vector<float>>& weights);

// Graph app: run() launches the graph registered for the current batch size.
GpuAppHandle srpc_make_graph_app();
void srpc_graph_app_set(void* internal, int batch, cudaGraphExec_t exec);

// Stream capture helpers (thread-local capture mode, so other threads may keep
// issuing CUDA calls while a model is being captured).
// Both return 0 on success, else the CUDA error code.
int srpc_capture_begin(cudaStream_t stream);
int srpc_capture_end(cudaStream_t stream, cudaGraphExec_t* exec);
