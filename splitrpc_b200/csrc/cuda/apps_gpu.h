// Factory for the built-in GPU apps (echo, vec_add, matmul, lenet5).
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
