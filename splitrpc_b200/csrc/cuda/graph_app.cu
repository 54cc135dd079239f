// "graph" app: serves a model whose forward pass was captured into one CUDA graph
// per batch size.  The Python layer builds the model out of this library's
// kernels, captures the graphs on the app's work stream (the kernels read the
// request/response pointers through the device-visible stub, so one graph serves
// every position of the ring) and registers them here; the worker loop then
// launches graphs without entering Python (launch type 4 of reference
// src/p2p_rpc_app_ctx.h:93-95, generalised to models defined in PyTorch).
#include <cuda_runtime.h>

#include <map>
#include <mutex>

#include "../host/p2p_rpc_app.h"
#include "apps_gpu.h"

namespace {

struct GraphAppState {
  std::mutex mu;
  std::map<int, cudaGraphExec_t> graphs;
  uint64_t launches = 0, missing = 0;
};

int graph_init(AppCtx* c) {
  c->launch_type = 4;
  return 1;
}
int graph_run(AppCtx* c) {
  GraphAppState* s = static_cast<GraphAppState*>(c->app_ctx_internal);
  cudaGraphExec_t g = nullptr;
  {
    std::lock_guard<std::mutex> lk(s->mu);
    auto it = s->graphs.find(c->curr_batch_size);
    if (it != s->graphs.end()) g = it->second;
  }
  if (!g) {
    s->missing++;
    srpc_log(SRPC_LOG_ERROR, "graph app: no graph registered for batch size %d", c->curr_batch_size);
    return 0;
  }
  cudaSetDevice(c->device_id);
  s->launches++;
  return cudaGraphLaunch(g, c->work_stream) == cudaSuccess;
}
int graph_complete(AppCtx*) { return 1; }
int graph_cleanup(AppCtx* c) {
  GraphAppState* s = static_cast<GraphAppState*>(c->app_ctx_internal);
  cudaSetDevice(c->device_id);
  for (auto& kv : s->graphs) cudaGraphExecDestroy(kv.second);
  delete s;
  c->app_ctx_internal = nullptr;
  return 1;
}

}  // namespace

GpuAppHandle srpc_make_graph_app() {
  GpuAppHandle h;
  h.internal = new GraphAppState;
  h.init = graph_init;
  h.run = graph_run;
  h.cleanup = graph_cleanup;
  h.complete = graph_complete;
  return h;
}

void srpc_graph_app_set(void* internal, int batch, cudaGraphExec_t exec) {
  GraphAppState* s = static_cast<GraphAppState*>(internal);
  std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->graphs.find(batch);
  if (it != s->graphs.end()) cudaGraphExecDestroy(it->second);
  s->graphs[batch] = exec;
}

int srpc_capture_begin(cudaStream_t stream) { return (int)cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal); }

int srpc_capture_end(cudaStream_t stream, cudaGraphExec_t* exec) {
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(stream, &g);
  if (e != cudaSuccess) return (int)e;
  e = cudaGraphInstantiate(exec, g, 0);
  cudaGraphDestroy(g);
  return (int)e;
}
