// Launch API of the GPU header processor, the reference-format LeNet and the LSTM wavefront kernel.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

// Turns n request headers into reply headers in place (swap MAC/IP/port, clear checksums, recompute the UDP
// pseudo-header checksum, optionally clear the low half of the sockperf word).  Either an array of header
// pointers or one contiguous array of 64-byte headers.
cudaError_t srpc_swap_hdrs(void* const* d_hdr_ptrs, void* d_hdrs_contig, int n, int clear_sockperf, cudaStream_t s);

// GPU header-processing API of the original (reference src/transport/g_udp_handler.cuh:8-24): a context that turns
// bursts of request headers living in GPU-visible memory into reply headers, either with one kernel launch per burst
// (launch type 1) or through a resident kernel behind a doorbell (launch type 2, the default, env
// P2P_RPC_G_PP_LAUNCH_TYPE).  Unlike the original's resident kernel this one leaves after an idle limit
// (P2P_RPC_G_PP_IDLE_MS) and is launched again on demand, and do_g_pp returns a status because its wait is bounded:
// 0 ok, -1 the wait ran out, -2 the resident kernel could not be (re)started, -3 CUDA error.
struct p2p_hbufs;
struct pp_params {
  uint64_t hdr_ptrs[1024];
  uint32_t num_items;
  uint32_t clear_sockperf;
};
struct pp_handler_ctx;
pp_handler_ctx* setup_g_pp(int device = 0, int launch_type = -1);
int do_g_pp(pp_handler_ctx* ctx, const p2p_hbufs* h_wi, int clear_sockperf = 0);
void stop_g_pp(pp_handler_ctx* ctx);
void g_pp_counters(const pp_handler_ctx* ctx, uint64_t* bursts, uint64_t* rearmed, uint64_t* timeouts, int* launch_type);

// 20/50/10 LeNet on uint8 28x28 images; reads requests / writes 10 fp32 probabilities through the stub or directly.
cudaError_t srpc_lenet_ref(const void* d_stub, const void* direct_in, float* direct_out, const float* c1, const float* c2,
                           const float* fc, const float* fb, int batch, cudaStream_t s);

// 8-layer x 8-step LSTM, hidden 256.  weights: per layer W[4][256][256], U[4][256][256], b[4][256] (gate order
// input, cell, forget, output).  scratch: srpc_lstm_scratch_bytes(max_clusters) bytes.
size_t srpc_lstm_scratch_bytes(int max_clusters);
cudaError_t srpc_lstm(const void* d_stub, const float* direct_in, float* direct_out, const float* weights, float* scratch,
                      int max_clusters, int batch, float forget_bias, cudaStream_t s);

// Loads this file's kernels on the current device, so that none of them is loaded lazily at a first launch that
// happens while a stream is parked on a doorbell.
void srpc_parity_preload();
