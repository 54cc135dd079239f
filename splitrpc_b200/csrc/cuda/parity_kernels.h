// Launch API of the GPU header processor, the reference-format LeNet and the LSTM wavefront kernel.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

// Turns n request headers into reply headers in place (swap MAC/IP/port, clear checksums, recompute the UDP
// pseudo-header checksum, optionally clear the low half of the sockperf word).  Either an array of header
// pointers or one contiguous array of 64-byte headers.
cudaError_t srpc_swap_hdrs(void* const* d_hdr_ptrs, void* d_hdrs_contig, int n, int clear_sockperf, cudaStream_t s);

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
