// Launch API of the tcgen05 GEMM / implicit-GEMM convolution kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "driver_api.h"

enum GemmAct { GEMM_ACT_NONE = 0, GEMM_ACT_RELU = 1, GEMM_ACT_GELU = 2, GEMM_ACT_TANH = 3 };
enum GemmErr {
  GEMM_OK = 0, GEMM_ERR_PRODUCER_WAIT = 1, GEMM_ERR_MMA_WAIT = 2, GEMM_ERR_EPILOGUE_WAIT = 3,
  GEMM_ERR_TP_SRC_WAIT = 4,     // a peer never published its shard
  GEMM_ERR_TP_BLOCK_WAIT = 5,   // a copier block never delivered a row block
  GEMM_ERR_TP_REDUCE_WAIT = 6,  // a source rank never delivered its partial tiles
};

// out[row, col] = act(acc + bias[col] + residual[row, col]); leading dimensions in elements.
struct GemmEpilogue {
  void* out = nullptr;
  int ldo = 0;
  int out_fp32 = 0;
  const float* bias = nullptr;
  const __nv_bfloat16* residual = nullptr;
  int ldr = 0;
  int act = GEMM_ACT_NONE;
};

struct ConvShape {
  int n, h, w, cin;     // input NHWC
  int cout, r, s;       // filter [cout][r][s][cin]
  int stride, pad;
  int oh, ow;
  // Input strides in elements; 0 = dense NHWC (pixel stride cin, row stride w*cin, image stride h*w*cin).  A pixel
  // stride smaller than cin makes neighbouring pixels overlap: a window of several narrow pixels is then read as one
  // 64-channel pixel without being copied first (TMA path only; every stride a multiple of 8 elements).
  long in_pix_stride = 0, in_row_stride = 0, in_img_stride = 0;
  // Input inside a request ring (TMA path): `in` is the ring base, in_ring_slots images of in_slot_bytes each are
  // addressable (both mappings of a double-mapped ring), and the batch starts at the slot that *(uint8_t**)in_stub
  // points to when the kernel runs.  in_img_stride must then equal in_slot_bytes / 2.
  const void* in_stub = nullptr;
  long in_ring_slots = 0;
  unsigned int in_slot_bytes = 0;
  // Second input of a two-input 1x1 convolution (TMA path, r = s = 1, pad = 0): dense NHWC [n, h2, w2, cin2] sampled
  // every stride2 pixels; the filter rows are then [cout][cin + cin2] and out = act(W1 . in + W2 . in2 + bias).  A
  // bottleneck's last convolution and its projection shortcut become one kernel this way.
  const void* in2 = nullptr;
  int h2 = 0, w2 = 0, cin2 = 0, stride2 = 1;
};

// D[M,N] = A[M,K] . B[N,K]^T, bf16 operands (row strides lda/ldb elements, multiples of 8), fp32 accumulation.
// `status` may be null; otherwise it receives a GemmErr code when a bounded wait ran out.
cudaError_t srpc_gemm_bf16(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                           uint32_t* status, cudaStream_t stream);

// Persistent variants (production path): double-buffered TMEM accumulators, TMA-store epilogue; the convolution
// reads its A operand with shifted 4-D TMA boxes instead of gathering rows.
cudaError_t srpc_gemm_bf16_v2(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                              uint32_t* status, cudaStream_t stream);
cudaError_t srpc_conv_bf16_tma(const void* in, const void* weight, const ConvShape& cs, const GemmEpilogue& ep,
                               uint32_t* status, cudaStream_t stream);

// Two-SM variant (CTA pairs, 256 x bn tiles with bn = 128, 192 or 256, tcgen05.mma.cta_group::2) for compute-bound
// shapes; bf16 output with 16-byte aligned rows only.  srpc_gemm_bf16_v2 selects it by itself; SPLITRPC_GEMM_2SM=0
// turns it off.
bool srpc_gemm_2sm_eligible(int M, int N, int K, const GemmEpilogue& ep);
cudaError_t srpc_gemm_bf16_2sm(const void* A, int lda, const void* B, int ldb, int M, int N, int K, int bn,
                               const GemmEpilogue& ep, uint32_t* status, cudaStream_t stream);

// Leaves `n` SMs out of the grids of the persistent kernels (see num_sms in gemm_persistent.cu); takes effect for
// launches (and graph captures) made afterwards.  srpc_gemm_grid_sms returns the SM count the grids are sized for.
void srpc_gemm_reserve_sms(int n);
int srpc_gemm_grid_sms();
int srpc_gemm_reserved_sms();

// Phase time stamps (ns, %globaltimer) of block 0 of the last persistent launch; returns 0 unless the library was
// built with -DSRPC_GEMM_TRACE.  Slots: 0 entry, 1 set-up done, 2 first loads issued, 3 first operands landed,
// 4 first tile's MMAs issued, 5 first accumulator ready, 6 first tile's store issued, 7 last epilogue done,
// 8 stores drained, 9 all warps done.
int srpc_gemm_trace_read(unsigned long long* out, int n);
// Same for the two-SM kernel; slots 10 and 11 = operands of k-blocks 8 and 24 of the first tile landed.
int srpc_gemm2_trace_read(unsigned long long* out, int n);

// NHWC bf16 convolution as an implicit GEMM; cin must be a multiple of 64.
cudaError_t srpc_conv_bf16(const void* in, const void* weight, const ConvShape& cs, const GemmEpilogue& ep,
                           uint32_t* status, cudaStream_t stream);
