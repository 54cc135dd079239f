// Memory-bound layers around the tensor-core kernels: request deserialisation,
// pooling, normalisation, softmax/argmax response writers, embedding and attention.
//
// These stand in for the cuDNN/TensorRT layers the original reaches through ONNX
// Runtime (reference src/apps/ort_app.h:511-516).  Activations are bf16 (NHWC for
// images, [tokens, hidden] for sequences); statistics are computed in fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../host/p2p_rpc_app.h"
#include "nn_kernels.h"
#include "per_device.h"
#include "ptx.cuh"
#include "resp_push.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int s = 16; s; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}

// Block-wide sum of one value per thread (blockDim.x <= 1024, multiple of 32).
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < nw) ? sh[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------ ResNet stem input
// Request = fp32 CHW image (3 x 224 x 224).  Writes the im2col matrix of the 7x7
// stride-2 pad-3 stem convolution: row = output pixel (n, oy, ox), 192 bf16
// columns ordered k = ky*24 + c*8 + kx (kx = 7 and k >= 168 are zero), after
// (x - mean[c]) * inv_std[c].  With this order one 16-byte chunk of a row is 7
// consecutive input pixels of one image row and channel, so a thread reads 28
// contiguous bytes and writes one 16-byte store.
__global__ void __launch_bounds__(256) stem_im2col(const g_params* stub, const float* __restrict__ direct_in, int batch,
                                                   __nv_bfloat16* __restrict__ out, float3 mean, float3 inv_std) {
  const float* in = direct_in ? direct_in : reinterpret_cast<const float*>(stub->req);
  const size_t total = (size_t)batch * 112 * 112 * 24;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int kc = (int)(i % 24);
    const size_t pix = i / 24;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (kc < 21) {
      const int ky = kc / 3, c = kc - ky * 3;
      const int ox = (int)(pix % 112), oy = (int)((pix / 112) % 112), n = (int)(pix / (112 * 112));
      const int iy = oy * 2 - 3 + ky, ix0 = ox * 2 - 3;
      if (iy >= 0 && iy < 224) {
        const float m = c == 0 ? mean.x : (c == 1 ? mean.y : mean.z);
        const float s = c == 0 ? inv_std.x : (c == 1 ? inv_std.y : inv_std.z);
        const float* row = in + (((size_t)n * 3 + c) * 224 + iy) * 224;
        float v[8];
#pragma unroll
        for (int j = 0; j < 7; j++) {
          const int ix = ix0 + j;
          v[j] = (ix >= 0 && ix < 224) ? (__ldg(row + ix) - m) * s : 0.f;
        }
        v[7] = 0.f;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int t = 0; t < 4; t++) h[t] = __floats2bfloat162_rn(v[2 * t], v[2 * t + 1]);
      }
    }
    *reinterpret_cast<uint4*>(out + pix * 192 + kc * 8) = o;
  }
}

// Space-to-depth form of the stem input.  The 7x7 stride-2 pad-3 convolution over 3 channels equals a 4x4 stride-1
// convolution over the 2x2 space-to-depth transform of the zero-padded (230 x 230) image.  Writes
// out[n][Y][X][16] bf16 with Y, X < 115 and channel dy*8 + dx*3 + c = normalised input pixel (2Y+dy-3, 2X+dx-3) of
// channel c (zero outside the image; channels 6, 7, 14, 15 are zero).  Four horizontally adjacent pixels are 64
// contiguous channels, so the convolution reads its rows straight from this array through a tensor map whose pixel
// stride is 16 elements: no im2col matrix is ever written (27 MB per 64 images instead of 308 MB).
__global__ void __launch_bounds__(256) stem_s2d(const g_params* stub, const float* __restrict__ direct_in, int batch,
                                                __nv_bfloat16* __restrict__ out, float3 mean, float3 inv_std) {
  const float* in = direct_in ? direct_in : reinterpret_cast<const float*>(stub->req);
  const size_t total = (size_t)batch * 115 * 115 * 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int dy = (int)(i & 1);
    const size_t pix = i >> 1;
    const int X = (int)(pix % 115), Y = (int)((pix / 115) % 115), n = (int)(pix / (115 * 115));
    const int iy = 2 * Y + dy - 3, ix0 = 2 * X - 3;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = 0.f;
    if (iy >= 0 && iy < 224) {
#pragma unroll
      for (int c = 0; c < 3; c++) {
        const float m = c == 0 ? mean.x : (c == 1 ? mean.y : mean.z);
        const float s = c == 0 ? inv_std.x : (c == 1 ? inv_std.y : inv_std.z);
        const float* row = in + (((size_t)n * 3 + c) * 224 + iy) * 224;
#pragma unroll
        for (int dx = 0; dx < 2; dx++) {
          const int ix = ix0 + dx;
          if (ix >= 0 && ix < 224) v[dx * 3 + c] = (__ldg(row + ix) - m) * s;
        }
      }
    }
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int t = 0; t < 4; t++) h[t] = __floats2bfloat162_rn(v[2 * t], v[2 * t + 1]);
    *reinterpret_cast<uint4*>(out + pix * 16 + dy * 8) = o;
  }
}

// 3x3 stride-2 pad-1 max pooling, NHWC bf16, 8 channels per thread.  Window positions outside the image are clamped
// to the nearest pixel inside (a duplicate does not change a maximum), so the nine 16-byte loads of a thread carry no
// branches and are all in flight together.
__global__ void __launch_bounds__(256) maxpool3x3s2(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                                    int n, int h, int w, int c) {
  const int oh = (h + 2 - 3) / 2 + 1, ow = (w + 2 - 3) / 2 + 1, cv = c / 8;
  const size_t total = (size_t)n * oh * ow * cv;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int cc = (int)(i % cv);
    size_t p = i / cv;
    const int ox = (int)(p % ow);
    p /= ow;
    const int oy = (int)(p % oh), b = (int)(p / oh);
    uint4 q[9];
#pragma unroll
    for (int dy = 0; dy < 3; dy++) {
      const int iy = min(max(oy * 2 - 1 + dy, 0), h - 1);
#pragma unroll
      for (int dx = 0; dx < 3; dx++) {
        const int ix = min(max(ox * 2 - 1 + dx, 0), w - 1);
        q[dy * 3 + dx] = __ldg(reinterpret_cast<const uint4*>(in + (((size_t)b * h + iy) * w + ix) * c + cc * 8));
      }
    }
    __nv_bfloat162 m[4];
    {
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&q[0]);
#pragma unroll
      for (int t = 0; t < 4; t++) m[t] = h0[t];
    }
#pragma unroll
    for (int k = 1; k < 9; k++) {
      const __nv_bfloat162* hq = reinterpret_cast<const __nv_bfloat162*>(&q[k]);
#pragma unroll
      for (int t = 0; t < 4; t++) m[t] = __hmax2(m[t], hq[t]);
    }
    uint4 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int t = 0; t < 4; t++) ho[t] = m[t];
    *reinterpret_cast<uint4*>(out + (((size_t)b * oh + oy) * ow + ox) * c + cc * 8) = o;
  }
}

// Global average pooling NHWC -> [n, c]; block (x = channel chunk of 512, y = image), two channels per thread, the
// pixel loop unrolled so that several loads are in flight.
__global__ void __launch_bounds__(256) global_avgpool(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                                      int hw, int c) {
  const int b = blockIdx.y, ch = (blockIdx.x * 256 + threadIdx.x) * 2;
  if (ch >= c) return;
  const __nv_bfloat16* src = in + (size_t)b * hw * c + ch;
  float s0 = 0.f, s1 = 0.f;
  int p = 0;
  for (; p + 7 <= hw; p += 7) {
    __nv_bfloat162 v[7];
#pragma unroll
    for (int j = 0; j < 7; j++) v[j] = *reinterpret_cast<const __nv_bfloat162*>(src + (size_t)(p + j) * c);
#pragma unroll
    for (int j = 0; j < 7; j++) {
      float2 f = __bfloat1622float2(v[j]);
      s0 += f.x;
      s1 += f.y;
    }
  }
  for (; p < hw; p++) {
    float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + (size_t)p * c));
    s0 += f.x;
    s1 += f.y;
  }
  *reinterpret_cast<__nv_bfloat162*>(out + (size_t)b * c + ch) = __floats2bfloat162_rn(s0 / hw, s1 / hw);
}

// Skinny fully connected layer: out[m, n] = sum_k a[m, k] * w[n, k] + bias[n] for a handful of rows, fp32 output.  A
// tensor-core tile would be 128 rows x 64 columns: with 64 rows that leaves 16 CTAs each walking all of K.  Here a
// block owns FC_NB output columns and FC_ROWS rows: the weight rows are staged in shared memory as fp32 once (two
// planes of float4 per column, so that the sixteen k-slices a warp reads together are contiguous), thread
// (row pair, kq) walks every sixteenth 8-element slice of its two rows of `a` with the next slice's loads in flight, and
// the sixteen partial sums of a row meet through shuffles.
constexpr int FC_NB = 8, FC_ROWS = 32;
__global__ void __launch_bounds__(256, 2) fc_skinny(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w,
                                                 int ldw, const float* __restrict__ bias, float* __restrict__ out, int ldo, int M,
                                                 int N, int K) {
  extern __shared__ __align__(16) float4 s_w[];  // [FC_NB][2][K/8]
  const int n0 = blockIdx.x * FC_NB, kvn = K / 8;
  for (int base = 0; base < FC_NB * kvn; base += 256 * 8) {
    uint4 q[8];  // eight loads in flight per thread: the weights usually come from DRAM
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int i = base + u * 256 + threadIdx.x, col = i / kvn, kv = i - col * kvn;
      q[u] = make_uint4(0, 0, 0, 0);
      if (i < FC_NB * kvn && n0 + col < N) q[u] = __ldg(reinterpret_cast<const uint4*>(w + (size_t)(n0 + col) * ldw + kv * 8));
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int i = base + u * 256 + threadIdx.x, col = i / kvn, kv = i - col * kvn;
      const __nv_bfloat162* hq = reinterpret_cast<const __nv_bfloat162*>(&q[u]);
      const float2 f0 = __bfloat1622float2(hq[0]), f1 = __bfloat1622float2(hq[1]), f2 = __bfloat1622float2(hq[2]),
                   f3 = __bfloat1622float2(hq[3]);
      if (i < FC_NB * kvn) {
        s_w[(col * 2) * kvn + kv] = make_float4(f0.x, f0.y, f1.x, f1.y);
        s_w[(col * 2 + 1) * kvn + kv] = make_float4(f2.x, f2.y, f3.x, f3.y);
      }
    }
  }
  __syncthreads();
  const int kq = threadIdx.x & 15;
  const int row0 = blockIdx.y * FC_ROWS + (threadIdx.x >> 4) * 2;
  // rows past M read row M-1 again (their results are not stored): no branch inside the loop
  const __nv_bfloat16* ar0 = a + (size_t)min(row0, M - 1) * lda;
  const __nv_bfloat16* ar1 = a + (size_t)min(row0 + 1, M - 1) * lda;
  // packed fp32 FMAs (two per instruction): lane x of an accumulator sums the even k, lane y the odd k
  float2 acc0[FC_NB], acc1[FC_NB];
#pragma unroll
  for (int j = 0; j < FC_NB; j++) acc0[j] = acc1[j] = make_float2(0.f, 0.f);
  auto step = [&](const uint4& c0, const uint4& c1, int kv) {
    float2 x0[4], x1[4];
    const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&c0);
    const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&c1);
#pragma unroll
    for (int t = 0; t < 4; t++) {
      x0[t] = __bfloat1622float2(h0[t]);
      x1[t] = __bfloat1622float2(h1[t]);
    }
#pragma unroll
    for (int j = 0; j < FC_NB; j++) {
      const float4 w0 = s_w[(j * 2) * kvn + kv], w1 = s_w[(j * 2 + 1) * kvn + kv];
      const float2 wa = make_float2(w0.x, w0.y), wb = make_float2(w0.z, w0.w), wc = make_float2(w1.x, w1.y),
                   wd = make_float2(w1.z, w1.w);
      acc0[j] = __ffma2_rn(x0[0], wa, acc0[j]);
      acc1[j] = __ffma2_rn(x1[0], wa, acc1[j]);
      acc0[j] = __ffma2_rn(x0[1], wb, acc0[j]);
      acc1[j] = __ffma2_rn(x1[1], wb, acc1[j]);
      acc0[j] = __ffma2_rn(x0[2], wc, acc0[j]);
      acc1[j] = __ffma2_rn(x1[2], wc, acc1[j]);
      acc0[j] = __ffma2_rn(x0[3], wd, acc0[j]);
      acc1[j] = __ffma2_rn(x1[3], wd, acc1[j]);
    }
  };
  auto load = [&](const __nv_bfloat16* r, int kv) {
    return kv < kvn ? __ldg(reinterpret_cast<const uint4*>(r + kv * 8)) : make_uint4(0, 0, 0, 0);
  };
  // two slices per trip, the next trip's four loads issued before this trip's arithmetic
  uint4 qa0 = load(ar0, kq), qa1 = load(ar1, kq), qb0 = load(ar0, kq + 16), qb1 = load(ar1, kq + 16);
  for (int kv = kq; kv < kvn; kv += 32) {
    const uint4 ca0 = qa0, ca1 = qa1, cb0 = qb0, cb1 = qb1;
    qa0 = load(ar0, kv + 32);
    qa1 = load(ar1, kv + 32);
    qb0 = load(ar0, kv + 48);
    qb1 = load(ar1, kv + 48);
    step(ca0, ca1, kv);
    if (kv + 16 < kvn) step(cb0, cb1, kv + 16);
  }
  float s0[FC_NB], s1[FC_NB];
#pragma unroll
  for (int j = 0; j < FC_NB; j++) {
    s0[j] = acc0[j].x + acc0[j].y;
    s1[j] = acc1[j].x + acc1[j].y;
#pragma unroll
    for (int d = 1; d < 16; d <<= 1) {
      s0[j] += __shfl_xor_sync(0xffffffffu, s0[j], d);
      s1[j] += __shfl_xor_sync(0xffffffffu, s1[j], d);
    }
  }
  // lane kq stores column kq & 7 of row kq >> 3
#pragma unroll
  for (int j = 0; j < FC_NB; j++) {
    if ((kq & 7) == j && n0 + j < N) {
      const int row = row0 + (kq >> 3);
      if (row < M) out[(size_t)row * ldo + n0 + j] = ((kq >> 3) ? s1[j] : s0[j]) + (bias ? bias[n0 + j] : 0.f);
    }
  }
}

// ------------------------------------------------------------------ response writers
// Softmax over `n` fp32 logits per row written as fp32 into the response slot of
// each request (stub->resp + row * resp_stride), optionally followed by the
// argmax class as int32.  When `flag` is set, the block that finishes last
// publishes `flag_value` with a system-scope release store: the response is in
// place (possibly in a peer GPU's or the host's memory) before the flag is seen.
// With a response-push block (`push`, see resp_push.cuh) each row goes straight to
// the place the producer named for its slot (the ingress transmit arena, in another
// process's pinned memory or on a peer GPU) and the row's block completes the slot.
__global__ void __launch_bounds__(256) softmax_response(const float* __restrict__ logits, int n, int ld, const g_params* stub,
                                                        uint8_t* direct_out, size_t resp_stride, int write_argmax,
                                                        uint32_t* counter, volatile uint32_t* flag, uint32_t flag_value,
                                                        const RespPushCtx* push) {
  __shared__ float sh[32];
  __shared__ float s_max, s_sum;
  __shared__ int s_arg;
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ld;
  // One thread reads the stub and the push block (mapped host memory: every read is a PCIe round trip) for the block.
  __shared__ RespPushTarget s_target;
  if (threadIdx.x == 0) {
    uint8_t* b = (direct_out ? direct_out : stub->resp) + (size_t)row * resp_stride;
    s_target = (!direct_out && push) ? resp_push_target(push, (uint32_t)row, b) : RespPushTarget{b, nullptr, nullptr};
  }
  __syncthreads();
  const RespPushTarget target = s_target;
  uint8_t* base = target.dst;
  float m = -FLT_MAX;
  int am = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    if (x[i] > m) {
      m = x[i];
      am = i;
    }
  // block arg-max
  float wm = warp_max(m);
  unsigned ball = __ballot_sync(0xffffffffu, m == wm);
  int src = __ffs(ball) - 1;
  int wam = __shfl_sync(0xffffffffu, am, src);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __shared__ int sh_i[32];
  if (l == 0) {
    sh[w] = wm;
    sh_i[w] = wam;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bm = sh[0];
    int bi = sh_i[0];
    for (int k = 1; k < nw; k++)
      if (sh[k] > bm) {
        bm = sh[k];
        bi = sh_i[k];
      }
    s_max = bm;
    s_arg = bi;
  }
  __syncthreads();
  const float mx = s_max;
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += __expf(x[i] - mx);
  s = block_sum(s, sh);
  if (threadIdx.x == 0) s_sum = s;
  __syncthreads();
  const float inv = 1.f / s_sum;
  float* o = reinterpret_cast<float*>(base);
  for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = __expf(x[i] - mx) * inv;
  if (write_argmax && threadIdx.x == 0) reinterpret_cast<int*>(base)[n] = s_arg;
  if (target.state) {
    __syncthreads();
    if (threadIdx.x == 0) resp_push_complete(target);
  }
  if (flag) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t prev = atomicAdd(counter, 1u);
      if (prev + 1 == gridDim.x) {
        atomicExch(counter, 0u);
        __threadfence_system();
        ptx::st_release_sys(flag, flag_value);
      }
    }
  }
}

// ------------------------------------------------------------------ LayerNorm (+ residual)
// y = LN(x + residual) * gamma + beta, one row per block; hidden <= 8 * blockDim.x.
__global__ void __launch_bounds__(256) layernorm_rows(const __nv_bfloat16* __restrict__ x,
                                                      const __nv_bfloat16* __restrict__ residual,
                                                      const float* __restrict__ gamma, const float* __restrict__ beta,
                                                      __nv_bfloat16* __restrict__ y, int hidden, float eps) {
  __shared__ float sh[32];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * hidden;
  const __nv_bfloat16* rr = residual ? residual + row * hidden : nullptr;
  float v[8];
  int cnt = 0;
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden && cnt < 8; i += blockDim.x, cnt++) {
    float f = __bfloat162float(xr[i]);
    if (rr) f += __bfloat162float(rr[i]);
    v[cnt] = f;
    s += f;
  }
  const float mean = block_sum(s, sh) / hidden;
  float q = 0.f;
  for (int k = 0; k < cnt; k++) q += (v[k] - mean) * (v[k] - mean);
  const float var = block_sum(q, sh) / hidden;
  const float rstd = rsqrtf(var + eps);
  cnt = 0;
  for (int i = threadIdx.x; i < hidden && cnt < 8; i += blockDim.x, cnt++)
    y[row * hidden + i] = __float2bfloat16((v[cnt] - mean) * rstd * gamma[i] + beta[i]);
}

// Warp-per-row LayerNorm for hidden sizes that are multiples of 256 (up to 2048): each lane owns hidden/32 values as
// 16-byte vectors, the row never leaves registers, and both reductions are warp shuffles.
template <int VPL>  // uint4 vectors per lane: hidden = VPL * 256
__global__ void __launch_bounds__(256) layernorm_rows_warp(const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ residual,
                                                           const float* __restrict__ gamma, const float* __restrict__ beta,
                                                           __nv_bfloat16* __restrict__ y, int rows, float eps) {
  constexpr int HIDDEN = VPL * 256;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * HIDDEN);
  const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + (size_t)row * HIDDEN) : nullptr;
  float v[VPL * 8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; i++) {
    uint4 q = xr[i * 32 + lane];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    uint4 q2 = rr ? rr[i * 32 + lane] : make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&q2);
#pragma unroll
    for (int t = 0; t < 4; t++) {
      float2 f = __bfloat1622float2(h[t]), g = __bfloat1622float2(h2[t]);
      v[i * 8 + 2 * t] = f.x + g.x;
      v[i * 8 + 2 * t + 1] = f.y + g.y;
      s += v[i * 8 + 2 * t] + v[i * 8 + 2 * t + 1];
    }
  }
  const float mean = warp_sum(s) * (1.f / HIDDEN);
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < VPL * 8; k++) q += (v[k] - mean) * (v[k] - mean);
  const float rstd = rsqrtf(warp_sum(q) * (1.f / HIDDEN) + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * HIDDEN);
#pragma unroll
  for (int i = 0; i < VPL; i++) {
    const int c0 = (i * 32 + lane) * 8;
    const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c0)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c0 + 4));
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + c0)), b1 = __ldg(reinterpret_cast<const float4*>(beta + c0 + 4));
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    uint4 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int t = 0; t < 4; t++)
      ho[t] = __floats2bfloat162_rn((v[i * 8 + 2 * t] - mean) * rstd * gg[2 * t] + bb[2 * t],
                                    (v[i * 8 + 2 * t + 1] - mean) * rstd * gg[2 * t + 1] + bb[2 * t + 1]);
    yr[i * 32 + lane] = o;
  }
}

// ------------------------------------------------------------------ BERT embedding
// Request = seq int32 token ids per sequence.  y[token] = LN(word[id] + pos[t] + type[0]).
// Reads ids through the stub (ring window) or from `direct_ids`.
__global__ void __launch_bounds__(256) bert_embed_ln(const g_params* stub, const int* __restrict__ direct_ids, size_t req_stride,
                                                     int seq, const __nv_bfloat16* __restrict__ word,
                                                     const __nv_bfloat16* __restrict__ pos,
                                                     const __nv_bfloat16* __restrict__ type, const float* __restrict__ gamma,
                                                     const float* __restrict__ beta, __nv_bfloat16* __restrict__ y, int hidden,
                                                     int vocab, float eps) {
  __shared__ float sh[32];
  const int tok = blockIdx.x, b = tok / seq, t = tok - b * seq;
  const int* ids = direct_ids ? direct_ids + (size_t)b * seq
                              : reinterpret_cast<const int*>(stub->req + (size_t)b * req_stride);
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  float v[8];
  int cnt = 0;
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden && cnt < 8; i += blockDim.x, cnt++) {
    float f = __bfloat162float(word[(size_t)id * hidden + i]) + __bfloat162float(pos[(size_t)t * hidden + i]) +
              __bfloat162float(type[i]);
    v[cnt] = f;
    s += f;
  }
  const float mean = block_sum(s, sh) / hidden;
  float q = 0.f;
  for (int k = 0; k < cnt; k++) q += (v[k] - mean) * (v[k] - mean);
  const float rstd = rsqrtf(block_sum(q, sh) / hidden + eps);
  cnt = 0;
  for (int i = threadIdx.x; i < hidden && cnt < 8; i += blockDim.x, cnt++)
    y[(size_t)tok * hidden + i] = __float2bfloat16((v[cnt] - mean) * rstd * gamma[i] + beta[i]);
}

// ------------------------------------------------------------------ attention (head dim 64)
// qkv: [tokens, 3*hidden] bf16 with q | k | v blocks; out: [tokens, hidden].
// One block = one (sequence, head, tile of 32 queries); K and V of the head sit in
// shared memory; one warp handles 4 queries at a time with fp32 accumulation.
// This is the simple SIMT form of the operator; it keeps every intermediate on chip.
template <int SEQ>
__global__ void __launch_bounds__(256) attention_d64(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out,
                                                     int heads, int ld_qkv, int q_off, int k_off, int v_off, int ld_out,
                                                     float scale) {
  extern __shared__ __align__(16) uint8_t att_smem[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(att_smem);        // [SEQ][64+2] padded rows
  __nv_bfloat16* sV = sK + SEQ * 66;                                     // [SEQ][64]
  float* sP = reinterpret_cast<float*>(sV + SEQ * 64);                   // [8 warps][SEQ]
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t tok0 = (size_t)b * SEQ;
  for (int i = threadIdx.x; i < SEQ * 32; i += blockDim.x) {
    const int r = i >> 5, c = (i & 31) * 2;
    const __nv_bfloat16* row = qkv + (tok0 + r) * ld_qkv + h * 64 + c;
    *reinterpret_cast<__nv_bfloat162*>(sK + r * 66 + c) = *reinterpret_cast<const __nv_bfloat162*>(row + k_off);
    *reinterpret_cast<__nv_bfloat162*>(sV + r * 64 + c) = *reinterpret_cast<const __nv_bfloat162*>(row + v_off);
  }
  __syncthreads();
  float* p = sP + warp * SEQ;
  for (int qi = warp; qi < 32; qi += 8) {
    const int q = qt * 32 + qi;
    if (q >= SEQ) break;
    const __nv_bfloat16* qrow = qkv + (tok0 + q) * ld_qkv + q_off + h * 64;
    float2 qv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qrow + lane * 2));
    // scores: each lane owns keys lane, lane+32, ...
    float mx = -FLT_MAX;
    for (int k0 = 0; k0 < SEQ; k0 += 32) {
      const int k = k0 + lane;
      float acc = 0.f;
#pragma unroll 8
      for (int d = 0; d < 64; d += 2) {
        float2 kv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sK + k * 66 + d));
        const float qx = __shfl_sync(0xffffffffu, qv.x, d >> 1), qy = __shfl_sync(0xffffffffu, qv.y, d >> 1);
        acc += qx * kv.x + qy * kv.y;
      }
      acc *= scale;
      p[k] = acc;
      mx = fmaxf(mx, acc);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int k = lane; k < SEQ; k += 32) {
      const float e = __expf(p[k] - mx);
      p[k] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    __syncwarp();
    // out: each lane owns dims 2*lane, 2*lane+1
    float o0 = 0.f, o1 = 0.f;
    for (int k = 0; k < SEQ; k++) {
      const float pk = p[k];
      float2 vv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sV + k * 64 + lane * 2));
      o0 += pk * vv.x;
      o1 += pk * vv.y;
    }
    const float inv = 1.f / sum;
    *reinterpret_cast<__nv_bfloat162*>(out + (tok0 + q) * ld_out + h * 64 + lane * 2) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
    __syncwarp();
  }
}

int grid_for(size_t total, int threads) {
  size_t b = (total + threads - 1) / threads;
  size_t cap = 148 * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

cudaError_t nn_stem_im2col(const void* d_stub, const float* direct_in, int batch, void* out, const float mean[3],
                           const float inv_std[3], cudaStream_t s) {
  size_t total = (size_t)batch * 112 * 112 * 24;
  stem_im2col<<<grid_for(total, 256), 256, 0, s>>>((const g_params*)d_stub, direct_in, batch, (__nv_bfloat16*)out,
                                                   make_float3(mean[0], mean[1], mean[2]),
                                                   make_float3(inv_std[0], inv_std[1], inv_std[2]));
  return cudaGetLastError();
}
cudaError_t nn_stem_s2d(const void* d_stub, const float* direct_in, int batch, void* out, const float mean[3],
                        const float inv_std[3], cudaStream_t s) {
  size_t total = (size_t)batch * 115 * 115 * 2;
  stem_s2d<<<grid_for(total, 256), 256, 0, s>>>((const g_params*)d_stub, direct_in, batch, (__nv_bfloat16*)out,
                                                make_float3(mean[0], mean[1], mean[2]),
                                                make_float3(inv_std[0], inv_std[1], inv_std[2]));
  return cudaGetLastError();
}
cudaError_t nn_maxpool3x3s2(const void* in, void* out, int n, int h, int w, int c, cudaStream_t s) {
  if (c % 8) return cudaErrorInvalidValue;
  int oh = (h - 1) / 2 + 1, ow = (w - 1) / 2 + 1;
  maxpool3x3s2<<<grid_for((size_t)n * oh * ow * (c / 8), 256), 256, 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, n,
                                                                          h, w, c);
  return cudaGetLastError();
}
cudaError_t nn_global_avgpool(const void* in, void* out, int n, int hw, int c, cudaStream_t s) {
  if (c % 2) return cudaErrorInvalidValue;
  global_avgpool<<<dim3((c + 511) / 512, n), 256, 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, hw, c);
  return cudaGetLastError();
}
cudaError_t nn_fc_skinny(const void* a, int lda, const void* w, int ldw, const float* bias, float* out, int ldo, int M, int N, int K,
                         cudaStream_t s) {
  const size_t smem = (size_t)FC_NB * K * sizeof(float);
  if (K % 8 || lda % 8 || ldw % 8 || (((uintptr_t)a | (uintptr_t)w) & 15) || smem > 200 * 1024 || M <= 0) return cudaErrorInvalidValue;
  static PerDeviceFlag attr_set;
  const int dev = PerDeviceFlag::current();
  if (attr_set.needed(dev)) {
    cudaError_t e = cudaFuncSetAttribute(fc_skinny, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_set.set(dev);
  }
  fc_skinny<<<dim3((N + FC_NB - 1) / FC_NB, (M + FC_ROWS - 1) / FC_ROWS), 256, smem, s>>>((const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w,
                                                                          ldw, bias, out, ldo, M, N, K);
  return cudaGetLastError();
}
cudaError_t nn_softmax_response(const float* logits, int rows, int n, int ld, const void* d_stub, void* direct_out,
                                size_t resp_stride, int write_argmax, uint32_t* counter, uint32_t* flag, uint32_t flag_value,
                                cudaStream_t s, const void* d_push) {
  if (rows <= 0) return cudaSuccess;
  softmax_response<<<rows, 256, 0, s>>>(logits, n, ld, (const g_params*)d_stub, (uint8_t*)direct_out, resp_stride,
                                        write_argmax, counter, flag, flag_value, (const RespPushCtx*)d_push);
  return cudaGetLastError();
}
cudaError_t nn_layernorm(const void* x, const void* residual, const float* gamma, const float* beta, void* y, int rows,
                         int hidden, float eps, cudaStream_t s) {
  if (hidden > 2048) return cudaErrorInvalidValue;
  const bool aligned = (((uintptr_t)x | (uintptr_t)y | (uintptr_t)residual | (uintptr_t)gamma | (uintptr_t)beta) & 15) == 0;
  const int grid = (rows + 7) / 8;
  const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *rp = (const __nv_bfloat16*)residual;
  __nv_bfloat16* yp = (__nv_bfloat16*)y;
  if (aligned && hidden == 768) layernorm_rows_warp<3><<<grid, 256, 0, s>>>(xp, rp, gamma, beta, yp, rows, eps);
  else if (aligned && hidden == 1024) layernorm_rows_warp<4><<<grid, 256, 0, s>>>(xp, rp, gamma, beta, yp, rows, eps);
  else if (aligned && hidden == 512) layernorm_rows_warp<2><<<grid, 256, 0, s>>>(xp, rp, gamma, beta, yp, rows, eps);
  else if (aligned && hidden == 256) layernorm_rows_warp<1><<<grid, 256, 0, s>>>(xp, rp, gamma, beta, yp, rows, eps);
  else layernorm_rows<<<rows, 256, 0, s>>>(xp, rp, gamma, beta, yp, hidden, eps);
  return cudaGetLastError();
}
cudaError_t nn_bert_embed_ln(const void* d_stub, const int* direct_ids, size_t req_stride, int batch, int seq, const void* word,
                             const void* pos, const void* type, const float* gamma, const float* beta, void* y, int hidden,
                             int vocab, float eps, cudaStream_t s) {
  if (hidden > 2048) return cudaErrorInvalidValue;
  bert_embed_ln<<<batch * seq, 256, 0, s>>>((const g_params*)d_stub, direct_ids, req_stride, seq, (const __nv_bfloat16*)word,
                                            (const __nv_bfloat16*)pos, (const __nv_bfloat16*)type, gamma, beta,
                                            (__nv_bfloat16*)y, hidden, vocab, eps);
  return cudaGetLastError();
}
cudaError_t nn_attention_d64(const void* qkv, void* out, int batch, int seq, int heads, int ld_qkv, int q_off, int k_off,
                             int v_off, int ld_out, cudaStream_t s) {
  const float scale = 0.125f;
  dim3 grid((seq + 31) / 32, heads, batch);
  if (seq == 128) {
    const int smem = 128 * 66 * 2 + 128 * 64 * 2 + 8 * 128 * 4;
    attention_d64<128><<<grid, 256, smem, s>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)out, heads, ld_qkv, q_off, k_off,
                                               v_off, ld_out, scale);
  } else if (seq == 384) {
    const int smem = 384 * 66 * 2 + 384 * 64 * 2 + 8 * 384 * 4;
    static PerDeviceFlag attr;
    const int dev = PerDeviceFlag::current();
    if (attr.needed(dev)) {
      cudaFuncSetAttribute(attention_d64<384>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      attr.set(dev);
    }
    attention_d64<384><<<grid, 256, smem, s>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)out, heads, ld_qkv, q_off, k_off,
                                               v_off, ld_out, scale);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}
