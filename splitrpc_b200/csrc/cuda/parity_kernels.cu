// Remaining device-side pieces of the original system, rebuilt for sm_100a:
//   swap_hdrs        reply-header construction on the GPU for headers that live in
//                    GPU-visible memory (reference src/transport/g_udp_handler.cu:96-178)
//   lenet_ref        the 20/50/10 LeNet of reference src/apps/lenet/lenet_vanilla.cu:17-192
//                    (uint8 pixels, (x-127)/128, conv 5x5 pad 1, tanh, 2x2 max pool, dense, softmax)
//                    as one kernel per batch instead of twelve launches per image
//   lstm_wavefront   the 8-layer x 8-step stacked LSTM (hidden 256) of reference
//                    src/apps/nnfusion_lstm/nnfusion_rt.cu:13870-13877,1213-1283 as one
//                    cluster launch per batch: the 8 blocks of a cluster own one layer
//                    each and advance along anti-diagonals with a cluster barrier per step
//                    (32 launches per inference in the original)
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <math.h>

#include "../host/p2p_rpc.h"
#include "../host/p2p_rpc_app.h"
#include "parity_kernels.h"
#include "ptx.cuh"

namespace cg = cooperative_groups;

namespace {

// ------------------------------------------------------------------ header swap
__global__ void swap_hdrs_kernel(p2p_rpc_hdr* const* hdrs, int n, int clear_sockperf) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  p2p_rpc_hdr* h = hdrs[i];
  swap_eth_hdr(h);
  if (clear_sockperf) set_sockperf_header(h);
  add_udp_cksum(h);
}

__global__ void swap_hdrs_contig_kernel(p2p_rpc_hdr* hdrs, int n, int clear_sockperf) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  p2p_rpc_hdr* h = hdrs + i;
  swap_eth_hdr(h);
  if (clear_sockperf) set_sockperf_header(h);
  add_udp_cksum(h);
}

// Resident header processor (launch type 2 of the GPU header-processing API): one block stays on the GPU and serves
// bursts of header pointers that the host posts in a mapped control block.  The doorbell is a sequence number, every
// poll also looks at the exit flag and the idle limit, and a burst is acknowledged by publishing its number in `done`.
__global__ void __launch_bounds__(1024) persistent_swap_hdrs(pp_params* stub, volatile uint32_t* door_bell, volatile uint32_t* done,
                                                             volatile uint32_t* exit_flag, volatile uint32_t* exited,
                                                             uint64_t idle_ns) {
  __shared__ uint32_t s_cmd, s_seq, s_n;
  uint32_t seen = *done;
  uint64_t last = ptx::globaltimer_ns();
  for (;;) {
    if (threadIdx.x == 0) {
      uint32_t cmd = 0;
      for (int spin = 0; spin < 4096; spin++) {
        if (ptx::ld_relaxed_sys(exit_flag) || ptx::globaltimer_ns() - last > idle_ns) {
          cmd = 2;
          break;
        }
        const uint32_t db = ptx::ld_acquire_sys(door_bell);
        if ((int32_t)(db - seen) > 0) {
          s_seq = db;
          s_n = ptx::ld_relaxed_sys(reinterpret_cast<const volatile uint32_t*>(&stub->num_items));
          cmd = 1;
          break;
        }
        __nanosleep(200);
      }
      s_cmd = cmd;
    }
    __syncthreads();
    const uint32_t cmd = s_cmd, seq = s_seq;
    uint32_t n = s_n;
    __syncthreads();
    if (cmd == 2) break;
    if (cmd == 0) continue;
    seen = seq;
    if (n > MAX_BI_SIZE) n = MAX_BI_SIZE;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
      p2p_rpc_hdr* h = reinterpret_cast<p2p_rpc_hdr*>(ptx::ld_relaxed_sys_u64(reinterpret_cast<const uint64_t*>(&stub->hdr_ptrs[i])));
      swap_eth_hdr(h);
      if (stub->clear_sockperf) set_sockperf_header(h);
      add_udp_cksum(h);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      ptx::st_release_sys(done, seen);
      last = ptx::globaltimer_ns();
    }
  }
  if (threadIdx.x == 0) ptx::st_release_sys(exited, 1u);
}

__global__ void swap_hdrs_stub_kernel(const pp_params* stub) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= stub->num_items) return;
  p2p_rpc_hdr* h = reinterpret_cast<p2p_rpc_hdr*>(stub->hdr_ptrs[i]);
  swap_eth_hdr(h);
  if (stub->clear_sockperf) set_sockperf_header(h);
  add_udp_cksum(h);
}

// ------------------------------------------------------------------ reference-format LeNet
struct LenetRefW {
  const float *c1, *c2, *fc, *fb;
};

// A cluster of eight blocks per image.
//   conv1   every block computes an eighth of the 20 x 13 x 13 pooled outputs (one thread each: the four window
//           positions from a 6 x 6 patch of the zero-bordered image, the 25 weights in registers) and stores them into
//           all eight blocks' copies through distributed shared memory;
//   conv2   2.5 of the 2.9 million multiply-adds of an inference.  Every block takes 6 or 7 of the 50 filters, weights
//           staged in shared memory once per block.  A warp is one pooled pixel; its lanes are (filter, quarter of the
//           input channels), so that the 6 x 6 input patch is a broadcast read and the weights fall into 28 different
//           banks; the quarters meet in shared-memory atomics.  0.6 shared-memory reads per multiply-add;
//   fc      every block multiplies its own 150 or 175 pooled values into the ten logits and adds them to block 0's,
//           block 0 writes the softmax.
// tanh is monotonic, so it is taken once, after the max over the window.  (One block per image with a thread per pooled
// output and weights read from global memory took 420 us per image, a cluster of four with redundant conv1 52 us.)
constexpr int LENET_REF_THREADS = 1024;
constexpr int LENET_REF_CLUSTER = 8;
constexpr int LENET_REF_KMAX = 7;      // filters of the second convolution per block (7, 7, 6, 6, 6, 6, 6, 6)
constexpr int LENET_P1_CH = 15 * 15;   // one zero-bordered 13 x 13 map

__device__ __forceinline__ float tanh_fast(float v) { return 1.f - __fdividef(2.f, 1.f + __expf(2.f * v)); }

__global__ void __cluster_dims__(LENET_REF_CLUSTER, 1, 1) __launch_bounds__(LENET_REF_THREADS, 1)
lenet_ref_kernel(const g_params* stub, const uint8_t* direct_in, float* direct_out, LenetRefW w, int batch) {
  cg::cluster_group cluster = cg::this_cluster();
  const int q = (int)cluster.block_rank();
  const int k_lo = q * 6 + (q < 2 ? q : 2), k_n = q < 2 ? 7 : 6;
  __shared__ __align__(16) float wc2[LENET_REF_KMAX * 500];  // [k_n][20][5][5]
  __shared__ float c2o[LENET_REF_KMAX * 100];                // [pixel][filter][2][2]: conv2 sums before max and tanh
  __shared__ float xp[30 * 32];                              // image with a zero border, rows 32 apart
  __shared__ float p1[20 * LENET_P1_CH];                     // conv1 output with a zero border
  __shared__ float p2[LENET_REF_KMAX * 25];
  __shared__ float lg[10];  // block 0: the logits
  __shared__ float wc1[500];
  const int t = threadIdx.x, warp = t / 32, lane = t % 32;
  for (int i = t; i < 500; i += LENET_REF_THREADS) wc1[i] = w.c1[i];
  for (int i = t; i < k_n * 125; i += LENET_REF_THREADS)
    reinterpret_cast<float4*>(wc2)[i] = __ldg(reinterpret_cast<const float4*>(w.c2 + (size_t)k_lo * 500) + i);
  for (int i = t; i < 30 * 32; i += LENET_REF_THREADS) xp[i] = 0.f;
  for (int i = t; i < 20 * LENET_P1_CH; i += LENET_REF_THREADS) p1[i] = 0.f;
  const uint8_t* in_base = direct_in ? direct_in : stub->req;
  float* out_base = direct_out ? direct_out : reinterpret_cast<float*>(stub->resp);
  float* lg_block0 = cluster.map_shared_rank(lg, 0);
  const int n_clusters = gridDim.x / LENET_REF_CLUSTER;
  cluster.sync();  // nobody stores into a block's p1 before that block has zeroed it
  for (int b = blockIdx.x / LENET_REF_CLUSTER; b < batch; b += n_clusters) {
    const uint8_t* in = in_base + (size_t)b * 784;
    float* out = out_base + (size_t)b * 10;
    if (t < 784) xp[(t / 28 + 1) * 32 + t % 28 + 1] = ((float)in[t] - 127.f) / 128.f;
    if (t < LENET_REF_KMAX * 100) c2o[t] = 0.f;
    if (q == 0 && t < 10) lg[t] = w.fb[t];
    __syncthreads();
    // conv1 (1->20, 5x5, pad 1: 28->26) + 2x2 max pool (->13) + tanh: this block's eighth, stored into every block
    {
      const int o = q * 423 + t;
      if (t < 423 && o < 20 * 169) {
        const int k = o / 169, r = (o % 169) / 13, c = o % 13;
        float wk[25];
#pragma unroll
        for (int i = 0; i < 25; i++) wk[i] = wc1[k * 25 + i];
        const float* xs = xp + (2 * r) * 32 + 2 * c;
        float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;
#pragma unroll
        for (int i = 0; i < 6; i++)
#pragma unroll
          for (int j = 0; j < 6; j++) {
            const float v = xs[i * 32 + j];
            if (i < 5 && j < 5) a00 += v * wk[i * 5 + j];
            if (i < 5 && j > 0) a01 += v * wk[i * 5 + j - 1];
            if (i > 0 && j < 5) a10 += v * wk[(i - 1) * 5 + j];
            if (i > 0 && j > 0) a11 += v * wk[(i - 1) * 5 + j - 1];
          }
        const float v = tanh_fast(fmaxf(fmaxf(a00, a01), fmaxf(a10, a11)));
        const int at = k * LENET_P1_CH + (r + 1) * 15 + c + 1;
#pragma unroll
        for (int d = 0; d < LENET_REF_CLUSTER; d++) cluster.map_shared_rank(p1, d)[at] = v;
      }
    }
    cluster.sync();  // every block holds the whole conv1 output
    // conv2 (20->50, 5x5, pad 1: 13->11) at the 10 x 10 positions that the pooling uses
    if (warp < 25) {
      const int pix = warp, quarter = lane & 3, kk = lane >> 2, r = pix / 5, c = pix % 5;
      if (kk < k_n) {
        float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;
        for (int ch = quarter * 5; ch < quarter * 5 + 5; ch++) {
          const float* ps = p1 + ch * LENET_P1_CH + (2 * r) * 15 + 2 * c;
          const float* wk = wc2 + (kk * 20 + ch) * 25;
#pragma unroll
          for (int i = 0; i < 6; i++)
#pragma unroll
            for (int j = 0; j < 6; j++) {
              const float v = ps[i * 15 + j];
              if (i < 5 && j < 5) a00 += v * wk[i * 5 + j];
              if (i < 5 && j > 0) a01 += v * wk[i * 5 + j - 1];
              if (i > 0 && j < 5) a10 += v * wk[(i - 1) * 5 + j];
              if (i > 0 && j > 0) a11 += v * wk[(i - 1) * 5 + j - 1];
            }
        }
        float* dst = c2o + (pix * LENET_REF_KMAX + kk) * 4;
        atomicAdd(dst, a00);
        atomicAdd(dst + 1, a01);
        atomicAdd(dst + 2, a10);
        atomicAdd(dst + 3, a11);
      }
    }
    __syncthreads();
    // 2x2 max pool + tanh, in the classifier's order [filter][pixel]
    if (t < k_n * 25) {
      const int kk = t / 25, pix = t % 25;
      const float* qv = c2o + (pix * LENET_REF_KMAX + kk) * 4;
      p2[t] = tanh_fast(fmaxf(fmaxf(qv[0], qv[1]), fmaxf(qv[2], qv[3])));
    }
    __syncthreads();
    // this block's share of the ten logits: one warp per output
    if (warp < 10) {
      float acc = 0.f;
      const float* fw = w.fc + warp * 1250 + k_lo * 25;
      for (int i = lane; i < k_n * 25; i += 32) acc += p2[i] * __ldg(fw + i);
      for (int sh = 16; sh; sh >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sh);
      if (lane == 0) atomicAdd(lg_block0 + warp, acc);
    }
    cluster.sync();  // all shares are in; p1, c2o and p2 are free for the next image
    if (q == 0 && t == 0) {
      float m = lg[0];
      for (int i = 1; i < 10; i++) m = fmaxf(m, lg[i]);
      float e[10], sum = 0.f;
      for (int i = 0; i < 10; i++) {
        e[i] = expf(lg[i] - m);
        sum += e[i];
      }
      for (int i = 0; i < 10; i++) out[i] = e[i] / sum;
    }
    __syncthreads();  // block 0: the logits are read before the next image's bias goes in
  }
  cluster.sync();  // no block leaves while another may still store into its shared memory
}

// ------------------------------------------------------------------ LSTM wavefront
constexpr int LH = 256, LLAYERS = 8, LSTEPS = 8;

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + __expf(-v)); }

// One cluster (8 blocks) per request; block l owns layer l.  At wave w block l computes cell (l, t = w - l):
//   gates = W_l . in + U_l . h_prev + b_l   (in = request step t for layer 0, else h of layer l-1 at step t)
// Layer outputs cross blocks through a small global scratch [request][layer][step][256]; the cluster barrier
// between waves orders the writes of wave w before the reads of wave w+1.
__global__ void __cluster_dims__(LLAYERS, 1, 1) __launch_bounds__(1024)
lstm_wavefront_kernel(const g_params* stub, const float* direct_in, float* direct_out, const float* __restrict__ weights,
                      float* __restrict__ scratch, int batch, float forget_bias) {
  cg::cluster_group cluster = cg::this_cluster();
  const int l = (int)cluster.block_rank();
  __shared__ float s_in[LH], s_h[LH], s_c[LH], s_g[4 * LH];
  const int t = threadIdx.x;
  const size_t per_layer = (size_t)8 * LH * LH + 4 * LH;
  const float* W = weights + (size_t)l * per_layer;
  const float* U = W + (size_t)4 * LH * LH;
  const float* B = U + (size_t)4 * LH * LH;
  const int n_clusters = gridDim.x / LLAYERS;
  const float* in_base = direct_in ? direct_in : reinterpret_cast<const float*>(stub->req);
  float* out_base = direct_out ? direct_out : reinterpret_cast<float*>(stub->resp);
  for (int req = blockIdx.x / LLAYERS; req < batch; req += n_clusters) {
    const float* x = in_base + (size_t)req * LSTEPS * LH;
    float* y = out_base + (size_t)req * LH;
    float* sc = scratch + (size_t)(blockIdx.x / LLAYERS) * LLAYERS * LSTEPS * LH;
    if (t < LH) {
      s_h[t] = 0.f;
      s_c[t] = 0.f;
    }
    __syncthreads();
    for (int w = 0; w < LLAYERS + LSTEPS - 1; w++) {
      const int step = w - l;
      if (step >= 0 && step < LSTEPS) {
        if (t < LH) s_in[t] = (l == 0) ? x[step * LH + t] : sc[((l - 1) * LSTEPS + step) * LH + t];
        __syncthreads();
        // 1024 threads = 4 gates x 256 outputs; each thread one dot product of length 512
        {
          const int g = t >> 8, o = t & 255;
          const float4* wr = reinterpret_cast<const float4*>(W + ((size_t)g * LH + o) * LH);
          const float4* ur = reinterpret_cast<const float4*>(U + ((size_t)g * LH + o) * LH);
          float acc = B[g * LH + o];
#pragma unroll 4
          for (int k = 0; k < LH / 4; k++) {
            const float4 a = __ldg(wr + k), b = __ldg(ur + k);
            acc += a.x * s_in[4 * k] + a.y * s_in[4 * k + 1] + a.z * s_in[4 * k + 2] + a.w * s_in[4 * k + 3];
            acc += b.x * s_h[4 * k] + b.y * s_h[4 * k + 1] + b.z * s_h[4 * k + 2] + b.w * s_h[4 * k + 3];
          }
          s_g[t] = acc;
        }
        __syncthreads();
        if (t < LH) {
          const float ig = s_g[t], gg = s_g[LH + t], fg = s_g[2 * LH + t], og = s_g[3 * LH + t];
          const float c = sigmoidf_(fg + forget_bias) * s_c[t] + sigmoidf_(ig) * tanhf(gg);
          const float h = tanhf(c) * sigmoidf_(og);
          s_c[t] = c;
          s_h[t] = h;
          sc[(l * LSTEPS + step) * LH + t] = h;
          if (l == LLAYERS - 1 && step == LSTEPS - 1) y[t] = h;
        }
        __syncthreads();
      }
      cluster.sync();
    }
  }
}

// ------------------------------------------------------------------ LSTM, whole-GPU wavefront
// The cluster kernel above gives a layer one SM, whose threads each walk one 1 KB weight row: a wave takes 74 us.  Here
// every wave is spread over the whole GPU.  A work item is (layer, hidden unit): a warp loads the unit's four gate
// rows of W and U (8 KB, coalesced 16-byte loads, kept in registers), then for every request of the group forms the
// four dot products with the layer's input and previous hidden state, reduces them across the warp and lets lane 0
// update the unit's cell and hidden state.  Up to eight requests share one pass over the weights; larger batches are
// served group after group.  Waves are separated by a grid-wide barrier (the kernel is launched cooperatively, so all
// blocks are resident; the wait on the barrier word is bounded).  Layer outputs of a wave live in hbuf[wave parity],
// which the next wave reads as input (layer below) and as previous state (same layer).
constexpr int LSTM_GROUP = 8;
constexpr long long LSTM_BARRIER_CYCLES = 4000000000ll;

struct LstmGridArgs {
  const g_params* stub;
  const float* direct_in;
  float* direct_out;
  const float* weights;
  float* hbuf;        // [2][LLAYERS][LSTM_GROUP][LH]
  float* cbuf;        // [LLAYERS][LSTM_GROUP][LH]
  unsigned* counter;  // zeroed before the launch
  uint32_t* status;   // may be null
  int batch;
  float forget_bias;
};

__device__ __forceinline__ float dot4(const float4& a, const float4& b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }

__global__ void __launch_bounds__(256) lstm_grid_kernel(const LstmGridArgs a) {
  __shared__ unsigned s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * 8 + warp, nw = gridDim.x * 8;
  const float* in_base = a.direct_in ? a.direct_in : reinterpret_cast<const float*>(a.stub->req);
  float* out_base = a.direct_out ? a.direct_out : reinterpret_cast<float*>(a.stub->resp);
  const size_t per_layer = (size_t)8 * LH * LH + 4 * LH;
  unsigned target = 0;
  for (int g0 = 0; g0 < a.batch; g0 += LSTM_GROUP) {
    const int nb = a.batch - g0 < LSTM_GROUP ? a.batch - g0 : LSTM_GROUP;
    for (int d = 0; d < LLAYERS + LSTEPS - 1; d++) {
      const int l_lo = d - (LSTEPS - 1) > 0 ? d - (LSTEPS - 1) : 0, l_hi = d < LLAYERS - 1 ? d : LLAYERS - 1;
      const int n_items = (l_hi - l_lo + 1) * LH;
      const float* h_read = a.hbuf + (size_t)((d + 1) & 1) * LLAYERS * LSTM_GROUP * LH;  // what wave d-1 wrote
      float* h_write = a.hbuf + (size_t)(d & 1) * LLAYERS * LSTM_GROUP * LH;
      for (int it = gw; it < n_items; it += nw) {
        const int l = l_lo + it / LH, j = it % LH, t = d - l;
        const float* W = a.weights + (size_t)l * per_layer;
        const float* U = W + (size_t)4 * LH * LH;
        const float* B = U + (size_t)4 * LH * LH;
        float4 w[4][2], u[4][2];
#pragma unroll
        for (int g = 0; g < 4; g++) {
          const float4* wr = reinterpret_cast<const float4*>(W + ((size_t)g * LH + j) * LH);
          w[g][0] = __ldg(wr + lane);
          w[g][1] = __ldg(wr + 32 + lane);
          if (t > 0) {
            const float4* ur = reinterpret_cast<const float4*>(U + ((size_t)g * LH + j) * LH);
            u[g][0] = __ldg(ur + lane);
            u[g][1] = __ldg(ur + 32 + lane);
          } else {
            u[g][0] = u[g][1] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        const float bi = B[j], bg = B[LH + j], bf = B[2 * LH + j] + a.forget_bias, bo = B[3 * LH + j];
        for (int b = 0; b < nb; b++) {
          const float4* xv = l == 0 ? reinterpret_cast<const float4*>(in_base + ((size_t)(g0 + b) * LSTEPS + t) * LH)
                                    : reinterpret_cast<const float4*>(h_read + ((size_t)(l - 1) * LSTM_GROUP + b) * LH);
          const float4 x0 = __ldcg(xv + lane), x1 = __ldcg(xv + 32 + lane);
          float sum[4];
#pragma unroll
          for (int g = 0; g < 4; g++) sum[g] = dot4(w[g][0], x0) + dot4(w[g][1], x1);
          if (t > 0) {
            const float4* hv = reinterpret_cast<const float4*>(h_read + ((size_t)l * LSTM_GROUP + b) * LH);
            const float4 h0 = __ldcg(hv + lane), h1 = __ldcg(hv + 32 + lane);
#pragma unroll
            for (int g = 0; g < 4; g++) sum[g] += dot4(u[g][0], h0) + dot4(u[g][1], h1);
          }
#pragma unroll
          for (int o = 16; o; o >>= 1) {
#pragma unroll
            for (int g = 0; g < 4; g++) sum[g] += __shfl_xor_sync(0xffffffffu, sum[g], o);
          }
          if (lane == 0) {
            float* cp = a.cbuf + ((size_t)l * LSTM_GROUP + b) * LH + j;
            const float c_prev = t > 0 ? *cp : 0.f;
            const float c = sigmoidf_(sum[2] + bf) * c_prev + sigmoidf_(sum[0] + bi) * tanhf(sum[1] + bg);
            const float h = tanhf(c) * sigmoidf_(sum[3] + bo);
            *cp = c;
            h_write[((size_t)l * LSTM_GROUP + b) * LH + j] = h;
            if (l == LLAYERS - 1 && t == LSTEPS - 1) out_base[(size_t)(g0 + b) * LH + j] = h;
          }
        }
      }
      // grid-wide barrier, bounded
      __syncthreads();
      if (threadIdx.x == 0) {
        target += gridDim.x;
        __threadfence();
        atomicAdd(a.counter, 1u);
        unsigned ok = 1;
        const long long t0 = clock64();
        while ((int)(ptx::ld_acquire_gpu(a.counter) - target) < 0) {
          if (clock64() - t0 > LSTM_BARRIER_CYCLES) {
            ok = 0;
            break;
          }
        }
        s_ok = ok;
      }
      __syncthreads();
      if (!s_ok) {
        if (threadIdx.x == 0 && a.status) atomicExch(a.status, 0x4C53u);  // 'LS': the LSTM's grid barrier ran out
        return;
      }
    }
  }
}

}  // namespace

cudaError_t srpc_swap_hdrs(void* const* d_hdr_ptrs, void* d_hdrs_contig, int n, int clear_sockperf, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  if (d_hdr_ptrs) swap_hdrs_kernel<<<(n + 255) / 256, 256, 0, s>>>((p2p_rpc_hdr* const*)d_hdr_ptrs, n, clear_sockperf);
  else swap_hdrs_contig_kernel<<<(n + 255) / 256, 256, 0, s>>>((p2p_rpc_hdr*)d_hdrs_contig, n, clear_sockperf);
  return cudaGetLastError();
}

cudaError_t srpc_lenet_ref(const void* d_stub, const void* direct_in, float* direct_out, const float* c1, const float* c2,
                           const float* fc, const float* fb, int batch, cudaStream_t s) {
  LenetRefW w{c1, c2, fc, fb};
  if (batch <= 0) return cudaSuccess;
  const int clusters = batch < 16 ? batch : 16;  // 16 clusters of eight blocks of 1024 threads fill the 148 SMs
  lenet_ref_kernel<<<LENET_REF_CLUSTER * clusters, LENET_REF_THREADS, 0, s>>>((const g_params*)d_stub, (const uint8_t*)direct_in, direct_out, w, batch);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ GPU header-processing API
struct pp_handler_ctx {
  pp_params* h_stub = nullptr;  // mapped pinned: the burst the host posts
  pp_params* d_stub = nullptr;
  volatile uint32_t* h_words = nullptr;  // [0] doorbell, [1] done, [2] exit flag, [3] exited
  uint32_t* d_words = nullptr;
  cudaStream_t g_stream = nullptr;
  uint8_t launch_type = 0;  // 0 none, 1 one kernel launch per burst, 2 resident kernel
  int device = 0;
  uint32_t seq = 0;
  bool resident = false;
  uint64_t idle_ns = 200000000ull, wait_ns = 2000000000ull;
  uint64_t bursts = 0, rearmed = 0, timeouts = 0;
};

static bool g_pp_stop_resident(pp_handler_ctx* c) {
  if (!c->resident) return true;
  __atomic_store_n(&c->h_words[2], 1u, __ATOMIC_RELEASE);
  const uint64_t t0 = getCurNs();
  while (__atomic_load_n(&c->h_words[3], __ATOMIC_ACQUIRE) == 0) {
    if (getCurNs() - t0 > c->wait_ns) return false;
  }
  cudaStreamSynchronize(c->g_stream);
  c->resident = false;
  return true;
}
static bool g_pp_ensure_resident(pp_handler_ctx* c) {
  if (c->resident && __atomic_load_n(&c->h_words[3], __ATOMIC_ACQUIRE) == 0) return true;
  if (!g_pp_stop_resident(c)) return false;  // it left after its idle limit: collect it, then launch again
  if (c->bursts) c->rearmed++;
  c->h_words[0] = c->seq;
  c->h_words[1] = c->seq;
  c->h_words[2] = 0;
  c->h_words[3] = 0;
  std::atomic_thread_fence(std::memory_order_seq_cst);
  persistent_swap_hdrs<<<1, 1024, 0, c->g_stream>>>(c->d_stub, c->d_words, c->d_words + 1, c->d_words + 2, c->d_words + 3, c->idle_ns);
  if (cudaGetLastError() != cudaSuccess) return false;
  c->resident = true;
  return true;
}

pp_handler_ctx* setup_g_pp(int device, int launch_type) {
  if (launch_type < 0) launch_type = (int)readEnvInfo<uint16_t>("P2P_RPC_G_PP_LAUNCH_TYPE", 2);
  if (cudaSetDevice(device) != cudaSuccess) return nullptr;
  srpc_parity_preload();
  pp_handler_ctx* c = new pp_handler_ctx;
  c->device = device;
  c->launch_type = (uint8_t)((launch_type == 1 || launch_type == 2) ? launch_type : 0);
  c->idle_ns = (uint64_t)readEnvInfo<uint64_t>("P2P_RPC_G_PP_IDLE_MS", 200) * 1000000ull;
  void *h = nullptr, *w = nullptr;
  if (cudaStreamCreateWithFlags(&c->g_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaHostAlloc(&h, sizeof(pp_params), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess ||
      cudaHostAlloc(&w, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    delete c;
    return nullptr;
  }
  std::memset(h, 0, sizeof(pp_params));
  std::memset(w, 0, 64);
  c->h_stub = (pp_params*)h;
  c->h_words = (volatile uint32_t*)w;
  cudaHostGetDevicePointer((void**)&c->d_stub, h, 0);
  cudaHostGetDevicePointer((void**)&c->d_words, w, 0);
  if (c->launch_type == 2 && !g_pp_ensure_resident(c)) c->launch_type = 1;
  return c;
}

int do_g_pp(pp_handler_ctx* c, const p2p_hbufs* h_wi, int clear_sockperf) {
  if (!c || c->launch_type == 0 || !h_wi || h_wi->num_items == 0) return 0;
  cudaSetDevice(c->device);
  const uint32_t n = h_wi->num_items;
  for (uint32_t i = 0; i < n; i++) c->h_stub->hdr_ptrs[i] = h_wi->burst_items[i];
  c->h_stub->num_items = n;
  c->h_stub->clear_sockperf = (uint32_t)clear_sockperf;
  std::atomic_thread_fence(std::memory_order_release);
  c->bursts++;
  if (c->launch_type == 2) {
    for (int attempt = 0; attempt < 2; attempt++) {
      if (!g_pp_ensure_resident(c)) return -2;
      const uint32_t s = ++c->seq;
      __atomic_store_n(&c->h_words[0], s, __ATOMIC_RELEASE);
      const uint64_t t0 = getCurNs();
      bool gone = false;
      for (;;) {
        if (__atomic_load_n(&c->h_words[1], __ATOMIC_ACQUIRE) == s) return 0;
        if (__atomic_load_n(&c->h_words[3], __ATOMIC_ACQUIRE) != 0) {
          gone = true;
          break;
        }
        if (getCurNs() - t0 > c->wait_ns) break;
      }
      // it left (idle limit) around the doorbell, or the wait ran out: stop it for good before anything else.  A header
      // swap is not idempotent, so the burst is only repeated when the kernel left without having touched it.
      const bool served = __atomic_load_n(&c->h_words[1], __ATOMIC_ACQUIRE) == s;
      if (!g_pp_stop_resident(c)) return -2;
      if (served || __atomic_load_n(&c->h_words[1], __ATOMIC_ACQUIRE) == s) return 0;
      if (!gone) {
        c->timeouts++;
        return -1;
      }
    }
    c->timeouts++;
    return -1;
  }
  swap_hdrs_stub_kernel<<<(n + 255) / 256, 256, 0, c->g_stream>>>(c->d_stub);
  if (cudaGetLastError() != cudaSuccess) return -3;
  return cudaStreamSynchronize(c->g_stream) == cudaSuccess ? 0 : -3;
}

void g_pp_counters(const pp_handler_ctx* c, uint64_t* bursts, uint64_t* rearmed, uint64_t* timeouts, int* launch_type) {
  *bursts = c->bursts;
  *rearmed = c->rearmed;
  *timeouts = c->timeouts;
  *launch_type = c->launch_type;
}

void stop_g_pp(pp_handler_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  g_pp_stop_resident(c);
  cudaStreamSynchronize(c->g_stream);
  cudaStreamDestroy(c->g_stream);
  cudaFreeHost(c->h_stub);
  cudaFreeHost((void*)c->h_words);
  delete c;
}

void srpc_parity_preload() {
  cudaFuncAttributes fa;
  (void)cudaFuncGetAttributes(&fa, persistent_swap_hdrs);
  (void)cudaFuncGetAttributes(&fa, swap_hdrs_stub_kernel);
  (void)cudaFuncGetAttributes(&fa, swap_hdrs_kernel);
  (void)cudaFuncGetAttributes(&fa, swap_hdrs_contig_kernel);
  (void)cudaFuncGetAttributes(&fa, lenet_ref_kernel);
  (void)cudaFuncGetAttributes(&fa, lstm_wavefront_kernel);
  (void)cudaFuncGetAttributes(&fa, lstm_grid_kernel);
  (void)cudaGetLastError();
}

static constexpr size_t kLstmHbufFloats = (size_t)2 * LLAYERS * LSTM_GROUP * LH, kLstmCbufFloats = (size_t)LLAYERS * LSTM_GROUP * LH;
static size_t lstm_grid_scratch_bytes() { return (kLstmHbufFloats + kLstmCbufFloats) * sizeof(float) + 256; }

size_t srpc_lstm_scratch_bytes(int max_clusters) {
  const size_t cluster_form = (size_t)max_clusters * LLAYERS * LSTEPS * LH * sizeof(float);
  return cluster_form > lstm_grid_scratch_bytes() ? cluster_form : lstm_grid_scratch_bytes();
}

cudaError_t srpc_lstm(const void* d_stub, const float* direct_in, float* direct_out, const float* weights, float* scratch,
                      int max_clusters, int batch, float forget_bias, cudaStream_t s) {
  if (batch < 1) return cudaSuccess;
  // Whole-GPU wavefront (cooperative launch); SPLITRPC_LSTM_CLUSTER=1 or a refused cooperative launch falls back to
  // the one-cluster-per-request kernel.
  static const int use_cluster = [] { const char* e = getenv("SPLITRPC_LSTM_CLUSTER"); return e ? atoi(e) : 0; }();
  static int grid_blocks = 0;
  if (!use_cluster) {
    if (!grid_blocks) {
      int dev = 0, sms = 0, per_sm = 0, coop = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lstm_grid_kernel, 256, 0);
      grid_blocks = (coop && sms > 0 && per_sm > 0) ? sms : -1;
    }
    if (grid_blocks > 0) {
      LstmGridArgs a;
      a.stub = (const g_params*)d_stub;
      a.direct_in = direct_in;
      a.direct_out = direct_out;
      a.weights = weights;
      a.hbuf = scratch;
      a.cbuf = scratch + kLstmHbufFloats;
      a.counter = reinterpret_cast<unsigned*>(scratch + kLstmHbufFloats + kLstmCbufFloats);
      a.status = nullptr;
      a.batch = batch;
      a.forget_bias = forget_bias;
      cudaError_t e = cudaMemsetAsync(a.counter, 0, sizeof(unsigned), s);
      if (e != cudaSuccess) return e;
      void* args[] = {&a};
      e = cudaLaunchCooperativeKernel((const void*)lstm_grid_kernel, dim3((unsigned)grid_blocks), dim3(256), args, 0, s);
      if (e == cudaSuccess) return cudaSuccess;
      (void)cudaGetLastError();
      grid_blocks = -1;  // not possible on this device or in this context: use the cluster kernel from now on
    }
  }
  int clusters = batch < max_clusters ? batch : max_clusters;
  if (clusters < 1) return cudaSuccess;
  lstm_wavefront_kernel<<<clusters * LLAYERS, 1024, 0, s>>>((const g_params*)d_stub, direct_in, direct_out, weights, scratch,
                                                           batch, forget_bias);
  return cudaGetLastError();
}
