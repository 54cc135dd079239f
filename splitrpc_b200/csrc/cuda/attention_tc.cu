// Multi-head attention (head dim 64, all-ones mask) on tcgen05 tensor cores.
//
// One CTA serves one (sequence, head) and loops over its 128-query tiles.
//   scores = Q . K^T      tcgen05.mma, M=128, N=128 per key block, K=64, fp32 in TMEM
//   P = softmax(scores)   four warps, one query row per thread, read from TMEM,
//                         written as bf16 into 128-byte-swizzled shared memory
//   O = P . V             tcgen05.mma, M=128, N=64, K=SEQ, fp32 in TMEM
// All operands arrive by TMA (no multicast) from this GPU's memory:
//   Q and K from the [tokens, 2*hidden] output of the fused Q|K projection,
//   V^T from the [hidden, tokens] output of the V projection computed with
//   swapped GEMM operands, so that it is already K-major for the second product.
// The V bias is added to the output instead (softmax rows sum to one).
// Replaces the attention subgraph the original runs inside ONNX Runtime
// (reference src/apps/ort_defs.h:141-190).  Waits are bounded; a timeout sets
// *status, the CTA stops, frees its tensor memory and returns.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>

#include "driver_api.h"
#include "nn_kernels.h"
#include "ptx.cuh"
#include "per_device.h"

namespace {

constexpr int HD = 64;          // head dim
constexpr int QT = 128;         // queries per tile
constexpr int ATT_THREADS = 160;  // warps 0-3 softmax/epilogue, warp 4 TMA + MMA issue

template <int SEQ>
struct AttSmem {
  static constexpr int Q_BYTES = QT * 128;            // 128 rows x 64 bf16
  static constexpr int K_BYTES = SEQ * 128;           // SEQ rows x 64 bf16
  static constexpr int VT_BYTES = (SEQ / 64) * 64 * 128;  // SEQ/64 atoms of 64 rows x 64 keys
  static constexpr int P_BYTES = (SEQ / 64) * QT * 128;   // SEQ/64 atoms of 128 rows x 64 keys
  // With a single query tile (SEQ == 128) Q and K are dead once the scores exist, and the scores are dead once P is
  // written: P takes the place of Q|K in shared memory and the output accumulator the place of the scores in tensor
  // memory.  48 KB and 128 columns per CTA let four CTAs share an SM, so every (sequence, head) of a 32 x 12 batch is
  // resident at once and the SM interleaves their load -> MMA -> softmax -> MMA chains.
  static constexpr bool ALIAS = SEQ == QT;
  static constexpr int P_OFFSET = ALIAS ? 0 : Q_BYTES + K_BYTES + VT_BYTES;
  static constexpr int TOTAL = ALIAS ? Q_BYTES + K_BYTES + VT_BYTES : Q_BYTES + K_BYTES + VT_BYTES + P_BYTES;
  static constexpr int TMEM_COLS = ALIAS ? 128 : ((SEQ + HD) <= 256 ? 256 : 512);
  static_assert(!ALIAS || P_BYTES <= Q_BYTES + K_BYTES, "P must fit over Q and K");
};

// VMN = true: V is read in place from the fused Q|K|V projection ([tokens, 3*hidden], V in the last third).  A V tile
// is then [keys, 64] with the head dimension contiguous, i.e. an MN-major B operand of the second product: same
// 128-byte-swizzled shared-memory tile and descriptor, "B is MN-major" in the instruction descriptor, and a step of 16
// keys along K is 2048 bytes (two 8-row groups) instead of 32.  No transposed copy of V and no separate V GEMM.
template <int SEQ, bool VMN>
__global__ void __launch_bounds__(ATT_THREADS)
attention_tc(const __grid_constant__ CUtensorMap tmap_qk, const __grid_constant__ CUtensorMap tmap_vt,
             __nv_bfloat16* __restrict__ out, int ld_out, const float* __restrict__ v_bias, int hidden, float scale_log2e,
             uint32_t* status) {
  using L = AttSmem<SEQ>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + L::Q_BYTES;
  uint8_t* sVT = sK + L::K_BYTES;
  uint8_t* sP = smem + L::P_OFFSET;
  __shared__ __align__(8) uint64_t bar_kv, bar_q, bar_s, bar_p, bar_o;
  __shared__ uint32_t tmem_base_smem;
  __shared__ uint32_t s_error;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x, seq_idx = blockIdx.y;
  const int tok0 = seq_idx * SEQ;
  constexpr int NQT = SEQ / QT;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar_kv, 1);
    ptx::mbar_init(&bar_q, 1);
    ptx::mbar_init(&bar_s, 1);
    ptx::mbar_init(&bar_p, 4);
    ptx::mbar_init(&bar_o, 1);
    ptx::fence_mbar_init();
    s_error = 0;
    ptx::prefetch_tmap(&tmap_qk);
    ptx::prefetch_tmap(&tmap_vt);
  }
  if (warp == 4) {
    ptx::tmem_alloc(&tmem_base_smem, L::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_s = tmem_base_smem;          // scores: columns [0, SEQ)
  const uint32_t tmem_o = tmem_base_smem + (L::ALIAS ? 0 : SEQ);  // output: columns [SEQ, SEQ+64), or over the scores

  if (warp == 4) {
    if (ptx::elect_one()) {
      // K and V^T of this head stay resident for all query tiles.
      ptx::mbar_expect_tx(&bar_kv, L::K_BYTES + L::VT_BYTES);
      for (int nb = 0; nb < SEQ / 128; nb++)
        ptx::tma_load_2d(sK + nb * 128 * 128, &tmap_qk, &bar_kv, hidden + head * HD, tok0 + nb * 128);
      if constexpr (VMN) {
        for (int nb = 0; nb < SEQ / 128; nb++)
          ptx::tma_load_2d(sVT + nb * 128 * 128, &tmap_qk, &bar_kv, 2 * hidden + head * HD, tok0 + nb * 128);
      } else {
        for (int a = 0; a < SEQ / 64; a++) ptx::tma_load_2d(sVT + a * 64 * 128, &tmap_vt, &bar_kv, tok0 + a * 64, head * HD);
      }
      bool ok = ptx::mbar_wait(&bar_kv, 0);
      const uint32_t idesc_s = ptx::umma_idesc_bf16(QT, 128);
      const uint32_t idesc_o = ptx::umma_idesc_bf16(QT, HD) | (VMN ? (1u << 16) : 0u);  // bit 16: B is MN-major
      for (int qt = 0; qt < NQT && ok; qt++) {
        const uint32_t ph = (uint32_t)qt & 1u;
        // Q tile (the previous tile's score MMAs have completed: bar_s was awaited by the softmax warps and
        // bar_o, which follows it, by this thread's successors; this thread itself waited bar_p below).
        ptx::mbar_expect_tx(&bar_q, L::Q_BYTES);
        ptx::tma_load_2d(sQ, &tmap_qk, &bar_q, head * HD, tok0 + qt * QT);
        if (!(ok = ptx::mbar_wait(&bar_q, ph))) break;
        ptx::tc_fence_after();
        const uint32_t q_addr = ptx::smem_u32(sQ), k_addr = ptx::smem_u32(sK);
        for (int nb = 0; nb < SEQ / 128; nb++)
#pragma unroll
          for (int k = 0; k < HD / 16; k++)
            ptx::umma_bf16(tmem_s + nb * 128, ptx::umma_desc_sw128(q_addr + k * 32),
                           ptx::umma_desc_sw128(k_addr + nb * 128 * 128 + k * 32), idesc_s, k != 0 ? 1u : 0u);
        ptx::umma_commit(&bar_s);
        // P ready (written by the softmax warps)
        if (!(ok = ptx::mbar_wait(&bar_p, ph))) break;
        ptx::tc_fence_after();
        const uint32_t p_addr = ptx::smem_u32(sP), vt_addr = ptx::smem_u32(sVT);
        for (int kk = 0; kk < SEQ / 16; kk++) {
          const int atom = kk >> 2, sub = kk & 3;
          const uint32_t v_desc_addr = VMN ? vt_addr + kk * 2048 : vt_addr + atom * 64 * 128 + sub * 32;
          ptx::umma_bf16(tmem_o, ptx::umma_desc_sw128(p_addr + atom * QT * 128 + sub * 32), ptx::umma_desc_sw128(v_desc_addr),
                         idesc_o, kk != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&bar_o);
      }
      if (!ok) atomicExch(&s_error, 1u);
    }
  } else {
    const int row = warp * 32 + lane;  // query row inside the tile; warp == TMEM lane quarter
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int qt = 0; qt < NQT; qt++) {
      const uint32_t ph = (uint32_t)qt & 1u;
      if (*(volatile uint32_t*)&s_error != 0 || !ptx::mbar_wait(&bar_s, ph)) {
        atomicExch(&s_error, 2u);
        break;
      }
      ptx::tc_fence_after();
      // pass 1: row maximum
      float mx = -3.0e38f;
#pragma unroll 1
      for (int c = 0; c < SEQ; c += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(tmem_s + lane_base + c, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j++) mx = fmaxf(mx, __uint_as_float(r[j]));
      }
      // pass 2: exponentials, row sum, P in bf16 to swizzled shared memory
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < SEQ; c += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(tmem_s + lane_base + c, r);
        ptx::tmem_ld_wait();
        uint8_t* prow = sP + (size_t)(c >> 6) * QT * 128 + (size_t)row * 128;
        const int chunk0 = (c & 63) >> 3;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint4 q;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const float e0 = exp2f((__uint_as_float(r[j * 8 + 2 * t]) - mx) * scale_log2e);
            const float e1 = exp2f((__uint_as_float(r[j * 8 + 2 * t + 1]) - mx) * scale_log2e);
            h[t] = __floats2bfloat162_rn(e0, e1);
            // the row sum uses the rounded values that the second product will see
            float2 back = __bfloat1622float2(h[t]);
            sum += back.x + back.y;
          }
          *reinterpret_cast<uint4*>(prow + (((chunk0 + j) ^ (row & 7)) << 4)) = q;
        }
      }
      ptx::tc_fence_before();
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar_p);
      // output tile
      if (!ptx::mbar_wait(&bar_o, ph)) {
        atomicExch(&s_error, 3u);
        break;
      }
      ptx::tc_fence_after();
      const float inv = 1.f / sum;
      __nv_bfloat16* orow = out + (size_t)(tok0 + qt * QT + row) * ld_out + head * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(tmem_o + lane_base + c, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint4 q;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const int d = c + j * 8 + 2 * t;
            const float b0 = v_bias ? __ldg(v_bias + head * HD + d) : 0.f;
            const float b1 = v_bias ? __ldg(v_bias + head * HD + d + 1) : 0.f;
            h[t] = __floats2bfloat162_rn(__uint_as_float(r[j * 8 + 2 * t]) * inv + b0,
                                         __uint_as_float(r[j * 8 + 2 * t + 1]) * inv + b1);
          }
          *reinterpret_cast<uint4*>(orow + c + j * 8) = q;
        }
      }
      ptx::tc_fence_before();
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (s_error != 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, 0x100u | s_error);
    __nanosleep(1000000);
    __syncthreads();
  }
  if (warp == 4) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base_smem, L::TMEM_COLS);
  }
}

cudaError_t encode(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t stride_bytes, uint32_t box_inner,
                   uint32_t box_outer) {
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->TensorMapEncodeTiled) return cudaErrorNotSupported;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t st[1] = {stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t es[2] = {1, 1};
  CUresult r = d->TensorMapEncodeTiled(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, st, box, es,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int SEQ, bool VMN>
cudaError_t launch(const CUtensorMap& tqk, const CUtensorMap& tvt, void* out, int ld_out, const float* v_bias, int hidden,
                   int batch, int heads, uint32_t* status, cudaStream_t s) {
  static PerDeviceFlag attr;
  const int dev = PerDeviceFlag::current();
  const int smem = AttSmem<SEQ>::TOTAL + 1024;
  if (attr.needed(dev)) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc<SEQ, VMN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr.set(dev);
  }
  const float scale_log2e = 0.125f * 1.4426950408889634f;
  attention_tc<SEQ, VMN><<<dim3(heads, batch), ATT_THREADS, smem, s>>>(tqk, tvt, (__nv_bfloat16*)out, ld_out, v_bias, hidden,
                                                                  scale_log2e, status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t nn_attention_tc(const void* qk, int ld_qk, const void* vt, int ld_vt, void* out, int ld_out, const float* v_bias,
                            int batch, int seq, int heads, uint32_t* status, cudaStream_t s) {
  const int hidden = heads * HD;
  const int tokens = batch * seq;
  if ((ld_qk % 8) || (ld_out % 8) || ((uintptr_t)qk & 15) || ((uintptr_t)out & 15)) return cudaErrorInvalidValue;
  CUtensorMap tqk, tvt;
  if (!vt) {  // V in place: qk is the [tokens, 3*hidden] output of the fused Q|K|V projection
    cudaError_t e = encode(&tqk, qk, (uint64_t)3 * hidden, (uint64_t)tokens, (uint64_t)ld_qk * 2, 64, 128);
    if (e != cudaSuccess) return e;
    if (seq == 128) return launch<128, true>(tqk, tqk, out, ld_out, v_bias, hidden, batch, heads, status, s);
    if (seq == 384) return launch<384, true>(tqk, tqk, out, ld_out, v_bias, hidden, batch, heads, status, s);
    return cudaErrorInvalidValue;
  }
  if ((ld_vt % 8) || ((uintptr_t)vt & 15)) return cudaErrorInvalidValue;
  cudaError_t e = encode(&tqk, qk, (uint64_t)2 * hidden, (uint64_t)tokens, (uint64_t)ld_qk * 2, 64, 128);
  if (e != cudaSuccess) return e;
  e = encode(&tvt, vt, (uint64_t)tokens, (uint64_t)hidden, (uint64_t)ld_vt * 2, 64, 64);
  if (e != cudaSuccess) return e;
  if (seq == 128) return launch<128, false>(tqk, tvt, out, ld_out, v_bias, hidden, batch, heads, status, s);
  if (seq == 384) return launch<384, false>(tqk, tvt, out, ld_out, v_bias, hidden, batch, heads, status, s);
  return cudaErrorInvalidValue;
}
