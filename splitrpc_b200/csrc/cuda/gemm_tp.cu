// Tensor-parallel GEMMs fused with their collectives over NVLink peer memory.
//
// The original system has no multi-GPU path at all (one device per process,
// reference src/utils/config_utils.h:42-44); these kernels are what lets one model
// span several B200s.  Both are the persistent tcgen05 GEMM (TMA-fed operands,
// TMEM accumulators, 128 x 128 tiles) with the collective folded in:
//
//  all-gather -> GEMM   D[T, N_local] = act(concat_r(X_r)[T, K] . W[N_local, K]^T + bias)
//    X is sharded by rows over the ranks.  A few "copier" blocks of the same launch
//    pull the remote shards over NVLink (rings of 16 KB bulk copies, no multicast)
//    into a local gathered buffer, one 128-row block at a time, and publish each
//    block with a release store; the GEMM blocks visit row blocks in rotated
//    order (own shard first) and their TMA producer waits (bounded) for a block's
//    flag before loading it from LOCAL memory.  So each remote byte crosses
//    NVLink once, and the transfer overlaps the math tile by tile.
//
//  GEMM -> reduce-scatter   P_r[T, N] = A_r[T, K_local] . W_r[N, K_local]^T,  D = sum_r P_r sharded by rows
//    Every rank computes partial tiles and its epilogue stores each finished tile
//    straight into the owner rank's slot for this source (peer stores, coalesced
//    16-byte vectors out of the shared-memory staging tile).  When a rank has
//    delivered all tiles of an owner it publishes a flag in that owner's memory
//    with a system-scope release.  The owner's reduction (sum of the slots + bias
//    + residual + LayerNorm, see layernorm_reduce) waits for the flags, so the
//    reduction itself is fused into the normalisation that follows.
//
// No load uses multicast; remote data is only touched by plain loads/stores and non-multicast bulk copies.
// Every wait on a flag (another block's or another rank's) is bounded: when it
// runs out the kernel records an error code and winds down.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "gemm_tcgen05.h"
#include "gemm_tp.h"
#include "ptx.cuh"
#include "per_device.h"
#include "tp_device.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64, UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int THREADS = 320;
constexpr int EPI_THREADS = 256;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int OUT_HALF_BYTES = BM * 128, OUT_BYTES = 2 * OUT_HALF_BYTES;

__device__ __forceinline__ float gelu_f(float x) { return ptx::gelu_erf_fast(x); }
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ bool named_bar_all(int id, int count, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %3, 0;\n\t"
      "barrier.cta.red.and.pred p, %1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(out)
      : "r"(id), "r"(count), "r"((uint32_t)pred)
      : "memory");
  return out != 0;
}

using tpdev::copier;
using tpdev::wait_flag_gpu;
using tpdev::wait_flag_sys;

__global__ void __launch_bounds__(THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_out, int M, int N, int K, GemmEpilogue ep, const TpParams tp_in,
               uint32_t* status) {
  TpParams tp = tp_in;
  if (tp.epoch_base) tp.epoch += *tp.epoch_base;
  const int gemm_ctas = (int)gridDim.x - tp.n_copy;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  if ((int)blockIdx.x >= gemm_ctas) {
    copier(tp, (int)blockIdx.x - gemm_ctas, smem, status);
    return;
  }
  uint8_t* stage_out = smem + (size_t)STAGES * STAGE_BYTES;
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ uint32_t s_error;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; a++) {
      ptx::mbar_init(&tmem_full_bar[a], 1);
      ptx::mbar_init(&tmem_empty_bar[a], 8);
    }
    ptx::fence_mbar_init();
    s_error = 0;
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_base_smem, 2 * BN);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  // Tile order: row blocks rotated so that this rank's own shard comes first.
  auto tile_mn = [&](int tile, int* m_idx, int* n_idx) {
    *n_idx = tile % tiles_n;
    *m_idx = (tile / tiles_n + tp.m_rot) % tiles_m;
  };

  if (warp == 0) {
    if (ptx::elect_one()) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && *(volatile uint32_t*)&s_error == 0; tile += gemm_ctas) {
        int m_idx, n_idx;
        tile_mn(tile, &m_idx, &n_idx);
        if (tp.mblock_ready) {
          // Remote row blocks arrive through the copier blocks of this launch.
          const int owner = m_idx / tp.mblocks_per_rank;
          if (owner != tp.rank) {
            if (!wait_flag_gpu(tp.mblock_ready + m_idx, tp.epoch)) {
              atomicExch(&s_error, GEMM_ERR_TP_BLOCK_WAIT);
              break;
            }
            ptx::fence_proxy_async_all();  // generic-proxy writes of the copier -> async-proxy (TMA) reads
          }
        }
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u)) {
            atomicExch(&s_error, GEMM_ERR_PRODUCER_WAIT);
            break;
          }
          uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
          ptx::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          ptx::tma_load_2d(sa, &tmap_a, &full_bar[s], kb * BK, m_idx * BM);
          ptx::tma_load_2d(sa + A_BYTES, &tmap_b, &full_bar[s], kb * BK, n_idx * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      const uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
      uint32_t it = 0, local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && *(volatile uint32_t*)&s_error == 0; tile += gemm_ctas, local++) {
        const uint32_t acc = local & 1u;
        if (!ptx::mbar_wait(&tmem_empty_bar[acc], ((local >> 1) & 1u) ^ 1u)) {
          atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait(&full_bar[s], ph)) {
            atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++)
            ptx::umma_bf16(d_tmem, ptx::umma_desc_sw128(sa + k * UMMA_K * 2), ptx::umma_desc_sw128(sb + k * UMMA_K * 2), idesc,
                           (kb | k) != 0 ? 1u : 0u);
          ptx::umma_commit(&empty_bar[s]);
        }
        if (!ok) break;
        ptx::umma_commit(&tmem_full_bar[acc]);
      }
    }
  } else {
    constexpr int CPW = BN / 2, NCH = CPW / 32;
    const int warp_q = warp & 3;
    const int chalf = (warp - 2) >> 2;
    const int row = warp_q * 32 + lane;
    const int et = threadIdx.x - 64;
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gemm_ctas, local++) {
      const uint32_t acc = local & 1u;
      int m_idx, n_idx;
      tile_mn(tile, &m_idx, &n_idx);
      const int n0 = n_idx * BN, cbase = chalf * CPW;
      const bool mine = (*(volatile uint32_t*)&s_error == 0) && ptx::mbar_wait(&tmem_full_bar[acc], (local >> 1) & 1u);
      if (!named_bar_all(2, EPI_THREADS, mine)) {
        if (lane == 0) atomicExch(&s_error, GEMM_ERR_EPILOGUE_WAIT);
        break;
      }
      ptx::tc_fence_after();
      uint32_t r[CPW];
#pragma unroll
      for (int ch = 0; ch < NCH; ch++)
        ptx::tmem_ld_32x32b_x32(tmem_base + acc * BN + ((uint32_t)(warp_q * 32) << 16) + (uint32_t)(cbase + ch * 32), r + ch * 32);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&tmem_empty_bar[acc]);
      uint8_t* sbuf = stage_out + (size_t)(local & 1u) * OUT_BYTES;
      if (!tp.rs) {
        if (et == 0) ptx::bulk_wait_read<1>();
      }
      named_bar_sync(1, EPI_THREADS);  // staging buffer free (TMA store drained, or the previous peer-store pass done)
#pragma unroll
      for (int ch = 0; ch < NCH; ch++) {
        const int c = cbase + ch * 32;
        const int col0 = n0 + c;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[ch * 32 + j]);
        if (ep.bias && col0 + 32 <= N) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 b4 = __ldg(reinterpret_cast<const float4*>(ep.bias + col0 + j));
            v[j] += b4.x;
            v[j + 1] += b4.y;
            v[j + 2] += b4.z;
            v[j + 3] += b4.w;
          }
        }
        if (ep.act == GEMM_ACT_GELU) {
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = gelu_f(v[j]);
        } else if (ep.act == GEMM_ACT_RELU) {
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = fmaxf(v[j], 0.f);
        }
        uint8_t* half = sbuf + (size_t)(c >> 6) * OUT_HALF_BYTES + (size_t)row * 128;
        const int chunk0 = (c & 63) >> 3;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint4 q;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
          for (int t = 0; t < 4; t++) h[t] = __floats2bfloat162_rn(v[j * 8 + 2 * t], v[j * 8 + 2 * t + 1]);
          *reinterpret_cast<uint4*>(half + (((chunk0 + j) ^ (row & 7)) << 4)) = q;
        }
      }
      if (!tp.rs) {
        ptx::fence_proxy_async_smem();
        named_bar_sync(1, EPI_THREADS);
        if (et == 0) {
          for (int hcol = 0; hcol < BN / 64; hcol++) {
            if (n0 + hcol * 64 >= N) break;
            ptx::tma_store_2d(&tmap_out, sbuf + (size_t)hcol * OUT_HALF_BYTES, n0 + hcol * 64, m_idx * BM);
          }
          ptx::bulk_commit();
        }
      } else {
        // Peer-store epilogue: the tile goes to the slot this rank owns on the row block's owner.
        named_bar_sync(1, EPI_THREADS);
        const int owner = m_idx / tp.mblocks_per_rank;
        const int local_m0 = (m_idx - owner * tp.mblocks_per_rank) * BM;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(tp.dst[owner]);
        // 16 threads write one 256-byte row segment; 16 rows per pass
        const int seg = et & 15, r0 = et >> 4;
#pragma unroll 2
        for (int rr = r0; rr < BM; rr += EPI_THREADS / 16) {
          const int col = n0 + seg * 8;
          if (col < N) {
            const uint8_t* src = sbuf + (size_t)(seg >> 3) * OUT_HALF_BYTES + (size_t)rr * 128 + (((seg & 7) ^ (rr & 7)) << 4);
            uint4 q = *reinterpret_cast<const uint4*>(src);
            *reinterpret_cast<uint4*>(dst + (size_t)(local_m0 + rr) * ep.ldo + col) = q;
          }
        }
        // one cumulative system-scope fence behind the barrier covers every thread's stores of the tile
        named_bar_sync(1, EPI_THREADS);
        if (et == 0) {
          __threadfence_system();
          const uint32_t done = atomicAdd(tp.owner_count + owner, 1u) + 1u;
          if (done == (uint32_t)tp.tiles_per_owner) {
            atomicExch(tp.owner_count + owner, 0u);
            __threadfence_system();
            ptx::st_release_sys(tp.dst_flag[owner], tp.epoch);
          }
        }
      }
    }
    if (!tp.rs && et == 0) ptx::bulk_wait_all<0>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (s_error != 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, s_error);
    __nanosleep(1000000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 2 * BN);
  }
}

cudaError_t map_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                   uint32_t box_inner, uint32_t box_outer) {
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->TensorMapEncodeTiled) return cudaErrorNotSupported;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t st[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t es[2] = {1, 1};
  CUresult r = d->TensorMapEncodeTiled(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, st, box, es,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Signals every peer that this rank's shard for `epoch` is complete.
__global__ void tp_signal_peers(TpSignal sig) {
  const int p = threadIdx.x;
  if (p < sig.tp) {
    const uint32_t e = sig.epoch + (sig.epoch_base ? *sig.epoch_base : 0u);
    __threadfence_system();
    ptx::st_release_sys(sig.peer_flag[p], e);
  }
}

__device__ __forceinline__ void reduce_signal(const TpReduce& rd);

// y = LN(sum_r slot_r[row] + bias + residual) * gamma + beta; waits (bounded) until every source rank has
// published `epoch` in flags[r].
__global__ void __launch_bounds__(256) layernorm_reduce(TpReduce rd, uint32_t* status) {
  __shared__ float sh[32];
  __shared__ uint32_t s_ok;
  if (threadIdx.x == 0) {
    uint32_t ok = 1;
    const uint32_t e = rd.epoch + (rd.epoch_base ? *rd.epoch_base : 0u);
    for (int r = 0; r < rd.tp && ok; r++) ok = wait_flag_sys(rd.flags + r, e) ? 1u : 0u;
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && status) atomicExch(status, GEMM_ERR_TP_REDUCE_WAIT);
    return;
  }
  const size_t row = blockIdx.x;
  float v[8];
  int cnt = 0;
  float s = 0.f;
  for (int i = threadIdx.x; i < rd.hidden && cnt < 8; i += blockDim.x, cnt++) {
    float f = rd.bias ? rd.bias[i] : 0.f;
    for (int r = 0; r < rd.tp; r++) f += __bfloat162float(rd.slots[r][row * rd.hidden + i]);
    if (rd.residual) f += __bfloat162float(rd.residual[row * rd.hidden + i]);
    v[cnt] = f;
    s += f;
  }
  auto block_sum = [&](float x) {
#pragma unroll
    for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (l == 0) sh[w] = x;
    __syncthreads();
    float t = (l < nw) ? sh[l] : 0.f;
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
  };
  const float mean = block_sum(s) / rd.hidden;
  float q = 0.f;
  for (int k = 0; k < cnt; k++) q += (v[k] - mean) * (v[k] - mean);
  const float rstd = rsqrtf(block_sum(q) / rd.hidden + rd.eps);
  cnt = 0;
  for (int i = threadIdx.x; i < rd.hidden && cnt < 8; i += blockDim.x, cnt++)
    rd.out[row * rd.hidden + i] = __float2bfloat16((v[cnt] - mean) * rstd * rd.gamma[i] + rd.beta[i]);
  reduce_signal(rd);
}

// Last block out publishes the step number to the peers (see TpReduce::sig_*).
__device__ __forceinline__ void reduce_signal(const TpReduce& rd) {
  if (rd.sig_tp <= 0 || !rd.done_count) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t old = atomicAdd(rd.done_count, 1u);
    if (old == gridDim.x - 1) {
      *rd.done_count = 0;  // every block has counted: ready for the next launch (and for graph replay)
      const uint32_t e = rd.sig_epoch + (rd.epoch_base ? *rd.epoch_base : 0u);
      __threadfence_system();
      for (int p = 0; p < rd.sig_tp; p++) ptx::st_release_sys(rd.sig_peer_flag[p], e);
    }
  }
}

// Same computation with one warp per row and 16-byte accesses; hidden = VPL * 256.
template <int VPL>
__global__ void __launch_bounds__(256) layernorm_reduce_warp(TpReduce rd, int rows, uint32_t* status) {
  __shared__ uint32_t s_ok;
  if (threadIdx.x == 0) {
    uint32_t ok = 1;
    const uint32_t e = rd.epoch + (rd.epoch_base ? *rd.epoch_base : 0u);
    for (int r = 0; r < rd.tp && ok; r++) ok = wait_flag_sys(rd.flags + r, e) ? 1u : 0u;
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && status) atomicExch(status, GEMM_ERR_TP_REDUCE_WAIT);
    return;
  }
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  constexpr int H = VPL * 256;
  if (row < rows) {
    float v[VPL * 8];
#pragma unroll
    for (int c = 0; c < VPL; c++) {
      const int col = (c * 32 + lane) * 8;
      if (rd.bias) {
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(rd.bias + col));
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(rd.bias + col + 4));
        v[c * 8 + 0] = b0.x; v[c * 8 + 1] = b0.y; v[c * 8 + 2] = b0.z; v[c * 8 + 3] = b0.w;
        v[c * 8 + 4] = b1.x; v[c * 8 + 5] = b1.y; v[c * 8 + 6] = b1.z; v[c * 8 + 7] = b1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; j++) v[c * 8 + j] = 0.f;
      }
    }
    auto add_row = [&](const __nv_bfloat16* base) {
#pragma unroll
      for (int c = 0; c < VPL; c++) {
        // slots are written by peers through NVLink: read them past L1
        const uint4 q = __ldcg(reinterpret_cast<const uint4*>(base + (size_t)row * H + (c * 32 + lane) * 8));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int t = 0; t < 4; t++) {
          const float2 f = __bfloat1622float2(h[t]);
          v[c * 8 + 2 * t] += f.x;
          v[c * 8 + 2 * t + 1] += f.y;
        }
      }
    };
    for (int r = 0; r < rd.tp; r++) add_row(rd.slots[r]);
    if (rd.residual) add_row(rd.residual);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < VPL * 8; j++) s += v[j];
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s / H;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < VPL * 8; j++) q += (v[j] - mean) * (v[j] - mean);
#pragma unroll
    for (int o = 16; o; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rstd = rsqrtf(q / H + rd.eps);
#pragma unroll
    for (int c = 0; c < VPL; c++) {
      const int col = (c * 32 + lane) * 8;
      float g[8], b[8];
      *reinterpret_cast<float4*>(g) = __ldg(reinterpret_cast<const float4*>(rd.gamma + col));
      *reinterpret_cast<float4*>(g + 4) = __ldg(reinterpret_cast<const float4*>(rd.gamma + col + 4));
      *reinterpret_cast<float4*>(b) = __ldg(reinterpret_cast<const float4*>(rd.beta + col));
      *reinterpret_cast<float4*>(b + 4) = __ldg(reinterpret_cast<const float4*>(rd.beta + col + 4));
      uint4 o;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int t = 0; t < 4; t++)
        h[t] = __floats2bfloat162_rn((v[c * 8 + 2 * t] - mean) * rstd * g[2 * t] + b[2 * t],
                                     (v[c * 8 + 2 * t + 1] - mean) * rstd * g[2 * t + 1] + b[2 * t + 1]);
      *reinterpret_cast<uint4*>(rd.out + (size_t)row * H + col) = o;
    }
  }
  reduce_signal(rd);
}

int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

cudaError_t srpc_gemm_tp(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                         const TpParams& tp_in, uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N < 0 || K <= 0 || (M % BM) != 0) return cudaErrorInvalidValue;
  if ((lda % 8) || (ldb % 8) || (K % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || (ep.ldo % 8)) return cudaErrorInvalidValue;
  TpParams tp = tp_in;
  if (tp.tp < 1 || tp.tp > TP_MAX_RANKS || (M / BM) % tp.tp != 0) return cudaErrorInvalidValue;
  if (srpc_gemm_tp_2sm_eligible(M, N, K, ep, tp)) return srpc_gemm_tp_2sm(A, lda, B, ldb, M, N, K, ep, tp, status, stream);
  tp.mblocks_per_rank = (M / BM) / tp.tp;
  tp.m_rot = tp.rank * tp.mblocks_per_rank;
  tp.mblock_bytes = (size_t)BM * lda * 2;
  const int tiles_n = (N + BN - 1) / BN;
  tp.tiles_per_owner = tp.mblocks_per_rank * tiles_n;
  if (!tp.mblock_ready) tp.n_copy = 0;
  tp.n_copy = std::min(tp.n_copy, std::max(1, (tp.tp - 1) * tp.mblocks_per_rank));  // a copier takes whole row blocks
  static PerDeviceFlag attr;
  const int dev = PerDeviceFlag::current();
  const int smem = STAGES * STAGE_BYTES + 2 * OUT_BYTES + 1024;
  if (attr.needed(dev)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr.set(dev);
  }
  CUtensorMap ta, tb, to;
  cudaError_t e = map_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM);
  if (e != cudaSuccess) return e;
  if (N > 0) {
    e = map_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN);
    if (e != cudaSuccess) return e;
  } else {
    tb = ta;
  }
  if (!tp.rs && N > 0) {
    e = map_2d(&to, ep.out, (uint64_t)N, (uint64_t)M, (uint64_t)ep.ldo * 2, 64, BM);
    if (e != cudaSuccess) return e;
  } else {
    to = ta;
  }
  const int tiles = (M / BM) * tiles_n;
  int gemm_ctas = std::min(std::max(tiles, 1), num_sms() - tp.n_copy);
  if (gemm_ctas < 1) return cudaErrorInvalidValue;
  gemm_tp_kernel<<<gemm_ctas + tp.n_copy, THREADS, smem, stream>>>(ta, tb, to, M, N, K, ep, tp, status);
  return cudaGetLastError();
}

// One block per (rank, 16 KB piece) of the batch; the last block to finish publishes control records and doorbells.
__global__ void __launch_bounds__(256) tp_fanout_kernel(const TpFanout f) {
  const uint8_t* src = *reinterpret_cast<const uint8_t* const*>(f.stub);  // g_params::req is the stub's first word
  const size_t total = (size_t)f.max_batch * f.req_bytes, live = (size_t)f.batch * f.req_bytes;
  const size_t piece = 16384;
  const size_t pieces = (total + piece - 1) / piece;
  for (size_t w = blockIdx.x; w < pieces * (size_t)f.tp; w += gridDim.x) {
    const int r = (int)(w / pieces);
    const size_t at = (w % pieces) * piece, end = at + piece < total ? at + piece : total;
    for (size_t o = at + (size_t)threadIdx.x * 16; o < end; o += (size_t)blockDim.x * 16) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (o < live) v = *reinterpret_cast<const uint4*>(src + o);
      *reinterpret_cast<uint4*>(f.dst[r] + o) = v;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // cumulative: covers the block's stores (ordered before the barrier)
    if (atomicAdd(f.arrivals, 1u) == gridDim.x - 1) {
      *f.arrivals = 0;
      const uint32_t s = *f.seq + 1u;
      *f.seq = s;
      for (int r = 0; r < f.tp; r++) {
        f.ctrl[r][0] = f.command;
        f.ctrl[r][1] = f.batch;
      }
      __threadfence_system();
      for (int r = 0; r < f.tp; r++) ptx::st_release_sys(f.doorbell[r], s);
    }
  }
}

cudaError_t srpc_tp_fanout(const TpFanout& f, cudaStream_t stream) {
  if (f.tp < 1 || f.tp > TP_MAX_RANKS || !f.stub || (f.req_bytes & 15u) || f.batch > f.max_batch || !f.seq || !f.arrivals)
    return cudaErrorInvalidValue;
  const size_t pieces = ((size_t)f.max_batch * f.req_bytes + 16383) / 16384;
  const int blocks = (int)std::min<size_t>(pieces * (size_t)f.tp, 64);
  tp_fanout_kernel<<<blocks > 0 ? blocks : 1, 256, 0, stream>>>(f);
  return cudaGetLastError();
}

cudaError_t srpc_tp_signal(const TpSignal& sig, cudaStream_t stream) {
  tp_signal_peers<<<1, 32, 0, stream>>>(sig);
  return cudaGetLastError();
}

__global__ void tp_wait_kernel(const uint32_t* flags, int n, uint32_t epoch, const uint32_t* epoch_base, uint32_t* status) {
  const int i = threadIdx.x;
  if (i < n) {
    const uint32_t e = epoch + (epoch_base ? *epoch_base : 0u);
    if (!wait_flag_sys(flags + i, e) && status) atomicExch(status, GEMM_ERR_TP_SRC_WAIT);
  }
}

// Sets the bound of the flag waits of every kernel in this file on the current device.
cudaError_t srpc_tp_set_wait_ns(uint64_t ns) {
  cudaError_t e = tpdev::set_wait_ns_here(ns);
  return e != cudaSuccess ? e : srpc_gemm_tp_2sm_set_wait_ns(ns);
}

cudaError_t srpc_tp_wait(const uint32_t* flags, int n, uint32_t epoch, const uint32_t* epoch_base, uint32_t* status,
                         cudaStream_t stream) {
  tp_wait_kernel<<<1, 32, 0, stream>>>(flags, n, epoch, epoch_base, status);
  return cudaGetLastError();
}

// Start of a pass in one launch: wait until flags[0..n) have reached the current base, then advance the base.
__global__ void tp_begin_kernel(const uint32_t* flags, int n, uint32_t* epoch_base, uint32_t delta, uint32_t* status) {
  const int i = threadIdx.x;
  if (i < n && !wait_flag_sys(flags + i, *epoch_base) && status) atomicExch(status, GEMM_ERR_TP_SRC_WAIT);
  __syncwarp();
  if (i == 0) *epoch_base += delta;
}

cudaError_t srpc_tp_begin(const uint32_t* flags, int n, uint32_t* epoch_base, uint32_t delta, uint32_t* status,
                          cudaStream_t stream) {
  if (n < 1 || n > 32 || !epoch_base) return cudaErrorInvalidValue;
  tp_begin_kernel<<<1, 32, 0, stream>>>(flags, n, epoch_base, delta, status);
  return cudaGetLastError();
}

__global__ void tp_bump_kernel(uint32_t* word, uint32_t delta) { *word += delta; }

cudaError_t srpc_tp_bump(uint32_t* word, uint32_t delta, cudaStream_t stream) {
  tp_bump_kernel<<<1, 1, 0, stream>>>(word, delta);
  return cudaGetLastError();
}

cudaError_t srpc_layernorm_reduce(const TpReduce& rd, int rows, uint32_t* status, cudaStream_t stream) {
  if (rd.hidden > 2048 || rd.tp < 1 || rd.tp > TP_MAX_RANKS) return cudaErrorInvalidValue;
  bool aligned = (((uintptr_t)rd.out | (uintptr_t)rd.residual | (uintptr_t)rd.bias | (uintptr_t)rd.gamma | (uintptr_t)rd.beta) & 15) == 0;
  for (int r = 0; r < rd.tp; r++) aligned = aligned && (((uintptr_t)rd.slots[r]) & 15) == 0;
  const int blocks = (rows + 7) / 8;
  if (aligned && rd.hidden == 1024) layernorm_reduce_warp<4><<<blocks, 256, 0, stream>>>(rd, rows, status);
  else if (aligned && rd.hidden == 768) layernorm_reduce_warp<3><<<blocks, 256, 0, stream>>>(rd, rows, status);
  else if (aligned && rd.hidden == 512) layernorm_reduce_warp<2><<<blocks, 256, 0, stream>>>(rd, rows, status);
  else if (aligned && rd.hidden == 256) layernorm_reduce_warp<1><<<blocks, 256, 0, stream>>>(rd, rows, status);
  else layernorm_reduce<<<rows, 256, 0, stream>>>(rd, status);
  return cudaGetLastError();
}
