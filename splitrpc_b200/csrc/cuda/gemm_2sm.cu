// Two-SM persistent GEMM:  D[M,N] = act(A[M,K] . B[N,K]^T + bias + residual), bf16 in and out, fp32 accumulation.
//
// The compute-bound shapes of the one-SM kernel (gemm_persistent.cu) stall on operand delivery: a 128 x 256 tile
// pulls 48 KB through the L2 -> SM path per 64-deep k-block, and at full tensor rate that is more than the path
// carries, so the tensor pipe idles a third of the time.  Here two CTAs of a cluster (an SM pair) compute one
// 256 x 256 tile with tcgen05.mma.cta_group::2: each CTA loads its own 128 rows of A and only HALF of the B rows
// (32 KB per k-block), the leader CTA's single MMA thread issues one instruction that reads both CTAs' shared memory
// and writes 128 accumulator rows into each CTA's tensor memory.
//
// Protocol (both CTAs run the same code; rank 0 of the pair is the leader):
//   producer   thread 0 of each CTA loads its A rows and its half of B for every k-block through a 5-stage ring.  The
//              "full" barrier of a stage is the LEADER's: the leader's producer posts the expected byte count of both
//              CTAs, and both CTAs' TMA loads (cp.async.bulk.tensor ... cta_group::2, no multicast) count on it.
//   MMA        one thread of the leader waits for a full stage, issues four 256 x 256 x 16 MMAs and commits them to
//              the stage's "empty" barrier in BOTH CTAs (tcgen05.commit with a two-CTA mask), then, per tile, to both
//              CTAs' "accumulator full" barriers.  Two accumulators (2 x 256 columns) alternate between tiles.
//   epilogue   16 warps per CTA read their CTA's 128 accumulator rows (tcgen05.ld), add bias (staged in shared memory)
//              and residual, apply the activation, stage the bf16 tile in swizzled shared memory and hand it to TMA
//              stores; each warp releases the accumulator by arriving on the LEADER's "accumulator empty" barrier.
// Every mbarrier wait is bounded; on a timeout the CTA records an error code and winds down; both CTAs always reach
// the two cluster barriers (after set-up and before tensor memory is freed).  All operands live in this GPU's memory.
//
// Tensor-parallel variant (template flag TP, entry point srpc_gemm_tp_2sm): the same pair tiles with
//   all-gather   copier clusters appended to the grid pull the peers' row shards of A over NVLink into this GPU's
//                gathered buffer (bulk copies through shared memory, no multicast) and publish each 128-row block; the
//                producer of a CTA waits (bounded) for the block its tile needs.  Tiles are ordered so that the rows
//                this rank already holds come first.
//   reduce-scatter  the epilogue stores the staged bf16 tile with 16-byte stores into the slot this rank owns in the
//                memory of the rank that owns the rows (its own slot for its own rows), fences, counts the tile and,
//                when the last tile for an owner is through, publishes the step number there.  Rows owned by peers
//                come first, so that their transfer overlaps the rest of the GEMM.
#include <algorithm>
#include <cstdlib>

#include "gemm_tcgen05.h"
#include "per_device.h"
#include "ptx.cuh"
#include "tp_device.cuh"

cudaError_t srpc_tensor_map_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                               uint32_t box_inner, uint32_t box_outer);

namespace {

constexpr int BM = 128;   // rows per CTA; a pair computes 256
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int OUT_HALF_BYTES = BM * 128;    // 128 rows x 64 bf16 columns

// Tile widths 128 / 192 / 256: one epilogue warp per 64 columns and TMEM lane quarter, as many stages as fit.
template <int BN>
struct Cfg {
  static constexpr int B_BYTES = (BN / 2) * BK * 2;  // this CTA's half of the B rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // The 256-wide tile writes its output in two passes of 128 columns through a 32 KB staging buffer: the memory goes
  // to a sixth operand stage, and the k loop runs at (round-trip latency) / (stages).
  static constexpr int PASSES = BN == 256 ? 2 : 1;
  static constexpr int PASS_COLS = BN / PASSES;
  static constexpr int STAGES = BN == 256 ? 6 : (BN == 192 ? 6 : 7);
  static constexpr int OUT_BYTES = (PASS_COLS / 64) * OUT_HALF_BYTES;
  static constexpr int EPI_THREADS = 2 * BN;
  static constexpr int THREADS = 64 + EPI_THREADS;
  static constexpr int ACC_STRIDE = BN == 192 ? 256 : BN;  // TMEM columns between the two accumulators
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BYTES;
};

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

// Optional phase time stamps of block 0 (build with -DSRPC_GEMM_TRACE), read back through srpc_gemm_trace_read.
#ifdef SRPC_GEMM_TRACE
__device__ unsigned long long g_gemm2_trace[16];
#define GEMM2_TRACE(slot)                                             \
  do {                                                                \
    if (blockIdx.x == 0) g_gemm2_trace[slot] = ptx::globaltimer_ns(); \
  } while (0)
#else
#define GEMM2_TRACE(slot) ((void)0)
#endif

struct PairTile {
  int m2, n;  // 256-row block, 256-column block
};

struct TileOrder {
  int clusters;  // clusters that compute tiles (the grid may hold copier clusters after them)
  int tiles_m2, tiles_n;
  int group_m;   // 256-row blocks per group
  int m_rot2;    // rotation of the 256-row blocks (tensor-parallel: which rank's rows come first)
};

// j-th tile of this cluster, grouped so that tiles in flight share A and B blocks in L2.
__device__ __forceinline__ bool pair_tile(int j, const TileOrder& o, PairTile* out) {
  const int tile = (int)(blockIdx.x >> 1) + j * o.clusters;
  if (tile >= o.tiles_m2 * o.tiles_n) return false;
  const int per_group = o.group_m * o.tiles_n;
  const int g = tile / per_group, in_g = tile - g * per_group;
  const int m_first = g * o.group_m;
  const int gm = (o.tiles_m2 - m_first) < o.group_m ? (o.tiles_m2 - m_first) : o.group_m;
  int m2 = m_first + in_g % gm + o.m_rot2;
  if (m2 >= o.tiles_m2) m2 -= o.tiles_m2;
  out->m2 = m2;
  out->n = in_g / gm;
  return true;
}

template <int BN, bool TP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg<BN>::THREADS, 1)
gemm_2sm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_out, int M, int N, int K, const TileOrder order, GemmEpilogue ep,
                uint32_t* status, const TpParams tp_in) {
  constexpr int B_BYTES = Cfg<BN>::B_BYTES, STAGE_BYTES = Cfg<BN>::STAGE_BYTES, STAGES = Cfg<BN>::STAGES;
  constexpr int EPI_THREADS = Cfg<BN>::EPI_THREADS, ACC_STRIDE = Cfg<BN>::ACC_STRIDE, TMEM_COLS = Cfg<BN>::TMEM_COLS;
  constexpr int PASSES = Cfg<BN>::PASSES, PASS_COLS = Cfg<BN>::PASS_COLS;
  constexpr int CH = PASS_COLS / 32 / (EPI_THREADS / 128);  // 32-column chunks per warp and pass
  (void)B_BYTES;
  extern __shared__ __align__(1024) uint8_t smem[];
  TpParams tp = tp_in;
  if constexpr (TP) {
    if (tp.epoch_base) tp.epoch += *tp.epoch_base;
    if ((int)(blockIdx.x >> 1) >= order.clusters) {
      // Copier CTA: neither of the pair takes part in the cluster barriers below, nor holds tensor memory.
      tpdev::copier(tp, (int)blockIdx.x - 2 * order.clusters, smem, status);
      return;
    }
  }
  uint8_t* stage_out = smem + (size_t)STAGES * STAGE_BYTES;
  __shared__ __align__(8) uint64_t full_bar[STAGES];   // used in the leader only
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];  // used in the leader only: arrivals from both CTAs' epilogue warps
  __shared__ uint32_t tmem_base_smem;
  __shared__ uint32_t s_error;
  // One buffer is enough: the last named barrier of a tile (before its store) comes after every read of that tile's
  // bias, and a thread writes the next tile's bias only after passing it.
  __shared__ __align__(16) float s_bias[BN];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = rank == 0;
  const int num_kb = (K + BK - 1) / BK;
  // The swizzled tiles and their descriptors need a 1024-byte aligned base; the layout is the same in both CTAs, so
  // both take the same decision.
  const bool layout_ok = (ptx::smem_u32(smem) & 1023u) == 0;

  if (threadIdx.x == 0) {
    GEMM2_TRACE(0);
    for (int s = 0; s < STAGES; s++) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; a++) {
      ptx::mbar_init(&tmem_full_bar[a], 1);
      ptx::mbar_init(&tmem_empty_bar[a], 2 * (EPI_THREADS / 32));
    }
    ptx::fence_mbar_init();
    s_error = layout_ok ? 0u : (uint32_t)GEMM_ERR_PRODUCER_WAIT;
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    ptx::prefetch_tmap(&tmap_out);
  }
  if (warp == 1) {
    ptx::tmem_alloc_2sm(&tmem_base_smem, TMEM_COLS);
    ptx::tmem_relinquish_2sm();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();  // the peer's barriers exist before anything signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  if (threadIdx.x == 0) GEMM2_TRACE(1);

  if (threadIdx.x == 0) {
    // ---------------- producer (one per CTA)
    int s = 0;
    uint32_t ph = 0;
    PairTile t;
    for (int j = 0; layout_ok && pair_tile(j, order, &t) && *(volatile uint32_t*)&s_error == 0; j++) {
      const int row0 = (t.m2 * 2 + (int)rank) * BM;
      const int brow0 = t.n * BN + (int)rank * (BN / 2);
      if constexpr (TP) {
        if (tp.mblock_ready) {
          // Rows of a peer arrive through the copier clusters of this launch, one 128-row block at a time.
          const int m_idx = t.m2 * 2 + (int)rank;
          if (m_idx / tp.mblocks_per_rank != tp.rank) {
            if (!tpdev::wait_flag_gpu(tp.mblock_ready + m_idx, tp.epoch)) {
              atomicExch(&s_error, GEMM_ERR_TP_BLOCK_WAIT);
              break;
            }
            ptx::fence_proxy_async_all();  // the copier's writes -> this thread's TMA reads
          }
        }
      }
      for (int kb = 0; kb < num_kb; kb++) {
        if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u)) {
          atomicExch(&s_error, GEMM_ERR_PRODUCER_WAIT);
          break;
        }
        const uint32_t full_leader = ptx::mapa_shared(ptx::smem_u32(&full_bar[s]), 0);
        if (leader) ptx::mbar_expect_tx(&full_bar[s], 2u * STAGE_BYTES);
        uint8_t* sa = smem + (size_t)s * STAGE_BYTES;
        ptx::tma_load_2d_2sm(sa, &tmap_a, full_leader, kb * BK, row0);
        ptx::tma_load_2d_2sm(sa + A_BYTES, &tmap_b, full_leader, kb * BK, brow0);
        if (j == 0 && kb == 0) GEMM2_TRACE(2);
        if (++s == STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (threadIdx.x == 32) {
    // ---------------- MMA issue (leader only)
    if (leader) {
      const uint32_t idesc = ptx::umma_idesc_bf16(2 * BM, BN);
      int s = 0;
      uint32_t ph = 0, local = 0;
      PairTile t;
      for (int j = 0; layout_ok && pair_tile(j, order, &t) && *(volatile uint32_t*)&s_error == 0; j++, local++) {
        const uint32_t acc = local & 1u;
        if (!ptx::mbar_wait(&tmem_empty_bar[acc], ((local >> 1) & 1u) ^ 1u)) {
          atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        bool ok = true;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!ptx::mbar_wait(&full_bar[s], ph)) {
            atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          if (j == 0 && kb == 0) GEMM2_TRACE(3);
          if (j == 0 && kb == 8) GEMM2_TRACE(10);
          if (j == 0 && kb == 24) GEMM2_TRACE(11);
          const uint32_t sa = ptx::smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++)
            ptx::umma_bf16_2sm(d_tmem, ptx::umma_desc_sw128(sa + k * UMMA_K * 2), ptx::umma_desc_sw128(sb + k * UMMA_K * 2), idesc,
                               (kb | k) != 0 ? 1u : 0u);
          ptx::umma_commit_2sm(&empty_bar[s], 3);  // frees the stage in both CTAs
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit_2sm(&tmem_full_bar[acc], 3);
        if (j == 0) GEMM2_TRACE(4);
      }
    }
  } else if (warp >= 2) {
    // ---------------- epilogue: the warps of a TMEM lane quarter (w, w+4, ...) split the columns of a pass
    const int warp_q = warp & 3;
    const int cgroup = (warp - 2) >> 2;      // 0 .. EPI_THREADS/128 - 1
    const int row = warp_q * 32 + lane;      // row of this CTA's half tile
    const int et = threadIdx.x - 64;
    const bool vec_res = ep.residual && ((ep.ldr & 7) == 0) && (((uintptr_t)ep.residual & 15) == 0);
    uint32_t local = 0;
    PairTile t;
    bool peer_store = false;
    if constexpr (TP) peer_store = tp.rs != 0;
    for (int j = 0; layout_ok && pair_tile(j, order, &t); j++, local++) {
      const uint32_t acc = local & 1u;
      const int row0 = (t.m2 * 2 + (int)rank) * BM;
      const int m = row0 + row;
      const bool row_ok = m < M;
      const int n0 = t.n * BN;
      float* bias_s = s_bias;
      if (ep.bias && et < BN) bias_s[et] = (n0 + et < N) ? __ldg(ep.bias + n0 + et) : 0.f;
      const bool mine = (*(volatile uint32_t*)&s_error == 0) && ptx::mbar_wait(&tmem_full_bar[acc], (local >> 1) & 1u);
      if (!named_bar_all(2, EPI_THREADS, mine)) {  // uniform outcome; also orders the bias writes before their reads
        if (lane == 0) atomicExch(&s_error, GEMM_ERR_EPILOGUE_WAIT);
        break;
      }
      ptx::tc_fence_after();
      if (j == 0 && et == 0) GEMM2_TRACE(5);
#pragma unroll
      for (int pass = 0; pass < PASSES; pass++) {
        // The previous store must have finished reading the staging buffer.
        if (et == 0 && !peer_store) ptx::bulk_wait_read<0>();
        named_bar_sync(1, EPI_THREADS);
#pragma unroll
        for (int ch = 0; ch < CH; ch++) {
          const int cp = (cgroup * CH + ch) * 32;   // column inside the pass
          const int c = pass * PASS_COLS + cp;      // column inside the tile
          const int col0 = n0 + c;
          uint32_t r[32];
          ptx::tmem_ld_32x32b_x32(tmem_base + acc * ACC_STRIDE + ((uint32_t)(warp_q * 32) << 16) + (uint32_t)c, r);
          ptx::tmem_ld_wait();
          if (pass == PASSES - 1 && ch == CH - 1) {  // last read: hand the accumulator back to the leader's MMA thread
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(ptx::smem_u32(&tmem_empty_bar[acc]), 0));
          }
          float v[32];
#pragma unroll
          for (int q = 0; q < 32; q++) v[q] = __uint_as_float(r[q]);
          if (ep.bias) {
#pragma unroll
            for (int q = 0; q < 32; q += 4) {
              const float4 b4 = *reinterpret_cast<const float4*>(bias_s + c + q);
              v[q] += b4.x;
              v[q + 1] += b4.y;
              v[q + 2] += b4.z;
              v[q + 3] += b4.w;
            }
          }
          if (ep.residual && row_ok && col0 < N) {
            const __nv_bfloat16* rp = ep.residual + (size_t)m * ep.ldr + col0;
            if (vec_res && col0 + 32 <= N) {
#pragma unroll
              for (int q = 0; q < 4; q++) {
                const uint4 rq = __ldg(reinterpret_cast<const uint4*>(rp) + q);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rq);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                  const float2 f = __bfloat1622float2(h[u]);
                  v[q * 8 + 2 * u] += f.x;
                  v[q * 8 + 2 * u + 1] += f.y;
                }
              }
            } else {
#pragma unroll
              for (int q = 0; q < 32; q++)
                if (col0 + q < N) v[q] += __bfloat162float(rp[q]);
            }
          }
          if (ep.act == GEMM_ACT_RELU) {
#pragma unroll
            for (int q = 0; q < 32; q++) v[q] = fmaxf(v[q], 0.f);
          } else if (ep.act == GEMM_ACT_GELU) {
#pragma unroll
            for (int q = 0; q < 32; q++) v[q] = ptx::gelu_erf_fast(v[q]);
          } else if (ep.act == GEMM_ACT_TANH) {
#pragma unroll
            for (int q = 0; q < 32; q++) v[q] = tanhf(v[q]);
          }
          uint8_t* half = stage_out + (size_t)(cp >> 6) * OUT_HALF_BYTES + (size_t)row * 128;
          const int chunk0 = (cp & 63) >> 3;
#pragma unroll
          for (int q = 0; q < 4; q++) {
            uint4 o;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int u = 0; u < 4; u++) h[u] = __floats2bfloat162_rn(v[q * 8 + 2 * u], v[q * 8 + 2 * u + 1]);
            *reinterpret_cast<uint4*>(half + (((chunk0 + q) ^ (row & 7)) << 4)) = o;
          }
        }
        if constexpr (TP) {
          if (peer_store) {
            // The tile goes to the slot this rank owns on the rank that owns these rows (rows per rank are a multiple
            // of 128, so a CTA's half tile has one owner).
            named_bar_sync(1, EPI_THREADS);
            const int m_idx = t.m2 * 2 + (int)rank;
            const int owner = m_idx / tp.mblocks_per_rank;
            const int local_m0 = (m_idx - owner * tp.mblocks_per_rank) * BM;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(tp.dst[owner]);
            constexpr int SEGS = PASS_COLS / 8;  // 16-byte segments per row of this pass
#pragma unroll 4
            for (int q = et; q < BM * SEGS; q += EPI_THREADS) {
              const int rr = q / SEGS, seg = q - rr * SEGS;
              const int col = n0 + pass * PASS_COLS + seg * 8;
              if (col < N) {
                const uint8_t* src = stage_out + (size_t)(seg >> 3) * OUT_HALF_BYTES + (size_t)rr * 128 + (((seg & 7) ^ (rr & 7)) << 4);
                *reinterpret_cast<uint4*>(dst + (size_t)(local_m0 + rr) * ep.ldo + col) = *reinterpret_cast<const uint4*>(src);
              }
            }
            if (pass == PASSES - 1) {
              // Every thread's stores of every pass are ordered before the barrier; the one system-scope fence behind
              // it (fences are cumulative) then makes the whole half tile visible on the owner before the count, and
              // through the count before the flag.  A fence per thread costs hundreds of them per tile.
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
            continue;
          }
        }
        ptx::fence_proxy_async_smem();
        named_bar_sync(1, EPI_THREADS);
        if (et == 0) {
#pragma unroll
          for (int hcol = 0; hcol < PASS_COLS / 64; hcol++) {
            const int col = n0 + pass * PASS_COLS + hcol * 64;
            if (col >= N || row0 >= M) break;
            ptx::tma_store_2d(&tmap_out, stage_out + (size_t)hcol * OUT_HALF_BYTES, col, row0);
          }
          ptx::bulk_commit();
          if (j == 0 && pass == PASSES - 1) GEMM2_TRACE(6);
        }
      }
    }
    if (et == 0) {
      GEMM2_TRACE(7);
      ptx::bulk_wait_read<0>();
      GEMM2_TRACE(8);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (s_error != 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, s_error);
    __nanosleep(1000000);  // let loads that are still in flight land before the block leaves
  }
  ptx::cluster_sync_all();  // the peer no longer reads this CTA's shared memory nor signals its barriers
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_2sm(tmem_base, TMEM_COLS);
  }
}


// Clusters of two CTAs that can be resident at once (queried once per instantiation and device).
template <int BN, bool TP>
cudaError_t max_clusters_2sm(int* out) {
  using C = Cfg<BN>;
  static std::atomic<int> per_device[64];
  const int dev = PerDeviceFlag::current();
  int max_clusters = per_device[dev].load(std::memory_order_acquire);
  if (!max_clusters) {
    cudaError_t e = cudaFuncSetAttribute(gemm_2sm_kernel<BN, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_2sm_kernel<BN, TP>, &cfg);
    if (e != cudaSuccess) return e;
    if (n < 1) return cudaErrorInvalidConfiguration;
    max_clusters = n;
    per_device[dev].store(n, std::memory_order_release);
  }
  *out = max_clusters;
  return cudaSuccess;
}

template <int BN>
cudaError_t launch_2sm(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                       uint32_t* status, cudaStream_t stream) {
  using C = Cfg<BN>;
  int max_clusters = 0;
  cudaError_t e = max_clusters_2sm<BN, false>(&max_clusters);
  if (e != cudaSuccess) return e;
  CUtensorMap ta, tb, to;
  e = srpc_tensor_map_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM);
  if (e != cudaSuccess) return e;
  e = srpc_tensor_map_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN / 2);
  if (e != cudaSuccess) return e;
  e = srpc_tensor_map_2d(&to, ep.out, (uint64_t)N, (uint64_t)M, (uint64_t)ep.ldo * 2, 64, BM);
  if (e != cudaSuccess) return e;
  TileOrder o;
  o.tiles_m2 = (M + 2 * BM - 1) / (2 * BM);
  o.tiles_n = (N + BN - 1) / BN;
  o.clusters = std::min(o.tiles_m2 * o.tiles_n, std::min(max_clusters, srpc_gemm_grid_sms() / 2));
  o.group_m = 4;
  o.m_rot2 = 0;
  gemm_2sm_kernel<BN, false><<<2 * o.clusters, C::THREADS, C::SMEM_BYTES, stream>>>(ta, tb, to, M, N, K, o, ep, status, TpParams{});
  return cudaGetLastError();
}

// Tensor-parallel launch: `tp` arrives with mblocks_per_rank / mblock_bytes filled in and an even n_copy.
template <int BN>
cudaError_t launch_2sm_tp(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                          TpParams tp, uint32_t* status, cudaStream_t stream) {
  using C = Cfg<BN>;
  static_assert(C::SMEM_BYTES >= tpdev::COPY_SLOTS * tpdev::COPY_CHUNK, "the copier's ring lives in the operand stages");
  int max_clusters = 0;
  cudaError_t e = max_clusters_2sm<BN, true>(&max_clusters);
  if (e != cudaSuccess) return e;
  max_clusters = std::min(max_clusters, srpc_gemm_grid_sms() / 2);
  const int copy_clusters = tp.n_copy / 2;
  if (max_clusters - copy_clusters < 1) return cudaErrorInvalidValue;
  CUtensorMap ta, tb, to;
  e = srpc_tensor_map_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM);
  if (e != cudaSuccess) return e;
  e = srpc_tensor_map_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN / 2);
  if (e != cudaSuccess) return e;
  if (!tp.rs) {
    e = srpc_tensor_map_2d(&to, ep.out, (uint64_t)N, (uint64_t)M, (uint64_t)ep.ldo * 2, 64, BM);
    if (e != cudaSuccess) return e;
  } else {
    to = ta;  // never used: the epilogue stores to the owners' slots
  }
  TileOrder o;
  o.tiles_m2 = M / (2 * BM);
  o.tiles_n = (N + BN - 1) / BN;
  o.clusters = std::min(o.tiles_m2 * o.tiles_n, max_clusters - copy_clusters);
  const int m2_per_rank = tp.mblocks_per_rank / 2;
  o.group_m = 1;
  for (int g = 2; g <= 4; g++)
    if (m2_per_rank % g == 0) o.group_m = g;  // groups never straddle two ranks' rows
  // all-gather: own rows first (they are here already); reduce-scatter: own rows last (the peers' cross NVLink)
  o.m_rot2 = (tp.rs ? (tp.rank + 1) % tp.tp : tp.rank) * m2_per_rank;
  tp.tiles_per_owner = tp.mblocks_per_rank * o.tiles_n;
  gemm_2sm_kernel<BN, true><<<2 * (o.clusters + copy_clusters), C::THREADS, C::SMEM_BYTES, stream>>>(ta, tb, to, M, N, K, o, ep, status, tp);
  return cudaGetLastError();
}

}  // namespace

int srpc_gemm2_trace_read(unsigned long long* out, int n) {
#ifdef SRPC_GEMM_TRACE
  if (n > 16) n = 16;
  if (cudaMemcpyFromSymbol(out, g_gemm2_trace, n * sizeof(unsigned long long)) != cudaSuccess) return 0;
  return n;
#else
  (void)out;
  (void)n;
  return 0;
#endif
}

bool srpc_gemm_2sm_eligible(int M, int N, int K, const GemmEpilogue& ep) {
  static const int allow = [] { const char* e = getenv("SPLITRPC_GEMM_2SM"); return e ? atoi(e) : 1; }();
  if (!allow || ep.out_fp32 || (ep.ldo % 8) || ((uintptr_t)ep.out & 15)) return false;
  if (ep.bias && ((uintptr_t)ep.bias & 15)) return false;
  return M >= 256 && N >= 128 && K >= 64;
}

cudaError_t srpc_gemm_bf16_2sm(const void* A, int lda, const void* B, int ldb, int M, int N, int K, int bn, const GemmEpilogue& ep,
                               uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  if ((lda % 8) || (ldb % 8) || (K % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return cudaErrorInvalidValue;
  if (!srpc_gemm_2sm_eligible(M, N, K, ep)) return cudaErrorInvalidValue;
  if (bn == 256) return launch_2sm<256>(A, lda, B, ldb, M, N, K, ep, status, stream);
  if (bn == 192) return launch_2sm<192>(A, lda, B, ldb, M, N, K, ep, status, stream);
  if (bn == 128) return launch_2sm<128>(A, lda, B, ldb, M, N, K, ep, status, stream);
  return cudaErrorInvalidValue;
}

// Tensor-parallel entry point (see gemm_tp.h).  Takes the shapes where a rank's rows are whole 256-row pair tiles.
bool srpc_gemm_tp_2sm_eligible(int M, int N, int K, const GemmEpilogue& ep, const TpParams& tp) {
  static const int allow = [] { const char* e = getenv("SPLITRPC_TP_2SM"); return e ? atoi(e) : 1; }();
  if (!allow || tp.tp < 1 || N < 128 || (N % 8) || K < 64 || ep.out_fp32 || (ep.ldo % 8)) return false;
  if (ep.bias && ((uintptr_t)ep.bias & 15)) return false;
  if (!tp.rs && ((uintptr_t)ep.out & 15)) return false;
  return M % (2 * BM * tp.tp) == 0;
}

cudaError_t srpc_gemm_tp_2sm(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                             const TpParams& tp_in, uint32_t* status, cudaStream_t stream) {
  if (!srpc_gemm_tp_2sm_eligible(M, N, K, ep, tp_in)) return cudaErrorInvalidValue;
  TpParams tp = tp_in;
  tp.mblocks_per_rank = (M / BM) / tp.tp;
  tp.m_rot = 0;
  tp.mblock_bytes = (size_t)BM * lda * 2;
  // a copier takes whole 128-row blocks: more copiers than remote blocks would idle on SMs the GEMM could use
  tp.n_copy = tp.mblock_ready ? (std::min(tp.n_copy, (tp.tp - 1) * tp.mblocks_per_rank) + 1) & ~1 : 0;
  if (tp.rs)
    for (int o = 0; o < tp.tp; o++)
      if ((uintptr_t)tp.dst[o] & 15) return cudaErrorInvalidValue;
  const int bn = (N % 256 == 0) ? 256 : ((N % 192 == 0) ? 192 : (N % 128 == 0 ? 128 : (N >= 1024 ? 256 : 128)));
  if (bn == 256) return launch_2sm_tp<256>(A, lda, B, ldb, M, N, K, ep, tp, status, stream);
  if (bn == 192) return launch_2sm_tp<192>(A, lda, B, ldb, M, N, K, ep, tp, status, stream);
  return launch_2sm_tp<128>(A, lda, B, ldb, M, N, K, ep, tp, status, stream);
}

cudaError_t srpc_gemm_tp_2sm_set_wait_ns(uint64_t ns) { return tpdev::set_wait_ns_here(ns); }
