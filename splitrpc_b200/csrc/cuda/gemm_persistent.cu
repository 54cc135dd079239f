// Persistent tcgen05 GEMM / convolution kernel (the production path).
//
//   D[M,N] = act(A[M,K] . B[N,K]^T + bias + residual)          (GEMM mode)
//   out = act(conv(in NHWC, filter [Cout][R][S][Cin]) + bias + residual)   (convolution mode)
//
// One CTA per SM loops over output tiles (128 x BN).  Warp roles:
//   warp 0   one elected thread issues TMA loads for every k-block of every tile
//            of this CTA, running ahead through a STAGES-deep shared-memory ring
//            that is not drained at tile boundaries;
//   warp 1   one elected thread issues tcgen05.mma into one of two TMEM
//            accumulators (2 x BN columns), so tile i+1 accumulates while tile i
//            is being written out;
//   warps 2-9 read the accumulator with tcgen05.ld (two warps per TMEM lane
//            quarter, half of the columns each), release it at once, apply bias /
//            residual (prefetched before the accumulator is ready) / activation,
//            stage the bf16 tile in one of two 128-byte-swizzled shared-memory
//            buffers and hand it to a TMA store (full-line coalesced writes,
//            bounds clipped by the tensor map).
// In convolution mode the A operand needs no im2col and no gather: a tile is a
// PW x PH x PN patch of output pixels, and the rows for filter tap (fr, fs) are
// one 4-D TMA box over the NHWC input shifted by the tap offset, with element
// strides equal to the convolution stride; out-of-image coordinates are
// zero-filled by the TMA unit, which is exactly the padding.
// All operands live in this GPU's memory; no load uses multicast.  Every wait
// is bounded; on a timeout the kernel records an error code, stops issuing work,
// frees its tensor memory and returns.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "gemm_tcgen05.h"
#include "ptx.cuh"
#include "per_device.h"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
// Epilogue threads of the 128-wide tile: 512 (four warps per TMEM lane quarter, 32 columns each) measured 2-4 %
// faster than 256 on the memory-bound shapes once the TMA stores had moved to their own warp.
#ifndef SRPC_EPI128
#define SRPC_EPI128 512
#endif
// Output staging buffers per CTA.  A TMA store holds its buffer until the write has drained, which takes a few
// microseconds under load; with too few buffers the epilogue stalls on them and the store stream, not DRAM, sets
// the pace of memory-bound shapes.
constexpr int OUT_BUFS = 3;
constexpr int MAX_OUT_BUFS = 4;
// How many tiles ahead the residual tile is loaded (see TileParams::res_tma).
constexpr int RES_DIST = 2;
// warp 0 TMA, warp 1 MMA, then two epilogue warps per TMEM lane quarter (each takes half of the tile's columns)
template <int BN>
struct Threads {
  // BN = 256 / 192: four / three warps per quarter, 64 columns each
  static constexpr int EPI = BN == 256 ? 512 : (BN == 192 ? 384 : (BN == 128 ? SRPC_EPI128 : 256));
  static constexpr int TOTAL = 64 + EPI + 32;  // + the store warp
};

// Division by a launch-time constant as multiply-high + shift (dividends below 2^24): every thread of every role
// decodes a tile index per tile, and with small tiles the hardware divisions were a quarter of a microsecond per tile.
struct FastDiv {
  uint32_t mul, shr, d;
};
static inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  f.d = d ? d : 1;
  uint32_t l = 0;
  while ((1u << l) < f.d) l++;
  f.shr = l;
  f.mul = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << l) - f.d)) / f.d + 1);
  return f;
}
__device__ __forceinline__ uint32_t fdiv(const FastDiv& f, uint32_t n) { return (__umulhi(f.mul, n) + n) >> f.shr; }

struct TileParams {
  int mode;          // 0 GEMM, 1 convolution
  int M, N, K;       // GEMM view (M = rows, N = columns)
  int num_kb;
  int tiles_m, tiles_n;
  // convolution
  int pw, ph, pn;            // output patch of one tile
  int tiles_w, tiles_h;      // tiles along W and H (tiles_m = tiles_w * tiles_h * tiles_img)
  int oh, ow, nimg;
  int r, s, cblocks, stride, pad;
  uint32_t a_box_bytes;      // bytes one A box writes
  int rows_used;             // pw * ph * pn
  // B-stationary schedule (few k-blocks): every CTA keeps one column block for its whole life, loads that B panel into
  // shared memory once and streams only A.  Without it every tile re-reads the same few KB of weights from L2 and the
  // handful of L2 lines that hold them becomes the bottleneck of the whole GPU.
  int b_stationary;
  int ctas_per_n;            // CTAs that share one column block (grid = ctas_per_n * tiles_n)
  // Residual through TMA: the residual tile of a later tile is loaded into that tile's output staging buffer while
  // earlier tiles are still in their epilogue; the epilogue then adds the accumulator to it in place.  Plain loads
  // of the residual from the epilogue threads leave each of them waiting a full DRAM round trip per tile.
  int res_tma;
  // Row-tap reuse (stride-1 convolutions, patch width a multiple of 8): one A box per (filter column, channel block)
  // holds the patch rows with their halo (ph + r - 1 image rows), and the r filter rows are r groups of MMAs whose A
  // descriptors start fr * pw rows further into that box: a third of the loads (and of the round trips that pace a
  // short-tile k loop) for a 3 x 3 filter.  num_kb then counts load groups (s * cblocks); panel_kb counts all k-blocks.
  int reuse;
  int panel_kb;
  FastDiv fd_tiles_n, fd_group, fd_tiles_w, fd_tiles_h;  // filled in by launch()
  // Input that lives in a request ring (convolution mode): the tensor map covers the whole ring, one "image" per slot,
  // and the batch starts at the slot that the app stub's request pointer names when the kernel runs, so one captured
  // graph serves every ring position.  in_stub == nullptr: the input starts at image 0.
  const void* in_stub;
  unsigned long long in_ring_base;
  unsigned int in_slot_bytes;
  // two-input 1x1 convolution: k-blocks from kb_split on come from the second input (pixel stride2, no padding)
  int kb_split, stride2;
};

__device__ __forceinline__ float gelu_f(float x) { return ptx::gelu_erf_fast(x); }

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Barrier over `count` threads that also returns the AND of their predicates.
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

__device__ __forceinline__ void tma_load_4d_box(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                                int c3) {
  ptx::tma_load_4d(smem_dst, m, bar, c0, c1, c2, c3);
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(m),
               "r"(ptx::smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

// Optional phase time stamps of block 0 (build with -DSRPC_GEMM_TRACE): where a short kernel spends its time.
#ifdef SRPC_GEMM_TRACE
__device__ unsigned long long g_gemm_trace[16];
#define GEMM_TRACE(slot)                                                         \
  do {                                                                           \
    if (blockIdx.x == 0) g_gemm_trace[slot] = ptx::globaltimer_ns();             \
  } while (0)
#else
#define GEMM_TRACE(slot) ((void)0)
#endif

struct TileCoord {
  int m_idx, n_idx;
  int w0, h0, img0;  // convolution patch origin (output pixels)
};

// j-th tile of this CTA; false when the CTA has no more tiles.
__device__ __forceinline__ bool get_tile(const TileParams& p, int j, TileCoord* out) {
  TileCoord t;
  if (p.b_stationary) {
    const uint32_t q = fdiv(p.fd_tiles_n, blockIdx.x);
    t.n_idx = (int)(blockIdx.x - q * (uint32_t)p.tiles_n);
    t.m_idx = (int)q + j * p.ctas_per_n;
    if (t.m_idx >= p.tiles_m) return false;
  } else {
    const int tile = (int)blockIdx.x + j * (int)gridDim.x;
    if (tile >= p.tiles_m * p.tiles_n) return false;
    // Grouped order: the ~148 tiles in flight at any time cover GROUP_M row blocks x ~18 column blocks, so the A and
    // B blocks they share are read from DRAM once and then hit in L2.
    constexpr int GROUP_M = 8;
    const int per_group = GROUP_M * p.tiles_n;
    const int g = (int)fdiv(p.fd_group, (uint32_t)tile), in_g = tile - g * per_group;
    const int m_first = g * GROUP_M;
    const int gm = (p.tiles_m - m_first) < GROUP_M ? (p.tiles_m - m_first) : GROUP_M;
    if (gm == GROUP_M) {
      t.m_idx = m_first + (in_g & (GROUP_M - 1));
      t.n_idx = in_g >> 3;
    } else {  // last, shorter group
      t.m_idx = m_first + in_g % gm;
      t.n_idx = in_g / gm;
    }
  }
  t.w0 = t.h0 = t.img0 = 0;
  if (p.mode == 1) {
    const int rest = (int)fdiv(p.fd_tiles_w, (uint32_t)t.m_idx);
    const int tw = t.m_idx - rest * p.tiles_w;
    const int ti = (int)fdiv(p.fd_tiles_h, (uint32_t)rest);
    const int th = rest - ti * p.tiles_h;
    t.w0 = tw * p.pw;
    t.h0 = th * p.ph;
    t.img0 = ti * p.pn;
  }
  *out = t;
  return true;
}

template <int BN, int STAGES, int OB>
__global__ void __launch_bounds__(Threads<BN>::TOTAL, 1)
gemm_conv_persistent(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_res, TileParams p,
                     GemmEpilogue ep, int use_tma_store, uint32_t* status) {
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int OUT_HALF_BYTES = BM * 128;       // 128 rows x 64 bf16 columns
  constexpr int OUT_BYTES = (BN / 64) * OUT_HALF_BYTES;
  // No slack for manual alignment: the widest configuration then leaves 2 KB of the SM's shared memory, which is what
  // one small block of another stream (the scatter-gather kernel) needs to share the SM; a block that takes all of
  // it keeps every other block off its SM.
  extern __shared__ __align__(1024) uint8_t smem[];
  const bool layout_ok = (ptx::smem_u32(smem) & 1023u) == 0;
  uint8_t* stage_out = smem + (size_t)STAGES * STAGE_BYTES;
  constexpr int MAX_STAGES = 8;
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t bpanel_bar;
  // Streaming: STAGES stages of {A tile, B tile}.  B-stationary: the B panel (num_kb tiles) first, then a ring of A tiles.
  const int panel_bytes = p.b_stationary ? p.panel_kb * B_BYTES : 0;
  const int b_per_stage = p.b_stationary ? 0 : (p.reuse ? p.r : 1);  // B tiles that travel with every A box
  const int a_stride = A_BYTES + b_per_stage * B_BYTES;
  int nst_calc = (STAGES * STAGE_BYTES - panel_bytes) / a_stride;
  const int nst = nst_calc > MAX_STAGES ? MAX_STAGES : nst_calc;
  uint8_t* a_ring = smem + panel_bytes;
  // Four TMEM accumulators: up to four tiles can be between "MMA issued" and "accumulator read back", which hides
  // the commit -> wake-up -> tcgen05.ld -> release round trip of short (few k-block) tiles.
  constexpr int ACC = BN >= 192 ? 2 : 4;
  constexpr int ACC_LOG2 = BN >= 192 ? 1 : 2;
  constexpr int ACC_STRIDE = BN == 192 ? 256 : BN;  // TMEM columns between accumulators (allocation is a power of two)
  static_assert(OB >= 1 && OB <= MAX_OUT_BUFS, "output staging buffers");
  __shared__ __align__(8) uint64_t tmem_full_bar[ACC];
  __shared__ __align__(8) uint64_t tmem_empty_bar[ACC];
  __shared__ __align__(8) uint64_t res_full_bar[MAX_OUT_BUFS];
  // Staging buffers: the epilogue warps announce a finished tile on out_full, the store warp's thread issues the TMA
  // stores (and the next residual loads) and hands the buffer back on out_empty once the store has read it.  The
  // epilogue warps never wait for a TMA instruction to issue: that took 0.6 - 0.7 us per tile on their critical path.
  __shared__ __align__(8) uint64_t out_full_bar[MAX_OUT_BUFS];
  __shared__ __align__(8) uint64_t out_empty_bar[MAX_OUT_BUFS];
  __shared__ uint32_t tmem_base_smem;
  __shared__ uint32_t s_error;
  // Bias of the current tile's columns, double-buffered over consecutive tiles: fetched while the accumulator is still
  // being computed, then read as broadcasts (a global load per chunk would sit on the epilogue's critical path).
  __shared__ __align__(16) float s_bias[2][BN];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    GEMM_TRACE(0);
    ptx::mbar_init(&bpanel_bar, 1);
    for (int s = 0; s < MAX_STAGES; s++) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < ACC; a++) {
      ptx::mbar_init(&tmem_full_bar[a], 1);
      ptx::mbar_init(&tmem_empty_bar[a], Threads<BN>::EPI / 32);  // one arrival per epilogue warp
    }
    for (int b = 0; b < MAX_OUT_BUFS; b++) {
      ptx::mbar_init(&res_full_bar[b], 1);
      ptx::mbar_init(&out_full_bar[b], Threads<BN>::EPI / 32);
      ptx::mbar_init(&out_empty_bar[b], 1);
    }
    ptx::fence_mbar_init();
    s_error = layout_ok ? 0u : (uint32_t)GEMM_ERR_PRODUCER_WAIT;
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    if (use_tma_store) ptx::prefetch_tmap(&tmap_out);
    if (p.res_tma) ptx::prefetch_tmap(&tmap_res);
  }
  // TMA producer = thread 0.  Its state lives across two calls: the first fills the (initially free) ring right after
  // the barriers exist, before the block-wide set-up barrier, so that the first operands are already in flight while
  // tensor memory is being allocated; the second runs the rest of the schedule.
  int pr_s = 0, pr_j = 0, pr_kb = 0;
  uint32_t pr_ph = 0;
  bool pr_more = true;
  int img_off = 0;
  if (threadIdx.x == 0 && p.in_stub)
    img_off = (int)((*reinterpret_cast<const unsigned long long*>(p.in_stub) - p.in_ring_base) / p.in_slot_bytes);
  auto produce = [&](int budget) {
    const uint32_t b_tx = (uint32_t)(b_per_stage * B_BYTES);
    TileCoord tc;
    while (pr_more && budget > 0) {
      if (!get_tile(p, pr_j, &tc) || *(volatile uint32_t*)&s_error != 0) {
        pr_more = false;
        break;
      }
      for (; pr_kb < p.num_kb && budget > 0; pr_kb++, budget--) {
        if (!ptx::mbar_wait(&empty_bar[pr_s], pr_ph ^ 1u)) {
          atomicExch(&s_error, GEMM_ERR_PRODUCER_WAIT);
          pr_more = false;
          return;
        }
        uint8_t* sa = a_ring + (size_t)pr_s * a_stride;
        if (p.mode == 0) {
          ptx::mbar_expect_tx(&full_bar[pr_s], (uint32_t)A_BYTES + b_tx);
          ptx::tma_load_2d(sa, &tmap_a, &full_bar[pr_s], pr_kb * BK, tc.m_idx * BM);
        } else if (p.reuse) {
          // load group (fs, cb): the box covers filter rows 0 .. r-1 at once
          ptx::mbar_expect_tx(&full_bar[pr_s], p.a_box_bytes + b_tx);
          const int fs = pr_kb / p.cblocks, cb = pr_kb - fs * p.cblocks;
          tma_load_4d_box(sa, &tmap_a, &full_bar[pr_s], cb * BK, tc.w0 + fs - p.pad, tc.h0 - p.pad, tc.img0 + img_off);
          if (!p.b_stationary)
            for (int fr = 0; fr < p.r; fr++)
              ptx::tma_load_2d(sa + A_BYTES + fr * B_BYTES, &tmap_b, &full_bar[pr_s], ((fr * p.s + fs) * p.cblocks + cb) * BK,
                               tc.n_idx * BN);
        } else {
          ptx::mbar_expect_tx(&full_bar[pr_s], p.a_box_bytes + b_tx);
          if (pr_kb >= p.kb_split) {
            // second input of a two-input 1x1 convolution (its map travels in the residual map's place)
            tma_load_4d_box(sa, &tmap_res, &full_bar[pr_s], (pr_kb - p.kb_split) * BK, tc.w0 * p.stride2, tc.h0 * p.stride2,
                            tc.img0);
          } else {
            const int tap = pr_kb / p.cblocks, cb = pr_kb - tap * p.cblocks;
            const int fr = tap / p.s, fs = tap - fr * p.s;
            tma_load_4d_box(sa, &tmap_a, &full_bar[pr_s], cb * BK, tc.w0 * p.stride + fs - p.pad,
                            tc.h0 * p.stride + fr - p.pad, tc.img0 + img_off);
          }
        }
        if (!p.b_stationary && !p.reuse) ptx::tma_load_2d(sa + A_BYTES, &tmap_b, &full_bar[pr_s], pr_kb * BK, tc.n_idx * BN);
        if (pr_j == 0 && pr_kb == 0) GEMM_TRACE(2);
        if (++pr_s == nst) {
          pr_s = 0;
          pr_ph ^= 1u;
        }
      }
      if (pr_kb == p.num_kb) {
        pr_kb = 0;
        pr_j++;
      }
    }
  };
  if (threadIdx.x == 0 && layout_ok) {
    TileCoord tc;
    if (p.b_stationary && get_tile(p, 0, &tc)) {
      ptx::mbar_expect_tx(&bpanel_bar, (uint32_t)panel_bytes);
      for (int kb = 0; kb < p.panel_kb; kb++)
        ptx::tma_load_2d(smem + (size_t)kb * B_BYTES, &tmap_b, &bpanel_bar, kb * BK, tc.n_idx * BN);
    }
    produce(nst < 2 ? nst : 2);  // more would hold thread 0 (and with it the set-up barrier) behind a full TMA queue
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_base_smem, ACC * ACC_STRIDE);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  if (threadIdx.x == 0) GEMM_TRACE(1);

  if (threadIdx.x == 0) {
    produce(1 << 30);  // the rest of the k-blocks, paced by the MMA warp through the empty barriers
  } else if (warp == 0) {
    // lanes 1-31 of the producer warp have nothing to do
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      const uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
      uint32_t local = 0;
      int s = 0;
      uint32_t ph = 0;
      TileCoord tc;
      bool panel_ok = true;
      if (p.b_stationary && get_tile(p, 0, &tc)) {
        panel_ok = ptx::mbar_wait(&bpanel_bar, 0);
        if (!panel_ok) atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
      }
      for (int j = 0; panel_ok && get_tile(p, j, &tc) && *(volatile uint32_t*)&s_error == 0; j++, local++) {
        const uint32_t acc = local & (ACC - 1);
        if (!ptx::mbar_wait(&tmem_empty_bar[acc], ((local >> ACC_LOG2) & 1u) ^ 1u)) {
          atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        bool ok = true;
        for (int kb = 0; kb < p.num_kb; kb++) {
          if (!ptx::mbar_wait(&full_bar[s], ph)) {
            atomicExch(&s_error, GEMM_ERR_MMA_WAIT);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          if (j == 0 && kb == 0) GEMM_TRACE(3);
          const uint32_t sa = ptx::smem_u32(a_ring + (size_t)s * a_stride);
          if (p.reuse) {
            const int fs = kb / p.cblocks, cb = kb - fs * p.cblocks;
            for (int fr = 0; fr < p.r; fr++) {
              const uint32_t sa_fr = sa + (uint32_t)(fr * p.pw * 128);  // fr image rows further into the box
              const uint32_t sb = p.b_stationary
                                      ? ptx::smem_u32(smem + (size_t)((fr * p.s + fs) * p.cblocks + cb) * B_BYTES)
                                      : sa + A_BYTES + fr * B_BYTES;
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; k++)
                ptx::umma_bf16(d_tmem, ptx::umma_desc_sw128(sa_fr + k * UMMA_K * 2), ptx::umma_desc_sw128(sb + k * UMMA_K * 2),
                               idesc, (kb | fr | k) != 0 ? 1u : 0u);
            }
          } else {
            const uint32_t sb = p.b_stationary ? ptx::smem_u32(smem + (size_t)kb * B_BYTES) : sa + A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; k++)
              ptx::umma_bf16(d_tmem, ptx::umma_desc_sw128(sa + k * UMMA_K * 2), ptx::umma_desc_sw128(sb + k * UMMA_K * 2), idesc,
                             (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[s]);
          if (++s == nst) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit(&tmem_full_bar[acc]);
        if (j == 0) GEMM_TRACE(4);
      }
    }
  } else if (warp < 2 + Threads<BN>::EPI / 32) {
    // ---------------- epilogue warps (8): warp pair (w, w+4) shares a TMEM lane quarter and splits the columns
    constexpr int CPW = BN / (Threads<BN>::EPI / 128);  // columns per warp
    constexpr bool LEAN = BN >= 192 || Threads<BN>::EPI > 256;     // 14-18 warps per CTA: keep the accumulator in registers one chunk at a time
    constexpr int NCH = CPW / 32;        // 32-column chunks per warp
    constexpr int EPI_THREADS = Threads<BN>::EPI;
    const int warp_q = warp & 3;
    const int chalf = (warp - 2) >> 2;   // which 32-column group of the tile this warp takes
    const int row = warp_q * 32 + lane;  // row of the tile this thread owns
    const int et = threadIdx.x - 64;     // 0..255 among the epilogue threads
    const bool res_tma = OB > RES_DIST && p.res_tma != 0;
    const bool vec_res = !res_tma && ep.residual && ((ep.ldr & 7) == 0) && (((uintptr_t)ep.residual & 15) == 0);
    uint32_t local = 0;
    TileCoord tc;
    // Position of this thread's row inside a convolution patch (the same for every tile).
    int pw_i = 0, ph_i = 0, pn_i = 0;
    if (p.mode == 1) {
      const int rest = row / p.pw;
      pw_i = row - rest * p.pw;
      pn_i = rest / p.ph;
      ph_i = rest - pn_i * p.ph;
    }
    for (int j = 0; get_tile(p, j, &tc); j++, local++) {
      const uint32_t acc = local & (ACC - 1);
      // Where this thread's row lives in the output.
      bool row_ok;
      size_t row_off;  // pixel / row index (leading dimension not yet applied)
      if (p.mode == 0) {
        const int m = tc.m_idx * BM + row;
        row_ok = m < p.M;
        row_off = (size_t)m;
      } else {
        const int x = tc.w0 + pw_i, y = tc.h0 + ph_i, img = tc.img0 + pn_i;
        row_ok = row < p.rows_used && x < p.ow && y < p.oh && img < p.nimg;
        row_off = ((size_t)img * p.oh + y) * p.ow + x;
      }
      const int n0 = tc.n_idx * BN;
      const int cbase = chalf * CPW;  // first tile column of this warp
      // Residual rows are fetched before the accumulator is awaited, so their latency hides behind the MMAs.
      uint4 resq[LEAN ? 1 : CPW / 8];
      const bool res_vec_tile = vec_res && row_ok && (n0 + cbase + CPW <= p.N);
      if (!LEAN && res_vec_tile) {
        const __nv_bfloat16* rp = ep.residual + row_off * ep.ldr + n0 + cbase;
#pragma unroll
        for (int j = 0; j < CPW / 8; j++) resq[j] = __ldg(reinterpret_cast<const uint4*>(rp) + j);
      }
      if (j == 5 && et == 0) GEMM_TRACE(10);
      float* bias_s = s_bias[local & 1u];
      if (ep.bias && et < BN) bias_s[et] = (n0 + et < p.N) ? __ldg(ep.bias + n0 + et) : 0.f;
      // Each thread's wait is bounded; the vote makes the outcome uniform so that no
      // thread is left alone at a later barrier.  (It also orders the bias writes before their reads.)
      bool mine = (*(volatile uint32_t*)&s_error == 0) && ptx::mbar_wait(&tmem_full_bar[acc], (local >> ACC_LOG2) & 1u);
      // The staging buffer: with a prefetched residual it is ready when the residual has landed (the store warp loads
      // it only into a buffer whose last store has been read); otherwise when the store warp has handed it back.
      if (res_tma && mine) mine = ptx::mbar_wait(&res_full_bar[local % OB], (local / OB) & 1u);
      else if (use_tma_store && mine) mine = ptx::mbar_wait(&out_empty_bar[local % OB], ((local / OB) & 1u) ^ 1u);
      if (!named_bar_all(2, EPI_THREADS, mine)) {
        if (lane == 0) atomicExch(&s_error, GEMM_ERR_EPILOGUE_WAIT);
        break;
      }
      ptx::tc_fence_after();
      if (j == 0 && et == 0) GEMM_TRACE(5);
      if (j == 5 && et == 0) GEMM_TRACE(11);
      uint32_t r[LEAN ? 32 : CPW];
      const uint32_t t_addr = tmem_base + acc * ACC_STRIDE + ((uint32_t)(warp_q * 32) << 16) + (uint32_t)cbase;
      if (!LEAN) {
#pragma unroll
        for (int ch = 0; ch < NCH; ch++) ptx::tmem_ld_32x32b_x32(t_addr + ch * 32, r + ch * 32);
        ptx::tmem_ld_wait();
        // Accumulator is in registers: give it back to the MMA warp right away.
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&tmem_empty_bar[acc]);
      }
      if (j == 5 && et == 0) GEMM_TRACE(12);
      uint8_t* sbuf = stage_out + (size_t)(local % OB) * OUT_BYTES;
#pragma unroll
      for (int ch = 0; ch < NCH; ch++) {
        const int c = cbase + ch * 32;  // tile column of this chunk
        const int col0 = n0 + c;
        if (LEAN) {
          ptx::tmem_ld_32x32b_x32(t_addr + ch * 32, r);
          ptx::tmem_ld_wait();
          if (ch == NCH - 1) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tmem_empty_bar[acc]);
          }
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[(LEAN ? 0 : ch * 32) + j]);
        if (ep.bias) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 b4 = *reinterpret_cast<const float4*>(bias_s + c + j);
            v[j] += b4.x;
            v[j + 1] += b4.y;
            v[j + 2] += b4.z;
            v[j + 3] += b4.w;
          }
        }
        if (res_tma) {
          const uint8_t* half = sbuf + (size_t)(c >> 6) * OUT_HALF_BYTES + (size_t)row * 128;
          const int chunk0 = (c & 63) >> 3;
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint4 q = *reinterpret_cast<const uint4*>(half + (((chunk0 + j) ^ (row & 7)) << 4));
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
            for (int t = 0; t < 4; t++) {
              float2 f = __bfloat1622float2(h[t]);
              v[j * 8 + 2 * t] += f.x;
              v[j * 8 + 2 * t + 1] += f.y;
            }
          }
        } else if (ep.residual && row_ok && col0 < p.N) {
          if (res_vec_tile) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
              if (LEAN) resq[0] = __ldg(reinterpret_cast<const uint4*>(ep.residual + row_off * ep.ldr + col0) + j);
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&resq[LEAN ? 0 : ch * 4 + j]);
#pragma unroll
              for (int t = 0; t < 4; t++) {
                float2 f = __bfloat1622float2(h[t]);
                v[j * 8 + 2 * t] += f.x;
                v[j * 8 + 2 * t + 1] += f.y;
              }
            }
          } else {
            const __nv_bfloat16* rp = ep.residual + row_off * ep.ldr + col0;
            #pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < p.N) v[j] += __bfloat162float(rp[j]);
          }
        }
        if (ep.act == GEMM_ACT_RELU) {
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = fmaxf(v[j], 0.f);
        } else if (ep.act == GEMM_ACT_GELU) {
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = gelu_f(v[j]);
        } else if (ep.act == GEMM_ACT_TANH) {
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = tanhf(v[j]);
        }
        if (use_tma_store) {
          uint8_t* half = sbuf + (size_t)(c >> 6) * OUT_HALF_BYTES + (size_t)row * 128;
          const int chunk0 = (c & 63) >> 3;  // first 16-byte chunk of this 32-column group inside the 128-byte row
#pragma unroll
          for (int j = 0; j < 4; j++) {
            uint4 q;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
            for (int t = 0; t < 4; t++) h[t] = __floats2bfloat162_rn(v[j * 8 + 2 * t], v[j * 8 + 2 * t + 1]);
            *reinterpret_cast<uint4*>(half + (((chunk0 + j) ^ (row & 7)) << 4)) = q;
          }
        } else if (row_ok && col0 < p.N) {
          if (ep.out_fp32) {
            float* op = reinterpret_cast<float*>(ep.out) + row_off * ep.ldo + col0;
            #pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < p.N) op[j] = v[j];
          } else {
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(ep.out) + row_off * ep.ldo + col0;
            #pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < p.N) op[j] = __float2bfloat16(v[j]);
          }
        }
      }
      if (j == 5 && et == 0) GEMM_TRACE(13);
      if (use_tma_store) {
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&out_full_bar[local % OB]);
      }
    }
  } else if (lane == 0 && use_tma_store) {
    // ---------------- store warp (one thread): TMA stores of finished tiles, residual prefetch, buffer hand-back
    const bool res_tma = OB > RES_DIST && p.res_tma != 0;
    // Loads the residual tile of this CTA's jj-th tile into staging buffer jj % OB (one elected thread).
    auto load_residual = [&](int jj) {
      TileCoord tn;
      if (!get_tile(p, jj, &tn)) return;
      const int b = jj % OB;
      uint8_t* dst = stage_out + (size_t)b * OUT_BYTES;
      int boxes = 0;
      for (int hcol = 0; hcol < BN / 64; hcol++)
        if (tn.n_idx * BN + hcol * 64 < p.N) boxes++;
      ptx::mbar_expect_tx(&res_full_bar[b], (uint32_t)(boxes * OUT_HALF_BYTES));
      for (int hcol = 0; hcol < boxes; hcol++)
        ptx::tma_load_2d(dst + (size_t)hcol * OUT_HALF_BYTES, &tmap_res, &res_full_bar[b], tn.n_idx * BN + hcol * 64,
                         tn.m_idx * BM);
    };
    if (res_tma) {
      for (int jj = 0; jj < RES_DIST; jj++) load_residual(jj);
    }
    uint32_t local = 0;
    TileCoord tc;
    for (int j = 0; get_tile(p, j, &tc) && *(volatile uint32_t*)&s_error == 0; j++, local++) {
      const int b = (int)(local % OB);
      if (!ptx::mbar_wait(&out_full_bar[b], (local / OB) & 1u)) {
        atomicExch(&s_error, GEMM_ERR_EPILOGUE_WAIT);
        break;
      }
      const int n0 = tc.n_idx * BN;
      const uint8_t* sbuf = stage_out + (size_t)b * OUT_BYTES;
#pragma unroll
      for (int hcol = 0; hcol < BN / 64; hcol++) {
        if (n0 + hcol * 64 >= p.N) break;
        const void* src = sbuf + (size_t)hcol * OUT_HALF_BYTES;
        if (p.mode == 0) ptx::tma_store_2d(&tmap_out, src, n0 + hcol * 64, tc.m_idx * BM);
        else tma_store_4d(&tmap_out, src, n0 + hcol * 64, tc.w0, tc.h0, tc.img0);
      }
      ptx::bulk_commit();
      if (j == 0) GEMM_TRACE(6);
      if (res_tma) {
        // The tile RES_DIST ahead takes the buffer of the tile OB - RES_DIST back, so all stores but the last
        // OB - RES_DIST must have been read.
        ptx::bulk_wait_read<(OB > RES_DIST ? OB - RES_DIST : 0)>();
        load_residual(j + RES_DIST);
      } else if (OB == 1) {
        ptx::bulk_wait_read<0>();
        ptx::mbar_arrive(&out_empty_bar[0]);
      } else {
        // all stores but this one have been read: the previous tile's buffer is free again
        ptx::bulk_wait_read<1>();
        if (j >= 1) ptx::mbar_arrive(&out_empty_bar[(local - 1) % OB]);
      }
    }
    GEMM_TRACE(7);
    ptx::bulk_wait_all<0>();
    GEMM_TRACE(8);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) GEMM_TRACE(9);
  if (s_error != 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, s_error);
    __nanosleep(1000000);  // let loads that are still in flight land before the block leaves
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, ACC * ACC_STRIDE);
  }
}

// ------------------------------------------------------------------ host side
struct MapKey {
  const void* ptr;
  uint64_t d[5];
  uint64_t st[4];
  uint32_t box[5];
  uint32_t es[5];
  int rank;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; i++) h = (h ^ w[i]) * 1099511628211ull;
    return h;
  }
};

// Tensor maps are cached: encoding costs microseconds and the same layers run
// for every batch.
cudaError_t get_map(CUtensorMap* out, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, const uint32_t* estr) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey k;
  std::memset(&k, 0, sizeof(k));
  k.ptr = ptr;
  k.rank = rank;
  for (int i = 0; i < rank; i++) {
    k.d[i] = dims[i];
    k.box[i] = box[i];
    k.es[i] = estr[i];
    if (i + 1 < rank) k.st[i] = strides_bytes[i];
  }
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(k);
  if (it != cache.end()) {
    *out = it->second;
    return cudaSuccess;
  }
  const SrpcDriverApi* d = srpc_driver_api();
  if (!d->TensorMapEncodeTiled) return cudaErrorNotSupported;
  cuuint64_t gd[5], gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; i++) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = estr[i];
    if (i + 1 < rank) gs[i] = strides_bytes[i];
  }
  CUresult r = d->TensorMapEncodeTiled(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), gd, gs,
                                       bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(k, *out);
  return cudaSuccess;
}

cudaError_t map_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                   uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer}, st[1] = {row_stride_bytes};
  uint32_t box[2] = {box_inner, box_outer}, es[2] = {1, 1};
  return get_map(m, ptr, 2, dims, st, box, es);
}

// SMs that the persistent kernels size their grids for.  A persistent kernel has one block per SM and a fixed tile
// schedule; if a block of another stream (the scatter-gather kernel that runs beside the model) holds an SM, one of
// this kernel's blocks starts only when another has finished and the whole kernel takes twice as long.  Leaving a
// few SMs out of the grid keeps room for such blocks (srpc_gemm_reserve_sms, or SPLITRPC_GEMM_RESERVE_SMS).
int g_reserve_sms = -1;
int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  if (g_reserve_sms < 0) {
    const char* e = getenv("SPLITRPC_GEMM_RESERVE_SMS");
    g_reserve_sms = e ? atoi(e) : 0;
  }
  const int r = g_reserve_sms < n / 2 ? g_reserve_sms : n / 2;
  return n - r;
}

template <int BN, int STAGES, int OB>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tr,
                   const TileParams& p_in, const GemmEpilogue& ep, int use_tma_store, uint32_t* status, cudaStream_t st) {
  static PerDeviceFlag attr;
  const int dev = PerDeviceFlag::current();
  const int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + OB * (BN / 64) * BM * 128;
  if (attr.needed(dev)) {
    cudaError_t e = cudaFuncSetAttribute(gemm_conv_persistent<BN, STAGES, OB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr.set(dev);
  }
  TileParams p = p_in;
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = std::min(tiles, num_sms());
  p.b_stationary = 0;
  p.ctas_per_n = 0;
  p.fd_tiles_n = make_fastdiv((uint32_t)p.tiles_n);
  p.fd_group = make_fastdiv((uint32_t)(8 * p.tiles_n));  // GROUP_M row blocks x all column blocks (see get_tile)
  p.fd_tiles_w = make_fastdiv((uint32_t)(p.tiles_w > 0 ? p.tiles_w : 1));
  p.fd_tiles_h = make_fastdiv((uint32_t)(p.tiles_h > 0 ? p.tiles_h : 1));
  static const int allow_bs = [] { const char* e = getenv("SPLITRPC_GEMM_BSTAT"); return e ? atoi(e) : 1; }();
  // The panel may take the ring's memory as long as three A stages remain (a 3x3 convolution over 64 channels keeps its
  // nine 8 KB filter taps resident: otherwise every CTA re-reads the same few L2 lines for every tile).
  const int panel = p.panel_kb * BN * BK * 2, ring = STAGES * (BM * BK * 2 + BN * BK * 2);
  const bool panel_fits = p.mode == 1 ? panel + 3 * BM * BK * 2 <= ring : p.num_kb <= (BN >= 192 ? 2 : 4);
  if (allow_bs && panel_fits && p.tiles_n <= num_sms()) {
    const int per_n = std::min(num_sms() / p.tiles_n, p.tiles_m);
    if (per_n >= 1 && p.tiles_m >= 2 * per_n) {  // at least two tiles per CTA to pay for the panel load
      p.b_stationary = 1;
      p.ctas_per_n = per_n;
      grid = per_n * p.tiles_n;
    }
  }
  gemm_conv_persistent<BN, STAGES, OB><<<grid, Threads<BN>::TOTAL, smem, st>>>(ta, tb, to, tr, p, ep, use_tma_store, status);
  return cudaGetLastError();
}

cudaError_t dispatch(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tr,
                     const TileParams& p, const GemmEpilogue& ep, int use_tma_store, uint32_t* status, cudaStream_t st) {
  // Long k loops run at (round trip MMA done -> stage free -> TMA -> stage full) / (stages): give them the staging
  // buffers' memory as extra stages.  Short k loops are bound by the output stream and keep three staging buffers.
  static const int allow_deep = [] { const char* e = getenv("SPLITRPC_GEMM_DEEP"); return e ? atoi(e) : 1; }();
  const bool deep = allow_deep && !p.res_tma && p.panel_kb >= 8;
  if (bn == 64) {
    if (deep) return launch<64, 8, 1>(ta, tb, to, tr, p, ep, use_tma_store, status, st);
    return launch<64, 6, OUT_BUFS>(ta, tb, to, tr, p, ep, use_tma_store, status, st);
  }
  if (bn == 256) return launch<256, 3, 1>(ta, tb, to, tr, p, ep, use_tma_store, status, st);
  if (bn == 192) return launch<192, 4, 1>(ta, tb, to, tr, p, ep, use_tma_store, status, st);
  if (deep) return launch<128, 6, 1>(ta, tb, to, tr, p, ep, use_tma_store, status, st);
  return launch<128, 4, OUT_BUFS>(ta, tb, to, tr, p, ep, use_tma_store, status, st);
}

}  // namespace

void srpc_gemm_reserve_sms(int n) { g_reserve_sms = n < 0 ? 0 : n; }
int srpc_gemm_grid_sms() { return num_sms(); }
int srpc_gemm_reserved_sms() {
  (void)num_sms();
  return g_reserve_sms > 0 ? g_reserve_sms : 0;
}

cudaError_t srpc_tensor_map_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                               uint32_t box_inner, uint32_t box_outer) {
  return map_2d(m, ptr, inner, outer, row_stride_bytes, box_inner, box_outer);
}

int srpc_gemm_trace_read(unsigned long long* out, int n) {
#ifdef SRPC_GEMM_TRACE
  if (n > 16) n = 16;
  if (cudaMemcpyFromSymbol(out, g_gemm_trace, n * sizeof(unsigned long long)) != cudaSuccess) return 0;
  return n;
#else
  (void)out;
  (void)n;
  return 0;
#endif
}

// Tile shape.  Narrow outputs take 64 columns.  Otherwise the shape with the lowest estimated time wins: rounds of
// tiles over the SMs (or SM pairs) x (k-blocks x time per k-block + hand-over).  The per-k-block times are what the
// kernels measure on large problems: the one-SM 128-wide tile is bound by the issue rate of its four MMAs per
// k-block, the wider one-SM tiles by operand delivery, the two-SM tiles (256 rows per SM pair, gemm_2sm.cu) by the
// tensor pipe.  Returns the width; *two_sm says which kernel.
static int pick_tile(int M, int N, int num_kb, bool bf16_out, bool allow_two_sm, bool* two_sm) {
  static const int allow256 = [] { const char* e = getenv("SPLITRPC_GEMM_BN256"); return e ? atoi(e) : 1; }();
  static const int allow192 = [] { const char* e = getenv("SPLITRPC_GEMM_BN192"); return e ? atoi(e) : 1; }();
  *two_sm = false;
  if (N <= 64) return 64;
  struct Cand {
    int bn, rows, units;
    double t_kb;  // microseconds per 64-deep k-block
    bool pair;
  };
  const int sms = num_sms();
  // (the pair kernels run at about 0.4 us per k-block whatever their width: the stage ring covers one round trip
  //  MMA done -> stage free -> TMA -> stage full, not more)
  const Cand cands[6] = {{256, 256, sms / 2, 0.40, true},  {192, 256, sms / 2, 0.40, true}, {128, 256, sms / 2, 0.40, true},
                         {256, 128, sms, 0.49, false},     {192, 128, sms, 0.37, false},    {128, 128, sms, 0.27, false}};
  int best = 128;
  double best_cost = 1e30;
  for (const Cand& c : cands) {
    // pairs only where the k loop dominates: short-K shapes are bound by memory and keep the B-stationary schedule
    if (c.pair && !(allow_two_sm && M >= 256 && num_kb >= 8)) continue;
    if (c.bn == 256 && !(allow256 && bf16_out && N >= 256 && ((N % 256) == 0 || N >= 1024))) continue;
    if (c.bn == 192 && !(allow192 && bf16_out && N >= 192 && ((N % 192) == 0 || N >= 1536))) continue;
    if (c.pair && c.bn == 128 && (N % 128) != 0 && N < 1024) continue;
    const long tiles = (long)((M + c.rows - 1) / c.rows) * ((N + c.bn - 1) / c.bn);
    const long rounds = (tiles + c.units - 1) / c.units;
    const double cost = (double)rounds * (num_kb * c.t_kb + 0.25) + (c.pair ? 0.3 : 0.0);  // pairs: cluster set-up
    if (cost < best_cost * 0.98) {  // near-ties go to the candidate listed first
      best_cost = cost;
      best = c.bn;
      *two_sm = c.pair;
    }
  }
  return best;
}

static int pick_bn(int N, int tiles_m, int num_kb, bool bf16_out) {
  bool two_sm;
  return pick_tile(tiles_m * BM, N, num_kb, bf16_out, false, &two_sm);
}

cudaError_t srpc_gemm_bf16_v2(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                              uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  if ((lda % 8) || (ldb % 8) || (K % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return cudaErrorInvalidValue;
  if (ep.bias && ((uintptr_t)ep.bias & 15)) return cudaErrorInvalidValue;
  int use_tma_store = (!ep.out_fp32 && (ep.ldo % 8) == 0 && ((uintptr_t)ep.out & 15) == 0) ? 1 : 0;
  static const int allow_res_tma = [] { const char* e = getenv("SPLITRPC_GEMM_RES_TMA"); return e ? atoi(e) : 1; }();
  static const int res_tma_max_k = [] { const char* e = getenv("SPLITRPC_GEMM_RES_TMA_MAXK"); return e ? atoi(e) : 512; }();
  // Short-K shapes are bound by memory and gain from the prefetched residual; with a long K the plain residual loads of
  // the epilogue hide behind the next tile's MMAs and the tile width matters more.
  const bool res_tma = allow_res_tma && use_tma_store == 1 && ep.residual && (ep.ldr % 8) == 0 &&
                       ((uintptr_t)ep.residual & 15) == 0 && K <= res_tma_max_k;
  // The residual ring lives in the output staging buffers, which the wide tiles have only one of.
  bool two_sm = false;
  const int bn = res_tma ? (N <= 64 ? 64 : 128)
                         : pick_tile(M, N, (K + BK - 1) / BK, ep.out_fp32 == 0, srpc_gemm_2sm_eligible(M, N, K, ep), &two_sm);
  if (two_sm) return srpc_gemm_bf16_2sm(A, lda, B, ldb, M, N, K, bn, ep, status, stream);
  TileParams p{};
  p.mode = 0;
  p.res_tma = res_tma ? 1 : 0;
  p.M = M;
  p.N = N;
  p.K = K;
  p.num_kb = (K + BK - 1) / BK;
  p.panel_kb = p.num_kb;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + bn - 1) / bn;
  CUtensorMap ta, tb, to;
  cudaError_t e = map_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM);
  if (e != cudaSuccess) return e;
  e = map_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, (uint32_t)bn);
  if (e != cudaSuccess) return e;
  CUtensorMap tr = ta;
  if (use_tma_store == 1) {
    e = map_2d(&to, ep.out, (uint64_t)N, (uint64_t)M, (uint64_t)ep.ldo * 2, 64, BM);
    if (e != cudaSuccess) return e;
    if (res_tma) {
      e = map_2d(&tr, ep.residual, (uint64_t)N, (uint64_t)M, (uint64_t)ep.ldr * 2, 64, BM);
      if (e != cudaSuccess) return e;
    }
  } else {
    to = ta;
  }
  return dispatch(bn, ta, tb, to, tr, p, ep, use_tma_store, status, stream);
}

// Picks the output patch (pw x ph x pn <= 128 pixels) that wastes the fewest tile rows.
static void pick_patch(int ow, int oh, int nimg, int* pw, int* ph, int* pn) {
  if (const char* e = getenv("SPLITRPC_CONV_PATCH")) {  // "w,h,n": experiments with the patch shape
    int w = 0, h = 0, n = 0;
    if (sscanf(e, "%d,%d,%d", &w, &h, &n) == 3 && w >= 1 && h >= 1 && n >= 1 && w * h * n <= 128 && w <= ow && h <= oh && n <= nimg) {
      *pw = w;
      *ph = h;
      *pn = n;
      return;
    }
  }
  double best = -1;
  for (int w = 1; w <= std::min(ow, 64); w++)
    for (int h = 1; h <= std::min(oh, 128 / w); h++) {
      int n = std::min(nimg, 128 / (w * h));
      if (n < 1) continue;
      long tiles = (long)((ow + w - 1) / w) * ((oh + h - 1) / h) * ((nimg + n - 1) / n);
      double eff = (double)ow * oh * nimg / ((double)tiles * 128.0);
      double score = eff + 1e-4 * w;  // ties: longer contiguous runs
      if (score > best) {
        best = score;
        *pw = w;
        *ph = h;
        *pn = n;
      }
    }
}

cudaError_t srpc_conv_bf16_tma(const void* in, const void* weight, const ConvShape& cs, const GemmEpilogue& ep,
                               uint32_t* status, cudaStream_t stream) {
  if (cs.cin % BK || cs.cout % 8) return cudaErrorInvalidValue;
  if (((uintptr_t)in & 15) || ((uintptr_t)weight & 15) || ((uintptr_t)ep.out & 15) || ep.out_fp32) return cudaErrorInvalidValue;
  if (ep.bias && ((uintptr_t)ep.bias & 15)) return cudaErrorInvalidValue;
  TileParams p{};
  p.mode = 1;
  p.oh = cs.oh;
  p.ow = cs.ow;
  p.nimg = cs.n;
  p.M = cs.n * cs.oh * cs.ow;
  p.N = cs.cout;
  p.K = cs.r * cs.s * cs.cin;
  p.r = cs.r;
  p.s = cs.s;
  p.cblocks = cs.cin / BK;
  p.num_kb = cs.r * cs.s * p.cblocks;
  p.kb_split = p.num_kb;
  p.stride2 = 1;
  if (cs.in2) {
    // out = act(W1 . in + W2 . in2(strided) + bias): the weight rows hold [W1 | W2]
    if (cs.r != 1 || cs.s != 1 || cs.pad != 0 || cs.in_stub || cs.cin2 % BK || cs.stride2 < 1 || ((uintptr_t)cs.in2 & 15))
      return cudaErrorInvalidValue;
    if ((cs.h2 - 1) / cs.stride2 + 1 != cs.oh || (cs.w2 - 1) / cs.stride2 + 1 != cs.ow) return cudaErrorInvalidValue;
    p.K += cs.cin2;
    p.num_kb += cs.cin2 / BK;
    p.stride2 = cs.stride2;
  }
  p.panel_kb = p.num_kb;
  p.stride = cs.stride;
  p.pad = cs.pad;
  // Row-tap reuse: 8-pixel-wide patches, so that a step of one image row inside the box is 1024 bytes (one swizzle
  // atom) and the shifted A descriptors stay aligned; the box (ph + r - 1 rows) must fit the 128-row A slot.
  static const int allow_reuse = [] { const char* e = getenv("SPLITRPC_CONV_REUSE"); return e ? atoi(e) : 1; }();
  const bool reuse = allow_reuse && cs.stride == 1 && cs.r >= 2 && cs.r <= 4 && cs.ow >= 14 && cs.oh >= 8;
  int bn;
  if (reuse) {
    p.reuse = 1;
    p.pw = 8;
    p.ph = std::min(cs.oh, 16 - (cs.r - 1));
    p.pn = 1;
    p.num_kb = cs.s * p.cblocks;  // load groups
  } else {
    pick_patch(cs.ow, cs.oh, cs.n, &p.pw, &p.ph, &p.pn);
  }
  p.rows_used = p.pw * p.ph * p.pn;
  p.tiles_w = (cs.ow + p.pw - 1) / p.pw;
  p.tiles_h = (cs.oh + p.ph - 1) / p.ph;
  p.tiles_m = p.tiles_w * p.tiles_h * ((cs.n + p.pn - 1) / p.pn);
  if (reuse) bn = cs.cout <= 64 ? 64 : 128;  // r B tiles travel with every A box: wider tiles leave too few stages
  else bn = pick_bn(cs.cout, p.tiles_m, p.num_kb, true);
  p.tiles_n = (cs.cout + bn - 1) / bn;
  const int box_rows = reuse ? p.ph + cs.r - 1 : p.ph * cs.stride;
  p.a_box_bytes = reuse ? (uint32_t)(box_rows * p.pw) * 128u : (uint32_t)p.rows_used * 128u;
  CUtensorMap ta, tb, to;
  {
    const uint64_t pix = cs.in_pix_stride ? (uint64_t)cs.in_pix_stride : (uint64_t)cs.cin;
    const uint64_t rowst = cs.in_row_stride ? (uint64_t)cs.in_row_stride : (uint64_t)cs.w * pix;
    const uint64_t imgst = cs.in_img_stride ? (uint64_t)cs.in_img_stride : (uint64_t)cs.h * rowst;
    if ((pix % 8) || (rowst % 8) || (imgst % 8)) return cudaErrorInvalidValue;
    if (cs.in_stub && (cs.in_ring_slots < cs.n || !cs.in_slot_bytes || imgst * 2 != cs.in_slot_bytes)) return cudaErrorInvalidValue;
    uint64_t dims[4] = {(uint64_t)cs.cin, (uint64_t)cs.w, (uint64_t)cs.h, (uint64_t)(cs.in_stub ? cs.in_ring_slots : cs.n)};
    uint64_t st[3] = {pix * 2, rowst * 2, imgst * 2};
    p.in_stub = cs.in_stub;
    p.in_ring_base = (unsigned long long)(uintptr_t)in;
    p.in_slot_bytes = cs.in_slot_bytes;
    uint32_t box[4] = {BK, (uint32_t)(p.pw * cs.stride), (uint32_t)box_rows, (uint32_t)p.pn};
    uint32_t es[4] = {1, (uint32_t)cs.stride, (uint32_t)cs.stride, 1};
    if (box[1] > 256 || box[2] > 256) return cudaErrorInvalidValue;
    cudaError_t e = get_map(&ta, in, 4, dims, st, box, es);
    if (e != cudaSuccess) return e;
  }
  CUtensorMap ta2 = ta;
  if (cs.in2) {
    uint64_t dims[4] = {(uint64_t)cs.cin2, (uint64_t)cs.w2, (uint64_t)cs.h2, (uint64_t)cs.n};
    uint64_t st[3] = {(uint64_t)cs.cin2 * 2, (uint64_t)cs.w2 * cs.cin2 * 2, (uint64_t)cs.h2 * cs.w2 * cs.cin2 * 2};
    uint32_t box[4] = {BK, (uint32_t)(p.pw * cs.stride2), (uint32_t)(p.ph * cs.stride2), (uint32_t)p.pn};
    uint32_t es[4] = {1, (uint32_t)cs.stride2, (uint32_t)cs.stride2, 1};
    if (box[1] > 256 || box[2] > 256) return cudaErrorInvalidValue;
    cudaError_t e2 = get_map(&ta2, cs.in2, 4, dims, st, box, es);
    if (e2 != cudaSuccess) return e2;
  }
  cudaError_t e = map_2d(&tb, weight, (uint64_t)p.K, (uint64_t)cs.cout, (uint64_t)p.K * 2, BK, (uint32_t)bn);
  if (e != cudaSuccess) return e;
  {
    uint64_t dims[4] = {(uint64_t)cs.cout, (uint64_t)cs.ow, (uint64_t)cs.oh, (uint64_t)cs.n};
    uint64_t st[3] = {(uint64_t)cs.cout * 2, (uint64_t)cs.ow * cs.cout * 2, (uint64_t)cs.oh * cs.ow * cs.cout * 2};
    uint32_t box[4] = {64, (uint32_t)p.pw, (uint32_t)p.ph, (uint32_t)p.pn};
    uint32_t es[4] = {1, 1, 1, 1};
    e = get_map(&to, ep.out, 4, dims, st, box, es);
    if (e != cudaSuccess) return e;
  }
  GemmEpilogue ep2 = ep;
  ep2.ldo = cs.cout;
  if (ep2.residual) ep2.ldr = cs.cout;
  return dispatch(bn, ta, tb, to, ta2, p, ep2, 1, status, stream);
}
