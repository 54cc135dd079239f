// Device-side pieces shared by the tensor-parallel kernels: bounded flag waits and the copier role that pulls
// remote row blocks into the local gathered buffer.
#pragma once

#include "gemm_tp.h"
#include "ptx.cuh"

namespace tpdev {

// Upper bound of every flag wait, in nanoseconds.  A run-time value (srpc_tp_set_wait_ns) so that a test can let a wait
// run out within milliseconds; the default is two seconds.  Every translation unit that includes this header has its
// own copy of the word and sets it through set_wait_ns_here().
static __device__ uint64_t g_flag_wait_ns = 2000000000ull;
#define FLAG_WAIT_NS (tpdev::g_flag_wait_ns)
static inline cudaError_t set_wait_ns_here(uint64_t ns) { return cudaMemcpyToSymbol(g_flag_wait_ns, &ns, sizeof(ns)); }

// Bounded wait until *flag >= epoch (flags only ever grow).
__device__ __forceinline__ bool wait_flag_gpu(const uint32_t* flag, uint32_t epoch) {
  for (int i = 0; i < 64; i++)  // fast path: no timer read when the flag is (almost) there
    if ((int32_t)(ptx::ld_acquire_gpu(flag) - epoch) >= 0) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 32; i++) {
      if ((int32_t)(ptx::ld_acquire_gpu(flag) - epoch) >= 0) return true;
      __nanosleep(100);
    }
    if (ptx::globaltimer_ns() - t0 > FLAG_WAIT_NS) return false;
  }
}
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t epoch) {
  for (int i = 0; i < 16; i++)
    if ((int32_t)(ptx::ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 32; i++) {
      if ((int32_t)(ptx::ld_acquire_sys(flag) - epoch) >= 0) return true;
      __nanosleep(200);
    }
    if (ptx::globaltimer_ns() - t0 > FLAG_WAIT_NS) return false;
  }
}

// Copier role: pulls remote row blocks into the local gathered buffer.  One thread per copier block drives a ring of
// 16 KB bulk copies (peer memory -> shared memory -> local memory; no multicast): COPY_AHEAD loads are in flight per
// block, so a handful of blocks keep a few MB on the wire, which is what NVLink's latency needs to run at link rate.
// (Plain 16-byte loads from 320 threads kept 20 KB per block in flight and reached about 100 GB/s.)
constexpr int COPY_CHUNK = 16384;
constexpr int COPY_SLOTS = 12;
constexpr int COPY_AHEAD = 10;

__device__ __forceinline__ void copier(const TpParams& tp, int copier_idx, uint8_t* ring, uint32_t* status) {
  __shared__ __align__(8) uint64_t cbar[COPY_SLOTS];
  if (threadIdx.x != 0) return;
  for (int s = 0; s < COPY_SLOTS; s++) ptx::mbar_init(&cbar[s], 1);
  ptx::fence_mbar_init();
  const int remote_blocks = (tp.tp - 1) * tp.mblocks_per_rank;
  const int my_blocks = copier_idx < remote_blocks ? (remote_blocks - copier_idx + tp.n_copy - 1) / tp.n_copy : 0;
  const uint32_t cpb = (uint32_t)((tp.mblock_bytes + COPY_CHUNK - 1) / COPY_CHUNK);  // chunks per row block
  const uint32_t total = (uint32_t)my_blocks * cpb;
  struct Chunk {
    const uint8_t* src;
    uint8_t* dst;
    uint32_t len;
    int r, m;
    bool first, last;
  };
  auto chunk_at = [&](uint32_t q) {
    Chunk c;
    const int i = copier_idx + (int)(q / cpb) * tp.n_copy;  // i-th remote block in rotated order: ranks rank+1, rank+2, ...
    const uint32_t k = q % cpb;
    c.r = (tp.rank + i / tp.mblocks_per_rank + 1) % tp.tp;
    const int blk = i % tp.mblocks_per_rank;
    c.m = c.r * tp.mblocks_per_rank + blk;
    const size_t off = (size_t)k * COPY_CHUNK;
    c.src = tp.src[c.r] + (size_t)blk * tp.mblock_bytes + off;
    c.dst = tp.gathered + (size_t)c.m * tp.mblock_bytes + off;
    const size_t left = tp.mblock_bytes - off;
    c.len = (uint32_t)(left < (size_t)COPY_CHUNK ? left : (size_t)COPY_CHUNK);
    c.first = k == 0;
    c.last = k + 1 == cpb;
    return c;
  };
  uint32_t q_load = 0, phase_bits = 0;
  bool ok = true;
  auto issue_load = [&]() {
    const Chunk c = chunk_at(q_load);
    if (c.first && !wait_flag_sys(tp.src_ready + c.r, tp.epoch)) {
      if (status) atomicExch(status, GEMM_ERR_TP_SRC_WAIT);
      return false;
    }
    const uint32_t s = q_load % COPY_SLOTS;
    // The store that last used this slot must have finished reading it.
    if (q_load >= COPY_SLOTS) ptx::bulk_wait_read<COPY_SLOTS - COPY_AHEAD - 1>();
    ptx::mbar_expect_tx(&cbar[s], c.len);
    ptx::bulk_g2s(ring + (size_t)s * COPY_CHUNK, c.src, c.len, &cbar[s]);
    q_load++;
    return true;
  };
  for (int i = 0; i < COPY_AHEAD && q_load < total && ok; i++) ok = issue_load();
  for (uint32_t q = 0; q < total && ok; q++) {
    if (q_load < total) ok = issue_load();
    if (!ok) break;
    const Chunk c = chunk_at(q);
    const uint32_t s = q % COPY_SLOTS;
    if (!ptx::mbar_wait(&cbar[s], (phase_bits >> s) & 1u)) {
      if (status) atomicExch(status, GEMM_ERR_TP_BLOCK_WAIT);
      ok = false;
      break;
    }
    phase_bits ^= (1u << s);
    ptx::bulk_s2g(c.dst, ring + (size_t)s * COPY_CHUNK, c.len);
    ptx::bulk_commit();
    if (c.last) {
      // Whole row block written: make the bulk stores visible, then publish the block to the GEMM blocks.
      ptx::bulk_wait_all<0>();
      ptx::fence_proxy_async_all();
      __threadfence();
      ptx::st_release_gpu(tp.mblock_ready + c.m, tp.epoch);
    }
  }
  ptx::bulk_wait_all<0>();
  if (!ok) __nanosleep(1000000);  // let loads that are still in flight land before the block leaves
}


}  // namespace tpdev
