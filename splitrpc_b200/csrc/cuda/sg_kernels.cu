// Scatter-gather copy kernels for sm_100a.
//
// Replaces the single-block persistent copy loop, the block-per-buffer kernel and
// the device-side memcpy kernel of reference src/transport/g_copy_ng.cu:17-163
// with chunked multi-block kernels:
//   sg_copy_simt     16-byte vector copies, any alignment handled by peeling
//   sg_copy_bulk     one thread per block drives a ring of shared-memory stages
//                    with cp.async.bulk (TMA) loads and stores; other warps take
//                    the chunks that are not 16-byte aligned
//   sg_cast_bf16     gather fused with fp32 -> bf16 deserialisation
//   sg_persistent    doorbell-driven resident variant (host rings a sequence
//                    number in mapped memory; the last block to finish publishes
//                    it back with a system-scope release store)
// All waits are bounded; a wait that runs out sets an error word and the kernel
// returns after draining its own outstanding copies.
#include <mutex>

#include "ptx.cuh"
#include "resp_push.cuh"
#include "sg_kernels.cuh"

namespace {

__device__ __forceinline__ uint32_t find_item(const SgItem* items, uint32_t n, uint32_t chunk) {
  uint32_t lo = 0, hi = n - 1;
  while (lo < hi) {
    uint32_t mid = (lo + hi + 1) >> 1;
    if (items[mid].first_chunk <= chunk) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

struct ChunkRef {
  const uint8_t* src;
  uint8_t* dst;
  uint32_t len;
};

__device__ __forceinline__ ChunkRef chunk_ref(const SgItem* items, uint32_t n_items, uint32_t chunk) {
  uint32_t it = find_item(items, n_items, chunk);
  uint64_t off = (uint64_t)(chunk - items[it].first_chunk) * SG_CHUNK;
  uint32_t left = items[it].len - (uint32_t)off;
  ChunkRef r;
  r.src = reinterpret_cast<const uint8_t*>(items[it].src + off);
  r.dst = reinterpret_cast<uint8_t*>(items[it].dst + off);
  r.len = left < SG_CHUNK ? left : SG_CHUNK;
  return r;
}

// Copies one chunk with `nthr` threads (thread index `t`).
__device__ __forceinline__ void copy_chunk_simt(const uint8_t* src, uint8_t* dst, uint32_t len, uint32_t t, uint32_t nthr) {
  uint32_t head = (uint32_t)((16 - ((uintptr_t)dst & 15)) & 15);
  if (head > len) head = len;
  for (uint32_t i = t; i < head; i += nthr) dst[i] = src[i];
  const uint8_t* s = src + head;
  uint8_t* d = dst + head;
  uint32_t body = len - head;
  if (((uintptr_t)s & 15) == 0) {
    uint32_t nv = body >> 4;
    const uint4* s4 = reinterpret_cast<const uint4*>(s);
    uint4* d4 = reinterpret_cast<uint4*>(d);
    // four independent 16-byte loads in flight per thread: a host-memory source answers after microseconds, and with
    // one load per thread a few blocks cannot keep the PCIe link busy
    uint32_t i = t;
    for (; i + 3 * nthr < nv; i += 4 * nthr) {
      const uint4 a = s4[i], b = s4[i + nthr], c = s4[i + 2 * nthr], e = s4[i + 3 * nthr];
      d4[i] = a;
      d4[i + nthr] = b;
      d4[i + 2 * nthr] = c;
      d4[i + 3 * nthr] = e;
    }
    if (i < nv) {  // fewer than four full rounds left (e.g. one 8 KB fragment): still issue every load before any store
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      const bool p1 = i + nthr < nv, p2 = i + 2 * nthr < nv;
      const uint4 a = s4[i], b = p1 ? s4[i + nthr] : z, c = p2 ? s4[i + 2 * nthr] : z;
      d4[i] = a;
      if (p1) d4[i + nthr] = b;
      if (p2) d4[i + 2 * nthr] = c;
    }
    for (uint32_t i2 = (nv << 4) + t; i2 < body; i2 += nthr) d[i2] = s[i2];
  } else if (((uintptr_t)s & 3) == 0) {
    uint32_t nv = body >> 2;
    const uint32_t* s1 = reinterpret_cast<const uint32_t*>(s);
    uint32_t* d1 = reinterpret_cast<uint32_t*>(d);
    for (uint32_t i = t; i < nv; i += nthr) d1[i] = s1[i];
    for (uint32_t i = (nv << 2) + t; i < body; i += nthr) d[i] = s[i];
  } else {
    for (uint32_t i = t; i < body; i += nthr) d[i] = s[i];
  }
}

// Epilogue shared by the copy kernels: see SgNotify.  Every thread fences its own stores at system scope before the
// block arrives; the block that arrives last has therefore seen (through the counter) that all bytes of the launch are
// visible to the peer GPU or the host, and only then rings the bells.
__device__ __forceinline__ void sg_notify_epilogue(const SgNotify& nt) {
  if (!nt.counter) return;
  __shared__ uint32_t s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(nt.counter, 1u);
    s_last = (prev + 1 == gridDim.x) ? 1u : 0u;
  }
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) atomicExch(nt.counter, 0u);
  __threadfence_system();
  const uint64_t now = nt.stamps_base ? ptx::globaltimer_ns() : 0ull;
  for (uint32_t i = threadIdx.x; i < nt.n_bells; i += blockDim.x) {
    if (nt.stamps_base) {
      const uint64_t slot = (nt.bells[i] - nt.states_base) >> 2;
      *reinterpret_cast<volatile uint64_t*>(nt.stamps_base + 16 * slot) = now;
    }
    ptx::st_release_sys(reinterpret_cast<volatile uint32_t*>(nt.bells[i]), nt.bell_value);
  }
  __syncthreads();
  if (threadIdx.x == 0 && nt.done_word) {
    __threadfence_system();
    ptx::st_release_sys(nt.done_word, nt.done_value);
  }
}

// Groups of 256 threads take chunks in turn.  Launched with 256 threads per block (many blocks: device and peer
// sources) or with 1024 (four groups per block: a few "fat" blocks reach the PCIe rate for host sources and occupy
// only as many SMs).
__global__ void __launch_bounds__(1024) sg_copy_simt(const SgItem* __restrict__ items, uint32_t n_items, uint32_t n_chunks,
                                                     SgNotify notify) {
  const uint32_t groups = blockDim.x >> 8;
  const uint32_t g = blockIdx.x * groups + (threadIdx.x >> 8), ng = gridDim.x * groups;
  for (uint32_t c = g; c < n_chunks; c += ng) {
    ChunkRef r = chunk_ref(items, n_items, c);
    copy_chunk_simt(r.src, r.dst, r.len, threadIdx.x & 255u, 256u);
  }
  sg_notify_epilogue(notify);
}

// One block per response of the batch: copy it from the response ring to where the producer wants it (when that is
// somewhere else) and complete the slot.
__global__ void __launch_bounds__(256) resp_push_kernel(const g_params* __restrict__ stub, const RespPushCtx* __restrict__ ctx) {
  const uint32_t row = blockIdx.x;
  __shared__ uint8_t* s_src;
  __shared__ uint32_t s_len;
  if (threadIdx.x == 0) {  // the stub and the push block are read once per block (host memory)
    s_len = ctx->resp_size;
    s_src = stub->resp + (size_t)row * s_len;
  }
  __syncthreads();
  uint8_t* src = s_src;
  const RespPushTarget t = resp_push_target_block(ctx, row, src);
  if (t.dst != src) copy_chunk_simt(src, t.dst, s_len, threadIdx.x, blockDim.x);
  __syncthreads();
  if (threadIdx.x == 0) resp_push_complete(t);
}

// Rewrites an app's parameter block (stub, push block, transmit offsets of the batch) in the GPU's own memory.  The
// stub and the push block arrive as launch arguments; the offsets either with them or, when the host could not know
// them at launch time (a window armed ahead of its requests), from the per-slot table in host memory, all rows at
// once so that the reads overlap.
struct WindowParams {
  g_params stub;
  RespPushCtx ctx;
  uint8_t* block;
  const volatile uint32_t* live_enabled;
  int n;
  int fetch;
  uint64_t off[APP_PARAM_INLINE_MAX];
};
__global__ void __launch_bounds__(128) window_params_kernel(const __grid_constant__ WindowParams p) {
  uint64_t* win = reinterpret_cast<uint64_t*>(p.block + APP_PARAM_WINDOW_OFFSET);
  uint32_t live = 1;
  if (threadIdx.x == 0 && p.live_enabled) live = *p.live_enabled;
  for (int r = threadIdx.x; r < p.n; r += blockDim.x) {
    uint64_t v = ~0ull;
    if (!p.fetch) v = p.off[r];
    else if (p.ctx.tx_off && p.ctx.pool_size) v = p.ctx.tx_off[(p.ctx.first_slot + (uint32_t)r) % p.ctx.pool_size];
    win[r] = v;
  }
  if (threadIdx.x == 0) {
    RespPushCtx c = p.ctx;
    c.tx_window = p.n > 0 ? win : nullptr;
    if (live == 0) c.enabled = 0;
    *reinterpret_cast<g_params*>(p.block) = p.stub;
    *reinterpret_cast<RespPushCtx*>(p.block + APP_PARAM_PUSH_OFFSET) = c;
  }
}

__device__ __forceinline__ bool bulk_ok(const ChunkRef& r) {
  return ((((uintptr_t)r.src) | ((uintptr_t)r.dst) | (uintptr_t)r.len) & 15) == 0 && r.len > 0;
}

constexpr int BULK_STAGES = 8;
constexpr int BULK_AHEAD = 4;
constexpr int BULK_THREADS = 128;

// Runs the bulk-copy pipeline of one block over chunks {first, first+stride, ...}
// that pass bulk_ok.  Called by one thread.  Returns false if a wait ran out.
__device__ bool bulk_pipeline(const SgItem* items, uint32_t n_items, uint32_t n_chunks, uint32_t first, uint32_t stride,
                              uint8_t* stages, uint64_t* bars, uint32_t& phase_bits) {
  // k counts eligible chunks handled by this block.
  uint32_t load_c = first, store_c = first;  // chunk cursors of the load and the store side
  uint32_t k_load = 0, k_store = 0;
  bool ok = true;
  auto next_eligible = [&](uint32_t c) {
    while (c < n_chunks) {
      ChunkRef r = chunk_ref(items, n_items, c);
      if (bulk_ok(r)) break;
      c += stride;
    }
    return c;
  };
  load_c = next_eligible(load_c);
  store_c = load_c;
  auto issue_load = [&]() {
    ChunkRef r = chunk_ref(items, n_items, load_c);
    uint32_t s = k_load % BULK_STAGES;
    // The store that last used this stage must have finished reading it.
    if (k_load >= BULK_STAGES) ptx::bulk_wait_read<BULK_STAGES - BULK_AHEAD - 1>();
    ptx::mbar_expect_tx(&bars[s], r.len);
    ptx::bulk_g2s(stages + (size_t)s * SG_CHUNK, r.src, r.len, &bars[s]);
    k_load++;
    load_c = next_eligible(load_c + stride);
  };
  for (int i = 0; i < BULK_AHEAD && load_c < n_chunks; i++) issue_load();
  while (store_c < n_chunks) {
    if (load_c < n_chunks) issue_load();
    ChunkRef r = chunk_ref(items, n_items, store_c);
    uint32_t s = k_store % BULK_STAGES;
    if (!ptx::mbar_wait(&bars[s], (phase_bits >> s) & 1u)) {
      ok = false;
      break;
    }
    phase_bits ^= (1u << s);
    ptx::bulk_s2g(r.dst, stages + (size_t)s * SG_CHUNK, r.len);
    ptx::bulk_commit();
    k_store++;
    store_c = next_eligible(store_c + stride);
  }
  ptx::bulk_wait_all<0>();
  return ok;
}

__global__ void __launch_bounds__(BULK_THREADS) sg_copy_bulk(const SgItem* __restrict__ items, uint32_t n_items,
                                                             uint32_t n_chunks, uint32_t* error) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint8_t* stages = smem_raw;
  __shared__ __align__(8) uint64_t bars[BULK_STAGES];
  if (threadIdx.x == 0) {
    for (int i = 0; i < BULK_STAGES; i++) ptx::mbar_init(&bars[i], 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t phase_bits = 0;
    if (!bulk_pipeline(items, n_items, n_chunks, blockIdx.x, gridDim.x, stages, bars, phase_bits) && error) *error = 1;
  } else if (threadIdx.x >= 32) {
    // Warps 1..3 take the chunks the bulk path cannot move.
    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
      ChunkRef r = chunk_ref(items, n_items, c);
      if (!bulk_ok(r)) copy_chunk_simt(r.src, r.dst, r.len, threadIdx.x - 32, BULK_THREADS - 32);
    }
  }
}

__global__ void __launch_bounds__(256) sg_cast_bf16(const SgItem* __restrict__ items, uint32_t n_items, uint32_t n_chunks,
                                                    float scale, float shift) {
  for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
    uint32_t it = find_item(items, n_items, c);
    uint64_t off = (uint64_t)(c - items[it].first_chunk) * SG_CHUNK;  // byte offset in the fp32 source
    uint32_t left = items[it].len - (uint32_t)off;
    uint32_t len = left < SG_CHUNK ? left : SG_CHUNK;
    const float* s = reinterpret_cast<const float*>(items[it].src + off);
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(items[it].dst + off / 2);
    uint32_t n = len >> 2;
    if (((((uintptr_t)s) & 15) | (((uintptr_t)d) & 7)) == 0) {
      uint32_t nv = n >> 2;
      for (uint32_t i = threadIdx.x; i < nv; i += blockDim.x) {
        float4 v = reinterpret_cast<const float4*>(s)[i];
        __nv_bfloat162 a = __floats2bfloat162_rn((v.x - shift) * scale, (v.y - shift) * scale);
        __nv_bfloat162 b = __floats2bfloat162_rn((v.z - shift) * scale, (v.w - shift) * scale);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&a);
        o.y = *reinterpret_cast<uint32_t*>(&b);
        reinterpret_cast<uint2*>(d)[i] = o;
      }
      for (uint32_t i = (nv << 2) + threadIdx.x; i < n; i += blockDim.x) d[i] = __float2bfloat16((s[i] - shift) * scale);
    } else {
      for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) d[i] = __float2bfloat16((s[i] - shift) * scale);
    }
  }
}

// Gather fused with the deserialisation of a ResNet request: the fragments of an fp32 3 x 224 x 224 image are read
// where the NIC put them and written, normalised and cast to bf16, in the space-to-depth layout that the stem
// convolution reads through TMA (see stem_s2d in nn_kernels.cu for the layout).  The copy list is the ordinary one:
// an item's destination address says which ring slot and which byte offset of the request the bytes belong to, so
// fragments may arrive split and in any order.  The slot then holds the [115][115][16] bf16 tensor (423,200 bytes,
// less than the 602,112-byte request it replaces); border pixels and padding channels are never written and keep
// the zeros the ring was created with.
__global__ void __launch_bounds__(1024) sg_stem_s2d(const SgItem* __restrict__ items, uint32_t n_items, uint32_t n_chunks,
                                                    SgStemS2d tr, SgNotify notify) {
  const uint32_t groups = blockDim.x >> 8;
  const uint32_t g = blockIdx.x * groups + (threadIdx.x >> 8), ng = gridDim.x * groups;
  const uint32_t t = threadIdx.x & 255u;
  for (uint32_t c = g; c < n_chunks; c += ng) {
    const uint32_t it = find_item(items, n_items, c);
    const uint64_t off = (uint64_t)(c - items[it].first_chunk) * SG_CHUNK;
    const uint32_t left = items[it].len - (uint32_t)off;
    const uint32_t len = left < SG_CHUNK ? left : SG_CHUNK;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(items[it].src + off);
    const uint64_t rel = items[it].dst + off - tr.ring_base;
    const uint64_t slot = rel / tr.slot_bytes;
    const uint32_t req_off = (uint32_t)(rel - slot * tr.slot_bytes);
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(tr.ring_base + slot * tr.slot_bytes);
    if ((req_off | len | (uint32_t)(uintptr_t)src) & 3u) continue;  // requests are whole floats
    const uint32_t e0 = req_off >> 2, n = len >> 2;
    auto put = [&](uint32_t e, float v) {
      if (e >= 3u * 224u * 224u) return;
      const uint32_t ch = e / 50176u, rem = e - ch * 50176u;
      const uint32_t iy = rem / 224u, ix = rem - iy * 224u;
      const uint32_t py = iy + 3u, px = ix + 3u;
      const float m = ch == 0 ? tr.mean[0] : (ch == 1 ? tr.mean[1] : tr.mean[2]);
      const float s = ch == 0 ? tr.inv_std[0] : (ch == 1 ? tr.inv_std[1] : tr.inv_std[2]);
      out[((py >> 1) * 115u + (px >> 1)) * 16u + (py & 1u) * 8u + (px & 1u) * 3u + ch] = __float2bfloat16((v - m) * s);
    };
    if ((((uintptr_t)src) & 15) == 0) {
      const uint32_t nv = n >> 2;
      const float4* s4 = reinterpret_cast<const float4*>(src);
      uint32_t i = t;
      for (; i + 3 * 256 < nv; i += 4 * 256) {  // four loads in flight per thread, as in the plain copy
        const float4 a = s4[i], b = s4[i + 256], d = s4[i + 512], f = s4[i + 768];
        const float4 q[4] = {a, b, d, f};
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const uint32_t e = e0 + 4u * (i + 256u * k);
          put(e, q[k].x);
          put(e + 1, q[k].y);
          put(e + 2, q[k].z);
          put(e + 3, q[k].w);
        }
      }
      for (; i < nv; i += 256) {
        const float4 a = s4[i];
        const uint32_t e = e0 + 4u * i;
        put(e, a.x);
        put(e + 1, a.y);
        put(e + 2, a.z);
        put(e + 3, a.w);
      }
      for (uint32_t j = (nv << 2) + t; j < n; j += 256) put(e0 + j, reinterpret_cast<const float*>(src)[j]);
    } else {
      for (uint32_t j = t; j < n; j += 256) put(e0 + j, reinterpret_cast<const float*>(src)[j]);
    }
  }
  sg_notify_epilogue(notify);
}

// Resident engine.  Each block polls the control block; a doorbell ahead of the block's own sequence number (compared
// as a signed difference, so a block can never mistake an older or equal value for new work) means the item list is
// valid.  The exit flag and the idle limit are looked at on every poll, before the doorbell, so a block always leaves
// within one poll of being asked to, whatever the doorbell says.  Blocks never wait for one another: each finishes its
// share, and the block that brings the arrival counter to gridDim.x publishes `done`.
__global__ void __launch_bounds__(256) sg_persistent(SgCtrl* ctrl, uint32_t* counter) {
  __shared__ uint32_t s_cmd, s_seq;
  __shared__ SgItem s_items[SG_PERSISTENT_ITEMS];
  uint32_t seen = ctrl->done;  // submissions up to `done` were served by an earlier launch
  uint64_t last = ptx::globaltimer_ns();
  const uint64_t idle_limit = ctrl->idle_limit_ns;
  for (;;) {
    if (threadIdx.x == 0) {
      uint32_t cmd = 0;  // 0 keep polling, 1 work, 2 leave
      for (int spin = 0; spin < 4096; spin++) {
        if (ptx::ld_relaxed_sys(&ctrl->exit_flag) || ptx::globaltimer_ns() - last > idle_limit) {
          cmd = 2;
          break;
        }
        const uint32_t db = ptx::ld_acquire_sys(&ctrl->doorbell);
        if ((int32_t)(db - seen) > 0) {
          s_seq = db;
          cmd = 1;
          break;
        }
        __nanosleep(200);
      }
      s_cmd = cmd;
    }
    __syncthreads();
    const uint32_t cmd = s_cmd, seq = s_seq;
    __syncthreads();
    if (cmd == 2) break;
    if (cmd == 0) continue;
    seen = seq;
    uint32_t n_items = ctrl->n_items, n_chunks = ctrl->n_chunks;
    if (n_items > SG_PERSISTENT_ITEMS) n_items = SG_PERSISTENT_ITEMS;
    // One pass over PCIe brings the list into shared memory; lookups stay on chip.
    {
      const uint64_t* src = reinterpret_cast<const uint64_t*>(const_cast<const SgItem*>(ctrl->items));
      uint64_t* dst = reinterpret_cast<uint64_t*>(s_items);
      for (uint32_t i = threadIdx.x; i < n_items * 3; i += blockDim.x) dst[i] = ptx::ld_relaxed_sys_u64(src + i);
    }
    __syncthreads();
    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
      ChunkRef r = chunk_ref(s_items, n_items, c);
      copy_chunk_simt(r.src, r.dst, r.len, threadIdx.x, blockDim.x);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t prev = atomicAdd(counter, 1u);
      if (prev + 1 == gridDim.x) {
        atomicExch(counter, 0u);
        __threadfence_system();
        ptx::st_release_sys(&ctrl->done, seen);
      }
      last = ptx::globaltimer_ns();
    }
  }
  if (threadIdx.x == 0) atomicAdd_system(const_cast<uint32_t*>(&ctrl->exited), 1u);
}

}  // namespace

// The copy kernels run beside the model's kernels, whose blocks need (almost) all of an SM's shared memory.  An SM
// keeps its L1 / shared-memory split while any block is resident, so a copy block that was placed on an SM set up
// for a large L1 keeps the big-tile kernels off that SM until it leaves.  Asking for the largest shared-memory
// carve-out (the copies stream and gain nothing from L1) lets both kinds of block share an SM.
template <typename K>
static void prefer_max_shared(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}
// Function attributes belong to a device: the set-up runs once per device (the engines of a multi-GPU server live in
// one process and launch from several threads).  Returns the error of the shared-memory opt-in of the bulk kernel.
static constexpr int kMaxDevices = 64;
static cudaError_t sg_kernel_setup() {
  static std::once_flag once[kMaxDevices];
  static cudaError_t result[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::call_once(once[dev], [dev] {
    // Load every kernel of this file now.  With lazy module loading a kernel is loaded at its first launch, and that
    // load can wait for the device to go idle; a work stream that is already parked on a doorbell (stream-armed mode)
    // never goes idle until the very gather that is trying to launch has run, so the first launch would deadlock.
    cudaFuncAttributes fa;
    (void)cudaFuncGetAttributes(&fa, sg_copy_simt);
    (void)cudaFuncGetAttributes(&fa, sg_copy_bulk);
    (void)cudaFuncGetAttributes(&fa, sg_cast_bf16);
    (void)cudaFuncGetAttributes(&fa, sg_stem_s2d);
    (void)cudaFuncGetAttributes(&fa, sg_persistent);
    (void)cudaFuncGetAttributes(&fa, resp_push_kernel);
    (void)cudaFuncGetAttributes(&fa, window_params_kernel);
    static const int on = [] { const char* e = getenv("P2P_RPC_SG_MAX_SHARED"); return e ? atoi(e) : 1; }();
    if (on) {
      prefer_max_shared(sg_copy_simt);
      prefer_max_shared(sg_cast_bf16);
      prefer_max_shared(sg_persistent);
      prefer_max_shared(sg_stem_s2d);
    }
    (void)cudaGetLastError();
    result[dev] = cudaFuncSetAttribute(sg_copy_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((size_t)BULK_STAGES * SG_CHUNK));
  });
  return result[dev];
}

static int clamp_blocks(int n_blocks, uint32_t n_chunks) {
  if (n_blocks <= 0) n_blocks = 148 * 4;
  if ((uint32_t)n_blocks > n_chunks) n_blocks = (int)n_chunks;
  return n_blocks < 1 ? 1 : n_blocks;
}

cudaError_t sg_launch_copy(const SgItem* d_items, uint32_t n_items, uint32_t n_chunks, int impl, int n_blocks,
                           cudaStream_t stream, const SgNotify* notify) {
  if (n_items == 0 || n_chunks == 0) return cudaSuccess;
  const cudaError_t bulk_attr = sg_kernel_setup();
  const SgNotify nt = notify ? *notify : SgNotify{};
  if (impl == SG_IMPL_BULK && nt.counter) return cudaErrorNotSupported;  // the bulk pipeline has no doorbell epilogue
  if (impl == SG_IMPL_BULK) {
    if (bulk_attr != cudaSuccess) return bulk_attr;
    size_t smem = (size_t)BULK_STAGES * SG_CHUNK;
    int nb = clamp_blocks(n_blocks > 0 ? n_blocks : 148, n_chunks);
    sg_copy_bulk<<<nb, BULK_THREADS, smem, stream>>>(d_items, n_items, n_chunks, nullptr);
  } else if (n_blocks < 0) {  // -n "fat" blocks of 1024 threads
    const uint32_t want = (uint32_t)(-n_blocks), most = (n_chunks + 3) / 4;
    sg_copy_simt<<<want < most ? want : most, 1024, 0, stream>>>(d_items, n_items, n_chunks, nt);
  } else {
    sg_copy_simt<<<clamp_blocks(n_blocks, n_chunks), 256, 0, stream>>>(d_items, n_items, n_chunks, nt);
  }
  return cudaGetLastError();
}

void sg_preload_kernels() { (void)sg_kernel_setup(); }

cudaError_t sg_launch_resp_push(const void* d_stub, const void* d_push, int n, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  sg_kernel_setup();
  resp_push_kernel<<<n, 256, 0, stream>>>((const g_params*)d_stub, (const RespPushCtx*)d_push);
  return cudaGetLastError();
}

cudaError_t sg_launch_window_params(void* block, const g_params* stub, const RespPushCtx* ctx, const uint64_t* offsets, int n,
                                    const uint32_t* live_enabled, cudaStream_t stream) {
  if (!block || !stub || !ctx || n < 0) return cudaErrorInvalidValue;
  if (offsets ? n > APP_PARAM_INLINE_MAX : n > APP_PARAM_WINDOW_MAX) return cudaErrorInvalidValue;
  sg_kernel_setup();
  WindowParams p;
  p.stub = *stub;
  p.ctx = *ctx;
  p.block = (uint8_t*)block;
  p.live_enabled = live_enabled;
  p.n = n;
  p.fetch = offsets ? 0 : 1;
  if (offsets)
    for (int i = 0; i < n; i++) p.off[i] = offsets[i];
  window_params_kernel<<<1, 128, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t sg_launch_cast_bf16(const SgItem* d_items, uint32_t n_items, uint32_t n_chunks, float scale, float shift,
                                int n_blocks, cudaStream_t stream) {
  if (n_items == 0 || n_chunks == 0) return cudaSuccess;
  sg_kernel_setup();
  sg_cast_bf16<<<clamp_blocks(n_blocks, n_chunks), 256, 0, stream>>>(d_items, n_items, n_chunks, scale, shift);
  return cudaGetLastError();
}

cudaError_t sg_launch_stem_s2d(const SgItem* d_items, uint32_t n_items, uint32_t n_chunks, const SgStemS2d& tr, int n_blocks,
                               cudaStream_t stream, const SgNotify* notify) {
  if (n_items == 0 || n_chunks == 0) return cudaSuccess;
  if (!tr.ring_base || !tr.slot_bytes || (tr.slot_bytes & 15u)) return cudaErrorInvalidValue;
  const SgNotify nt = notify ? *notify : SgNotify{};
  sg_kernel_setup();
  if (n_blocks < 0) {
    const uint32_t want = (uint32_t)(-n_blocks), most = (n_chunks + 3) / 4;
    sg_stem_s2d<<<want < most ? want : most, 1024, 0, stream>>>(d_items, n_items, n_chunks, tr, nt);
  } else {
    sg_stem_s2d<<<clamp_blocks(n_blocks, n_chunks), 256, 0, stream>>>(d_items, n_items, n_chunks, tr, nt);
  }
  return cudaGetLastError();
}

cudaError_t sg_launch_persistent(SgCtrl* d_ctrl, uint32_t* d_counter, int n_blocks, cudaStream_t stream) {
  sg_kernel_setup();
  sg_persistent<<<n_blocks, 256, 0, stream>>>(d_ctrl, d_counter);
  return cudaGetLastError();
}
