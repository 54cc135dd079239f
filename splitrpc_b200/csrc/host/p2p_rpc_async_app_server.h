// App registry and worker loops over the request-slot ring.
//
// Public surface follows reference src/p2p_rpc_async_app_server.h:14-361:
// P2pRpcAppInfo bundles an app's four callbacks with its slot pool and execution
// context; P2pRpcAsyncAppServer runs one of three consumer loops over the slots:
//   sync_worker_loop                    fixed batch size, run + wait per batch
//   dynamic_batching_sync_worker_loop   greedy: as many consecutive RX_COMPLETE
//                                       slots as are ready, up to a maximum
//   async_worker_loop                   the work stream is armed ahead of time
//                                       with wait(slot state) -> app -> write(doorbell);
//                                       the host only reaps finished batches
// Differences from the original: every wait is bounded and reported, batch-size
// changes are atomic, loops can be stopped after a request budget (for tests and
// benchmarks), and batch-size statistics are kept instead of printed.
#pragma once

#include <atomic>
#include <map>
#include <memory>
#include <mutex>

#include "p2p_rpc_app.h"

#define APP_RR_POOL_SIZE 4096

class P2pRpcAppInfo {
 public:
  int appIdx = -1;
  AppCtx* app_ctx = nullptr;
  int device_id;
  AppInitCB app_init;
  AppRunCB app_run;
  AppCleanupCB app_cleanup;
  AppCompleteCB app_complete;
  P2pRpcAppRrPool* app_rr_pool = nullptr;
  uint16_t rr_pool_size;
  size_t req_size, resp_size;
  g_params* h_stubs = nullptr;
  g_params* d_stubs = nullptr;
  uint32_t* door_bells = nullptr;
  uint32_t* d_door_bells = nullptr;
  bool init_ok = false;
  uint64_t consumer_seq = 0;  // slots consumed by the worker since the pool was initialised
  // The slots are filled by a producer that does not bind them through this pool's get_next() (another process that
  // mirrors the rings): window addresses then come from the ring arithmetic, not from the slots' stubs.
  bool use_window_stub = false;
  // The serving side stores every response where the producer asked for it and marks the slot WORK_COMPLETE itself
  // (from the app's last kernel, a push kernel behind it, or the CPU app's thread); the worker loops then leave the
  // slot states alone.  See RespPushCtx.
  bool completion_by_device = false;

  // `internal` is stored in app_ctx->app_ctx_internal before app_init runs, so a
  // callback set can be shared by several instances with different state.
  P2pRpcAppInfo(AppInitCB _init, AppRunCB _run, AppCleanupCB _cleanup, AppCompleteCB _complete, int _device_id,
                size_t _req_size, size_t _resp_size, int _pool_size = APP_RR_POOL_SIZE, void* internal = nullptr,
                int launch_type = -1, int batch_size = -1)
      : device_id(_device_id),
        app_init(_init),
        app_run(_run),
        app_cleanup(_cleanup),
        app_complete(_complete),
        rr_pool_size((uint16_t)_pool_size),
        req_size(_req_size),
        resp_size(_resp_size) {
    app_rr_pool = new P2pRpcAppRrPool(_pool_size, device_id, req_size, resp_size);
    app_ctx = new AppCtx;
    app_ctx->curr_batch_size = batch_size > 0 ? batch_size : get_ort_batch_size();
    app_ctx->next_batch_size = app_ctx->curr_batch_size;
    app_ctx->device_id = device_id;
    app_ctx->launch_type = (uint8_t)(launch_type >= 0 ? launch_type : get_work_launch_type());
    app_ctx->app_ctx_internal = internal;
    if (device_id >= 0) {
      const SrpcDeviceOps* ops = srpc_require_cuda("P2pRpcAppInfo");
      ops->stream_create(device_id, &app_ctx->work_stream);
      ops->event_create(&app_ctx->work_complete);
      // One allocation holds the stub and the doorbell; both are read by kernels
      // (indirect stub, persistent doorbell) and written by the host.
      // One allocation: stub at 0, doorbell at 128, response-push block at 256.
      void *h = nullptr, *d = nullptr;
      ops->host_alloc_mapped(512, &h, &d);
      h_stubs = (g_params*)h;
      d_stubs = (g_params*)d;
      door_bells = (uint32_t*)((uint8_t*)h + 128);
      d_door_bells = (uint32_t*)((uint8_t*)d + 128);
      app_ctx->h_push = (RespPushCtx*)((uint8_t*)h + 256);
      app_ctx->d_push = (RespPushCtx*)((uint8_t*)d + 256);
      // What kernels read: a copy of both in the GPU's own memory, rewritten by stage_window() before every batch.
      void* blk = nullptr;
      if (ops->window_params && ops->dev_alloc(device_id, APP_PARAM_BLOCK_BYTES, &blk) == 0 && blk) {
        ops->memset_async(blk, 0, APP_PARAM_BLOCK_BYTES, app_ctx->work_stream);
        ops->stream_sync(app_ctx->work_stream);
        app_ctx->param_block = (uint8_t*)blk;
      }
    } else {
      void* p = nullptr;
      if (posix_memalign(&p, 64, 512) != 0) std::abort();
      std::memset(p, 0, 512);
      h_stubs = d_stubs = (g_params*)p;
      door_bells = d_door_bells = (uint32_t*)((uint8_t*)p + 128);
      app_ctx->h_push = app_ctx->d_push = (RespPushCtx*)((uint8_t*)p + 256);
    }
    std::memset(app_ctx->h_push, 0, sizeof(RespPushCtx));
    app_ctx->h_stub = h_stubs;
    app_ctx->d_stub = app_ctx->d_stub_mapped = d_stubs;
    app_ctx->d_push_mapped = app_ctx->d_push;
    if (app_ctx->param_block) {
      app_ctx->d_stub = (g_params*)app_ctx->param_block;
      app_ctx->d_push = (RespPushCtx*)(app_ctx->param_block + APP_PARAM_PUSH_OFFSET);
    }
    app_ctx->door_bell = door_bells;
    app_ctx->d_door_bell = d_door_bells;
    app_ctx->h_stub->req = nullptr;
    app_ctx->h_stub->resp = nullptr;
    app_ctx->ResetAppRunStatus();
    init_ok = app_init ? (app_init(app_ctx) != 0) : true;
    if (!init_ok) srpc_log(SRPC_LOG_WARN, "app_init reported failure");
  }

  ~P2pRpcAppInfo() {
    if (app_cleanup) app_cleanup(app_ctx);
    if (device_id >= 0) {
      if (const SrpcDeviceOps* ops = srpc_cuda_ops()) {
        ops->stream_sync(app_ctx->work_stream);
        ops->stream_destroy(app_ctx->work_stream);
        ops->event_destroy(app_ctx->work_complete);
        if (app_ctx->param_block) ops->dev_free(app_ctx->param_block);
        ops->host_free(h_stubs);
      }
    } else {
      free(h_stubs);
    }
    delete app_ctx;
    delete app_rr_pool;
  }
  P2pRpcAppInfo(const P2pRpcAppInfo&) = delete;

  // Turns on completion by the serving side.  tx_base / tx_bytes describe the producer's transmit arena as THIS
  // process addresses it from the app's device (a device-side address on a GPU, a host address on the CPU device);
  // tx_base == 0 keeps responses in the response ring and only moves the state store to the serving side.
  void enable_device_completion(uint64_t tx_base, uint64_t tx_bytes) {
    RespPushCtx* p = app_ctx->h_push;
    P2pRpcAppRrMemPool* mp = app_rr_pool->rr_mem_pool;
    p->tx_base = tx_base;
    p->tx_bytes = tx_base ? tx_bytes : 0;
    p->tx_off = mp->get_tx_offsets_device();
    p->states = mp->get_doorbells_device();
    p->stamps = mp->get_stamps_device();
    p->pool_size = (uint32_t)rr_pool_size;
    p->resp_size = (uint32_t)resp_size;
    p->first_slot = 0;
    p->tx_window = nullptr;
    std::atomic_thread_fence(std::memory_order_release);
    p->enabled = 1;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    completion_by_device = true;
    stage_window(0, 0, false);
  }
  void disable_device_completion() {
    completion_by_device = false;
    app_ctx->h_push->enabled = 0;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    stage_window(0, 0, false);
  }

  // Makes the kernels of the next batch see the current stub and push block: on a GPU, queues the kernel that
  // rewrites the parameter block in the GPU's memory (in stream order, so batches already queued keep theirs).
  // `batch` requests starting at slot `first_slot`; their transmit offsets travel with the launch when the slots are
  // already filled (`armed` false), otherwise the kernel reads them from the slot table when it runs, which is after
  // the doorbell wait that the caller has queued before it.
  void stage_window(int first_slot, int batch, bool armed) {
    AppCtx* c = app_ctx;
    if (device_id < 0 || !c->param_block || c->launch_type == 3) return;  // resident kernels poll the mapped copies
    const SrpcDeviceOps* ops = srpc_require_cuda("parameter block");
    ops->set_device(device_id);  // callers include threads that never touched this GPU (a control-socket thread)
    RespPushCtx ctx = *c->h_push;
    ctx.first_slot = (uint32_t)first_slot;
    uint64_t offs[APP_PARAM_INLINE_MAX];
    const uint64_t* inline_offs = nullptr;
    int n = (completion_by_device && ctx.enabled) ? batch : 0;
    if (n > APP_PARAM_WINDOW_MAX) n = 0;  // kernels fall back to the slot table
    if (n > 0 && !armed && n <= APP_PARAM_INLINE_MAX) {
      for (int r = 0; r < n; r++)
        offs[r] = __atomic_load_n(app_rr_pool->get_app_rr((first_slot + r) % rr_pool_size)->h_tx_off, __ATOMIC_ACQUIRE);
      inline_offs = offs;
    }
    const uint32_t* live = armed ? &c->d_push_mapped->enabled : nullptr;
    if (ops->window_params(c->param_block, c->h_stub, &ctx, inline_offs, n, live, c->work_stream) != 0)
      srpc_log(SRPC_LOG_ERROR, "parameter block update failed: %s", ops->last_error());
  }

  // Stores the responses of the batch that just ran (app_ctx->curr_batch_size requests from slot h_push->first_slot on)
  // and completes their slots, unless the app's own kernels do that.  On a GPU this queues one kernel behind the app
  // on the work stream; on the CPU device it copies here.
  void push_responses() {
    if (!completion_by_device || app_ctx->self_push) return;
    RespPushCtx* p = app_ctx->h_push;
    const int n = app_ctx->curr_batch_size;
    if (device_id >= 0) {
      const SrpcDeviceOps* ops = srpc_require_cuda("response push");
      if (ops->resp_push(app_ctx->d_stub, app_ctx->d_push, n, app_ctx->work_stream) != 0)
        srpc_log(SRPC_LOG_ERROR, "response push failed: %s", ops->last_error());
      return;
    }
    for (int r = 0; r < n; r++) {
      uint32_t slot = (p->first_slot + (uint32_t)r) % p->pool_size;
      uint64_t off = p->tx_off[slot];
      if (p->tx_base && off != P2pRpcAppRrMemPool::kNoTxOffset && off + p->resp_size <= p->tx_bytes)
        std::memcpy((void*)(uintptr_t)(p->tx_base + off), app_ctx->h_stub->resp + (size_t)r * p->resp_size, p->resp_size);
      p->stamps[2 * slot + 1] = getCurNs();
      __atomic_store_n(&p->states[slot], (uint32_t)APP_RR_STATUS::WORK_COMPLETE, __ATOMIC_RELEASE);
    }
  }
};

struct WorkerStats {
  uint64_t num_req = 0, num_batches = 0, wait_timeouts = 0;
  std::map<int, uint64_t> batch_hist;
  std::vector<uint64_t> work_ns;  // per-batch host-observed run time (bounded sample)
};

class P2pRpcAsyncAppServer {
  std::vector<P2pRpcAppInfo*> all_apps;
  std::atomic<uint64_t> num_req{0};
  std::atomic<int32_t> force_quit_server{0};
  std::mutex stats_mu_;
  std::vector<WorkerStats> stats_;
  uint64_t stop_after_ = 0;  // 0 = run until quit()

  static uint32_t load_state(volatile uint32_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
  static void store_state(volatile uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
  bool should_stop() const {
    if (force_quit_server.load(std::memory_order_acquire)) return true;
    return stop_after_ && num_req.load(std::memory_order_relaxed) >= stop_after_;
  }
  void note_batch(int appIdx, int bs, uint64_t ns) {
    WorkerStats& s = stats_[appIdx];
    s.num_req += bs;
    s.num_batches++;
    s.batch_hist[bs]++;
    if (s.work_ns.size() < (1u << 20)) s.work_ns.push_back(ns);
  }

 public:
  P2pRpcAsyncAppServer() = default;

  void quit() { force_quit_server.store(1, std::memory_order_release); }
  void reset_quit() { force_quit_server.store(0, std::memory_order_release); }
  bool quitting() const { return force_quit_server.load(std::memory_order_acquire) != 0; }
  // Makes the worker loops return once this many requests have been served.
  void stop_after(uint64_t n) { stop_after_ = n; }
  uint64_t served() const { return num_req.load(); }
  WorkerStats stats(int appIdx) {
    std::lock_guard<std::mutex> g(stats_mu_);
    return stats_[appIdx];
  }

  int register_app(P2pRpcAppInfo* app) {
    std::lock_guard<std::mutex> g(stats_mu_);
    all_apps.push_back(app);
    stats_.emplace_back();
    app->appIdx = (int)all_apps.size() - 1;
    return app->appIdx;
  }
  P2pRpcAppInfo* get_app(int appIdx) { return all_apps[appIdx]; }
  size_t num_apps() const { return all_apps.size(); }

  // Applies a batch size requested through app_ctx->next_batch_size.  Only the
  // consumer loop calls this, between batches.
  void update_batch_size(int appIdx) {
    AppCtx* c = all_apps[appIdx]->app_ctx;
    c->curr_batch_size = __atomic_load_n(&c->next_batch_size, __ATOMIC_ACQUIRE);
  }
  void request_batch_size(int appIdx, int bs) {
    __atomic_store_n(&all_apps[appIdx]->app_ctx->next_batch_size, bs, __ATOMIC_RELEASE);
  }

  // Points the app's stub at slot rr_idx and starts the app; does not wait.
  void do_work(int appIdx, int rr_idx) {
    P2pRpcAppInfo* a = all_apps[appIdx];
    *a->app_ctx->h_stub = a->use_window_stub ? a->app_rr_pool->window_stub(a->consumer_seq)
                                             : *a->app_rr_pool->get_app_rr(rr_idx)->h_stub;
    a->app_ctx->h_push->first_slot = (uint32_t)rr_idx;
    std::atomic_thread_fence(std::memory_order_release);
    NVTX_R("AppRun");
    a->stage_window(rr_idx, a->app_ctx->curr_batch_size, false);
    a->app_run(a->app_ctx);
    a->push_responses();
    NVTX_P();
  }
  bool do_sync(int appIdx) {
    P2pRpcAppInfo* a = all_apps[appIdx];
    bool ok = a->app_ctx->WaitForAppRunComplete();
    if (a->app_complete) a->app_complete(a->app_ctx);
    return ok;
  }
  // Runs slot rr_idx (and the curr_batch_size-1 slots after it) to completion
  // without checking that the slots are ready.
  bool do_work_sync(int appIdx, int rr_idx) {
    do_work(appIdx, rr_idx);
    return do_sync(appIdx);
  }
  bool do_batch_work_sync(int appIdx, int start_rr_idx, int batch_size) {
    all_apps[appIdx]->app_ctx->curr_batch_size = batch_size;
    return do_work_sync(appIdx, start_rr_idx);
  }

  void sync_worker_loop(int appIdx) {
    P2pRpcAppInfo* a = all_apps[appIdx];
    P2pRpcAppRrPool* pool = a->app_rr_pool;
    const int n = a->rr_pool_size;
    int ci = 0, si = 0, win = 0;
    a->consumer_seq = 0;
    IdleBackoff backoff;
    while (!should_stop()) {
      if (load_state(pool->get_app_rr(ci)->h_state) != APP_RR_STATUS::RX_COMPLETE) {
        backoff.empty();
        continue;
      }
      backoff.busy();
      ci = (ci + 1) % n;
      if (++win < a->app_ctx->curr_batch_size) continue;
      uint64_t t0 = getCurNs();
      bool ok = do_work_sync(appIdx, si);
      if (!a->completion_by_device)
        for (int i = si; i != ci; i = (i + 1) % n) store_state(pool->get_app_rr(i)->h_state, APP_RR_STATUS::WORK_COMPLETE);
      {
        std::lock_guard<std::mutex> g(stats_mu_);
        note_batch(appIdx, win, getCurNs() - t0);
        if (!ok) stats_[appIdx].wait_timeouts++;
      }
      num_req.fetch_add((uint64_t)win);
      a->consumer_seq += (uint64_t)win;
      si = ci;
      win = 0;
      update_batch_size(appIdx);
    }
  }

  void dynamic_batching_sync_worker_loop(int appIdx, const int max_batch_size) {
    P2pRpcAppInfo* a = all_apps[appIdx];
    P2pRpcAppRrPool* pool = a->app_rr_pool;
    const int n = a->rr_pool_size;
    int ci = 0, si = 0, win = 0;
    a->consumer_seq = 0;
    IdleBackoff backoff;
    // A gather rings the doorbells of a whole burst of slots "at once", but the stores land one after the other: a
    // worker that looks in between would cut the burst into two small batches.  After the first ready slot it therefore
    // lingers for a few microseconds while the window is not full and slots keep arriving (P2P_RPC_BATCH_LINGER_US).
    const uint64_t linger_ns = (uint64_t)readEnvInfo<uint64_t>("P2P_RPC_BATCH_LINGER_US", 10) * 1000ull;
    while (!should_stop()) {
      uint64_t last_arrival = 0;
      for (;;) {
        bool grew = false;
        while (win < max_batch_size && load_state(pool->get_app_rr(ci)->h_state) == APP_RR_STATUS::RX_COMPLETE) {
          win++;
          ci = (ci + 1) % n;
          grew = true;
        }
        if (win == 0 || win >= max_batch_size || linger_ns == 0) break;
        uint64_t now = getCurNs();
        if (grew) last_arrival = now;
        else if (now - last_arrival > linger_ns) break;
      }
      if (win == 0) {
        backoff.empty();
        continue;
      }
      backoff.busy();
      uint64_t t0 = getCurNs();
      bool ok = do_batch_work_sync(appIdx, si, win);
      if (!a->completion_by_device)
        for (int i = si; i != ci; i = (i + 1) % n) store_state(pool->get_app_rr(i)->h_state, APP_RR_STATUS::WORK_COMPLETE);
      {
        std::lock_guard<std::mutex> g(stats_mu_);
        note_batch(appIdx, win, getCurNs() - t0);
        if (!ok) stats_[appIdx].wait_timeouts++;
      }
      num_req.fetch_add((uint64_t)win);
      a->consumer_seq += (uint64_t)win;
      win = 0;
      si = ci;
    }
  }

  // Queues, on the work stream: wait until slot last_rr_idx is RX_COMPLETE, run
  // the app on the window that starts at start_rr_idx, then write 1 into the
  // doorbell.  Nothing here blocks on a GPU device; on the CPU device the wait
  // is a bounded spin.
  void pre_launch_work(int appIdx, int start_rr_idx, int last_rr_idx) {
    P2pRpcAppInfo* a = all_apps[appIdx];
    AppCtx* c = a->app_ctx;
    // The window may not have been bound by its producer yet: take its addresses
    // from the ring arithmetic, not from the slot.
    *c->h_stub = a->app_rr_pool->window_stub(a->consumer_seq);
    c->h_push->first_slot = (uint32_t)start_rr_idx;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    c->AppRrRunNotify(a->app_rr_pool->get_app_rr(last_rr_idx)->d_state, APP_RR_STATUS::RX_COMPLETE);
    if (c->last_status == 0 || c->device_id >= 0) {
      a->stage_window(start_rr_idx, c->curr_batch_size, true);  // runs after the doorbell wait
      a->app_run(c);
      a->push_responses();
    }
    c->AppCompleteNotify(1U);
  }

  void async_worker_loop(int appIdx) {
    P2pRpcAppInfo* a = all_apps[appIdx];
    AppCtx* c = a->app_ctx;
    P2pRpcAppRrPool* pool = a->app_rr_pool;
    const int n = a->rr_pool_size;
    int ci = 0;
    a->consumer_seq = 0;
    c->ResetAppRunStatus();
    if (c->device_id < 0) c->wait_budget_ns = 20000000ull;  // CPU device: poll in 20 ms slices
    bool armed = false;
    IdleBackoff backoff;
    uint64_t t0 = getCurNs();
    while (!should_stop()) {
      if (!armed) {
        // On the CPU device the armed wait is synchronous; only arm when the
        // window is (about to be) ready so shutdown stays responsive.
        if (c->device_id < 0 &&
            load_state(pool->get_app_rr((ci + c->curr_batch_size - 1) % n)->h_state) != APP_RR_STATUS::RX_COMPLETE)
          continue;
        c->last_status = 0;
        t0 = getCurNs();
        pre_launch_work(appIdx, ci, (ci + c->curr_batch_size - 1) % n);
        armed = true;
      }
      if (!c->IsAppRunComplete()) {
        backoff.empty();
        continue;
      }
      backoff.busy();
      int bs = c->curr_batch_size;
      for (int i = 0; i < bs; i++) {
        if (!a->completion_by_device) store_state(pool->get_app_rr(ci)->h_state, APP_RR_STATUS::WORK_COMPLETE);
        ci = (ci + 1) % n;
      }
      {
        std::lock_guard<std::mutex> g(stats_mu_);
        note_batch(appIdx, bs, getCurNs() - t0);
      }
      num_req.fetch_add((uint64_t)bs);
      a->consumer_seq += (uint64_t)bs;
      update_batch_size(appIdx);
      c->ResetAppRunStatus();
      if (a->app_complete) a->app_complete(c);
      armed = false;
    }
    if (armed && c->device_id >= 0) {
      // Let the armed stream run through: mark the awaited slot ready, then wait
      // (bounded by the stream sync) for the queued work to drain.  The window
      // holds no requests, so the kernels must neither store responses nor
      // complete its slots: the push block is read when they run, switch it off.
      int last = (ci + c->curr_batch_size - 1) % n;
      const uint32_t push_was = c->h_push->enabled;
      c->h_push->enabled = 0;
      std::atomic_thread_fence(std::memory_order_seq_cst);
      store_state(pool->get_app_rr(last)->h_state, APP_RR_STATUS::RX_COMPLETE);
      c->WaitForAppRunComplete();
      store_state(pool->get_app_rr(last)->h_state, APP_RR_STATUS::FREE);
      c->h_push->enabled = push_was;
      c->ResetAppRunStatus();
    }
  }
};
