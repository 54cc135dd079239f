// Serving a GPU's app to a producer that lives in another process: the batched server and the producer's view of it.
//
// NvlBatchedServer is the NVLink counterpart of the original's host-side batched GPU server (reference
// src/splitrpc_rdma_transport/gpu_rdma_batched_server.cc:229-487): it owns one app with its request ring, response
// ring and per-slot doorbells, answers a buf_mon ALLOC by exposing those three regions to the producer, then runs one
// of the three worker modes (0 fixed batch, 1 stream armed, 2 dynamic batching) over the slots (a negative mode starts
// no worker: the embedding program consumes the slots itself).  The producer (the
// ingress process, the role of the original's SmartNIC proxy) fills slots and rings their doorbells from ITS side:
// payload stores followed by a release store of RX_COMPLETE into the slot's state word, both issued by the ingress
// GPU's gather kernel, so this server's CPU is not involved in a request's arrival.  Completion goes the other way
// without a CPU as well: the app's last kernel (or a small push kernel behind it) stores the response into the
// producer's transmit arena and release-stores WORK_COMPLETE, which the producer polls; the original's forwarder
// thread and its SEND_WITH_IMM per slot (:441-458) have no counterpart.
//
// NvlRemoteReplica is the producer's half (the original's P2pRpcBfRrPool + connection set-up, reference
// src/splitrpc_rdma_transport/p2p_rpc_bf_rr_pool.h:13-181, gpu_dpdk_rdma_proxy_handler.cc:327-382): it connects, sends
// ALLOC together with its transmit arena, maps the three regions, and offers a mirror of the slot pool plus a
// scatter-gather engine that writes into it.
//
// Failure detection: each side notices the other's death on the control socket (end of file).  The server then stops
// its worker, forgets the producer's arena and listens again; the producer reports the replica as not alive so that
// flow steering skips it.  No GPU is involved in detecting either.
#pragma once

#include <thread>

#include "nvl_transport_common.h"
#include "p2p_rpc_async_app_server.h"
#include "p2p_rpc_sg_engine.h"
#include "transport.h"

struct NvlServerCounters {
  std::atomic<uint64_t> allocs{0}, releases{0}, peers_lost{0}, refused{0};
};

class NvlBatchedServer {
  P2pRpcAppInfo* app_;
  std::string path_;
  uint32_t func_id_;
  int server_mode_, max_batch_;
  nvl_ingress_transform transform_{};
  int listen_fd_ = -1;
  P2pRpcAsyncAppServer app_server_;
  int app_idx_ = -1;
  std::thread ctl_thread_, worker_;
  std::atomic<bool> quit_{false};
  std::atomic<bool> serving_{false};
  SrpcSharedMem tx_arena_{};

  void start_worker() {
    P2pRpcAppRrPool* pool = app_->app_rr_pool;
    pool->init_pool();
    for (int i = 0; i < pool->get_pool_size(); i++) {
      P2pRpcAppRr* r = pool->get_app_rr(i);
      __atomic_store_n(r->h_state, (uint32_t)APP_RR_STATUS::FREE, __ATOMIC_RELEASE);
      *r->h_tx_off = P2pRpcAppRrMemPool::kNoTxOffset;
    }
    app_->consumer_seq = 0;
    app_->use_window_stub = true;
    app_->app_ctx->curr_batch_size = max_batch_;
    app_->app_ctx->next_batch_size = max_batch_;
    app_server_.reset_quit();
    serving_.store(true);
    if (server_mode_ < 0) return;  // the embedder runs the app itself (timing loops, tests)
    worker_ = std::thread([this] {
      switch (server_mode_) {
        case 1: app_server_.async_worker_loop(app_idx_); break;
        case 2: app_server_.dynamic_batching_sync_worker_loop(app_idx_, max_batch_); break;
        default: app_server_.sync_worker_loop(app_idx_); break;
      }
    });
  }
  void stop_worker() {
    if (!serving_.exchange(false)) return;
    app_server_.quit();
    if (worker_.joinable()) worker_.join();
    app_->disable_device_completion();
    app_->use_window_stub = false;
    srpc_shm_free(&tx_arena_);
  }

  bool handle_alloc(NvlCtrlChannel& ch, const buf_mon_rr& req, int* fds, int n_fds) {
    buf_mon_rr rep{};
    rep.type = BUF_MON_ALLOC;
    rep.func_id = func_id_;
    auto refuse = [&](int code) {
      for (int i = 0; i < n_fds; i++) ::close(fds[i]);
      rep.status = code;
      counters.refused++;
      ch.send_msg(&rep, sizeof(rep));
      return false;
    };
    if (req.func_id != func_id_) return refuse(-1);
    if (serving_.load()) return refuse(-2);  // one producer at a time
    AppRrPoolExport ex;
    if (!app_->app_rr_pool->rr_mem_pool->export_to(&ex, app_->req_size, app_->resp_size)) return refuse(-3);
    int out_fds[3] = {ex.req_fd, ex.resp_fd, ex.ctl_fd};
    // Measured before the worker starts: once a work stream is parked on a doorbell nothing new may be loaded or run
    // to completion on this GPU on the host's behalf.
    rep.timer_offset_ns = 0;  // a CPU app stamps with the steady clock itself
    if (app_->device_id >= 0) {
      const SrpcDeviceOps* ops = srpc_cuda_ops();
      if (ops && ops->timer_offset_ns) ops->timer_offset_ns(app_->device_id, &rep.timer_offset_ns);
    }
    // The producer's transmit arena, if it sent one: responses are stored there by this side.
    uint64_t tx_base = 0, tx_bytes = 0;
    if (n_fds >= 1 && req.tx_arena.length > 0) {
      if (srpc_shm_import(fds[0], req.tx_arena.length, app_->device_id >= 0, &tx_arena_)) {
        tx_base = (uint64_t)(uintptr_t)tx_arena_.dev;
        tx_bytes = tx_arena_.bytes;
      } else {
        ::close(fds[0]);
        srpc_log(SRPC_LOG_WARN, "batched server: could not map the producer's transmit arena; responses stay in the ring");
      }
      for (int i = 1; i < n_fds; i++) ::close(fds[i]);
    } else {
      for (int i = 0; i < n_fds; i++) ::close(fds[i]);
    }
    app_->enable_device_completion(tx_base, tx_bytes);
    start_worker();
    rep.status = 0;
    rep.queue_size = ex.pool_size;
    rep.req_size = app_->req_size;
    rep.resp_size = app_->resp_size;
    rep.device_id = app_->device_id;
    rep.server_mode = (uint32_t)server_mode_;
    rep.max_batch = (uint32_t)max_batch_;
    rep.device_completes = 1;
    rep.req_buf = {(uint64_t)(uintptr_t)app_->app_rr_pool->rr_mem_pool->get_req_addr_range(), ex.req_capacity, 0, 0};
    rep.resp_buf = {(uint64_t)(uintptr_t)app_->app_rr_pool->rr_mem_pool->get_resp_addr_range(), ex.resp_capacity, 1, 0};
    rep.ctl_buf = {(uint64_t)(uintptr_t)app_->app_rr_pool->rr_mem_pool->get_doorbells_host(), ex.ctl_bytes, 2, 0};
    rep.transform = transform_;
    bool ok = ch.send_msg(&rep, sizeof(rep), out_fds, 3);
    for (int f : out_fds) ::close(f);
    if (!ok) stop_worker();
    else counters.allocs++;
    return ok;
  }

  // Handles one message of the connected producer.  Returns false when the connection is over.
  bool serve_one(NvlCtrlChannel& ch) {
    buf_mon_rr msg{};
    int fds[4], n_fds = 0;
    int r = ch.recv_msg(&msg, sizeof(msg), fds, 4, &n_fds, 0);
    if (r == 0) return true;
    if (r < 0) {  // the producer went away (without RELEASE if it was still being served)
      if (serving_.load()) counters.peers_lost++;
      return false;
    }
    if (msg.type == BUF_MON_ALLOC) {
      handle_alloc(ch, msg, fds, n_fds);
    } else if (msg.type == BUF_MON_RELEASE) {
      stop_worker();
      counters.releases++;
      buf_mon_rr rep{};
      rep.type = BUF_MON_RELEASE;
      rep.func_id = func_id_;
      fill_stats(&rep);
      ch.send_msg(&rep, sizeof(rep));
    } else if (msg.type == BUF_MON_STATS) {
      buf_mon_rr rep{};
      rep.type = BUF_MON_STATS;
      rep.func_id = func_id_;
      fill_stats(&rep);
      ch.send_msg(&rep, sizeof(rep));
    }
    return true;
  }
  // A second producer while one is connected: read its request and refuse it.
  void refuse_connection(int fd) {
    NvlCtrlChannel ch(fd);
    buf_mon_rr msg{};
    int fds[4], n_fds = 0;
    if (ch.recv_msg(&msg, sizeof(msg), fds, 4, &n_fds, 200) == 1) {
      for (int i = 0; i < n_fds; i++) ::close(fds[i]);
      buf_mon_rr rep{};
      rep.type = msg.type;
      rep.func_id = func_id_;
      rep.status = -2;
      ch.send_msg(&rep, sizeof(rep));
    }
    counters.refused++;
  }
  void fill_stats(buf_mon_rr* rep) {
    WorkerStats w = app_server_.stats(app_idx_);
    rep->stat_served = w.num_req;
    rep->stat_batches = w.num_batches;
  }

  void ctl_loop() {
    NvlCtrlChannel conn;
    while (!quit_.load(std::memory_order_acquire)) {
      pollfd p[2] = {{listen_fd_, POLLIN, 0}, {conn.ok() ? conn.fd() : -1, POLLIN, 0}};
      if (::poll(p, 2, 50) <= 0) continue;
      if (p[1].revents && conn.ok() && !serve_one(conn)) {
        stop_worker();
        conn.close_fd();
      }
      if (p[0].revents & POLLIN) {
        int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd < 0) continue;
        if (conn.ok()) refuse_connection(fd);
        else conn = NvlCtrlChannel(fd);
      }
    }
    stop_worker();
  }

 public:
  NvlServerCounters counters;

  NvlBatchedServer(P2pRpcAppInfo* app, const std::string& path, uint32_t func_id, int server_mode, int max_batch)
      : app_(app), path_(path), func_id_(func_id), server_mode_(server_mode), max_batch_(max_batch) {
    app_idx_ = app_server_.register_app(app_);
  }
  ~NvlBatchedServer() { stop(); }

  // Producers must deserialise into this app's request ring with this transform (see SG_TRANSFORM_*).
  void set_ingress_transform(uint32_t kind, const float* params6) {
    transform_.kind = kind;
    for (int i = 0; i < 6; i++) transform_.params[i] = params6 ? params6[i] : 0.f;
  }

  bool start() {
    if (listen_fd_ >= 0) return true;
    listen_fd_ = NvlCtrlChannel::listen_at(path_);
    if (listen_fd_ < 0) return false;
    quit_.store(false);
    ctl_thread_ = std::thread([this] { ctl_loop(); });
    return true;
  }
  void stop() {
    if (listen_fd_ < 0) return;
    quit_.store(true, std::memory_order_release);
    if (ctl_thread_.joinable()) ctl_thread_.join();
    stop_worker();
    ::close(listen_fd_);
    ::unlink(path_.c_str());
    listen_fd_ = -1;
  }
  bool serving() const { return serving_.load(); }
  WorkerStats worker_stats() { return app_server_.stats(app_idx_); }
};

// GPU engine factory of the CUDA half (null without CUDA).
extern "C" P2pRpcSgEngine* srpc_make_gpu_sg_engine(int device_id, int copy_type);

class NvlRemoteReplica {
  NvlCtrlChannel ch_;
  std::unique_ptr<P2pRpcAppRrPool> pool_;
  std::unique_ptr<P2pRpcSgEngine> engine_;
  buf_mon_rr info_{};
  int64_t stamp_skew_ns_ = 0;
  std::mutex mu_;

 public:
  // Connects to the batched server listening at `path` and performs the ALLOC handshake.  `ingress_device`: the GPU
  // whose kernels will fill the rings (-1: the CPU engine; only for rings in host memory).  `tx`: this process's
  // transmit arena (may be null or unshareable: responses then stay in the response ring and are fetched from there).
  static std::unique_ptr<NvlRemoteReplica> connect(const std::string& path, uint32_t func_id, int ingress_device, int copy_type,
                                                   const TxArenaInfo* tx, int timeout_ms, std::string* err) {
    auto fail = [&](const std::string& m) {
      if (err) *err = m;
      return std::unique_ptr<NvlRemoteReplica>();
    };
    int fd = NvlCtrlChannel::connect_to(path, timeout_ms);
    if (fd < 0) return fail("no batched server at " + path);
    auto r = std::unique_ptr<NvlRemoteReplica>(new NvlRemoteReplica);
    r->ch_ = NvlCtrlChannel(fd);
    buf_mon_rr req{};
    req.type = BUF_MON_ALLOC;
    req.func_id = func_id;
    req.device_id = ingress_device;
    int tx_fd = -1;
    if (tx && tx->fd >= 0) {
      tx_fd = tx->fd;
      req.tx_arena = {(uint64_t)(uintptr_t)tx->host_base, tx->bytes, 0, 0};
    }
    if (!r->ch_.send_msg(&req, sizeof(req), tx_fd >= 0 ? &tx_fd : nullptr, tx_fd >= 0 ? 1 : 0)) return fail("ALLOC send failed");
    int fds[4], n_fds = 0;
    if (r->ch_.recv_msg(&r->info_, sizeof(r->info_), fds, 4, &n_fds, timeout_ms) != 1) return fail("no ALLOC reply");
    if (r->info_.status != 0 || n_fds != 3) {
      for (int i = 0; i < n_fds; i++) ::close(fds[i]);
      return fail("ALLOC refused, status " + std::to_string(r->info_.status));
    }
    AppRrPoolExport ex;
    ex.req_fd = fds[r->info_.req_buf.stag];
    ex.resp_fd = fds[r->info_.resp_buf.stag];
    ex.ctl_fd = fds[r->info_.ctl_buf.stag];
    ex.req_capacity = r->info_.req_buf.length;
    ex.resp_capacity = r->info_.resp_buf.length;
    ex.ctl_bytes = r->info_.ctl_buf.length;
    ex.pool_size = r->info_.queue_size;
    ex.owner_device = r->info_.device_id;
    ex.req_size = r->info_.req_size;
    ex.resp_size = r->info_.resp_size;
    const int dev = ex.owner_device < 0 ? -1 : ingress_device;
    if (ex.owner_device >= 0 && ingress_device < 0) {
      for (int i = 0; i < 3; i++) ::close(fds[i]);
      return fail("rings in GPU memory need a GPU on the producer side");
    }
    r->pool_.reset(new P2pRpcAppRrPool(ex, dev));
    if (!r->pool_->ok()) return fail("could not map the server's rings");
    r->pool_->init_pool();
    if (dev >= 0) {
      r->engine_.reset(srpc_make_gpu_sg_engine(dev, copy_type));
      if (!r->engine_) return fail("no GPU scatter-gather engine");
    } else {
      r->engine_.reset(new P2pRpcSgCpuEngine);
    }
    if (r->info_.transform.kind != 0 &&
        r->engine_->set_gather_transform((int)r->info_.transform.kind,
                                         (uint64_t)(uintptr_t)r->pool_->rr_mem_pool->get_req_addr_range(),
                                         (uint32_t)ex.req_size, r->info_.transform.params) != 0)
      return fail("the engine cannot apply the server's ingress transform");
    // Doorbell stamps come from the ingress device's timer, completion stamps from the serving device's.
    int64_t ingress_offset = 0;
    if (dev >= 0) {
      const SrpcDeviceOps* ops = srpc_cuda_ops();
      if (ops && ops->timer_offset_ns) ops->timer_offset_ns(dev, &ingress_offset);
    }
    r->stamp_skew_ns_ = r->info_.timer_offset_ns - ingress_offset;
    return r;
  }
  // (completion stamp - doorbell stamp) exceeds the true latency by this much: the two stamps come from different
  // devices' timers.
  int64_t stamp_skew_ns() const { return stamp_skew_ns_; }

  P2pRpcAppRrPool* pool() { return pool_.get(); }
  P2pRpcSgEngine* engine() { return engine_.get(); }
  const buf_mon_rr& info() const { return info_; }
  bool device_completes() const { return info_.device_completes != 0; }

  // false once the server has closed the control connection (it exited or was killed).
  bool alive() {
    std::lock_guard<std::mutex> g(mu_);
    if (!ch_.ok()) return false;
    char c;
    ssize_t r = ::recv(ch_.fd(), &c, 1, MSG_PEEK | MSG_DONTWAIT);
    if (r == 0) return false;
    if (r < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return false;
    return true;
  }
  bool query_stats(uint64_t* served, uint64_t* batches, int timeout_ms = 1000) {
    std::lock_guard<std::mutex> g(mu_);
    buf_mon_rr m{};
    m.type = BUF_MON_STATS;
    m.func_id = info_.func_id;
    if (!ch_.send_msg(&m, sizeof(m))) return false;
    if (ch_.recv_msg(&m, sizeof(m), nullptr, 0, nullptr, timeout_ms) != 1) return false;
    *served = m.stat_served;
    *batches = m.stat_batches;
    return true;
  }
  // Tells the server to stop its worker and forget this producer.
  bool release(int timeout_ms = 3000) {
    std::lock_guard<std::mutex> g(mu_);
    if (!ch_.ok()) return false;
    buf_mon_rr m{};
    m.type = BUF_MON_RELEASE;
    m.func_id = info_.func_id;
    bool ok = ch_.send_msg(&m, sizeof(m)) && ch_.recv_msg(&m, sizeof(m), nullptr, 0, nullptr, timeout_ms) == 1;
    ch_.close_fd();
    return ok;
  }
};
