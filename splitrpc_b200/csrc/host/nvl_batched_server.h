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

#include <deque>
#include <functional>
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
  // Pull mode: the producer's payload regions as this process maps them, the engine that fetches from them (this
  // app's own scatter-gather engine) and the thread that turns described slots into gathers.
  P2pRpcSgEngine* pull_engine_ = nullptr;
  SrpcSharedMem regions_[NVL_MAX_REGIONS];
  std::atomic<int> n_regions_{0};  // entries below it never change while the fetch thread runs
  std::thread puller_;
  std::atomic<bool> pull_quit_{false};
  bool pull_ = false;
  std::atomic<uint64_t> pulled_{0}, pull_errors_{0};

  // Fetch thread: takes described slots in ring order, builds their copy lists from the descriptors and hands them
  // to the engine, whose kernel (or memcpy) marks each slot RX_COMPLETE when its bytes are in the ring.
  void pull_loop() {
    P2pRpcAppRrPool* pool = app_->app_rr_pool;
    P2pRpcAppRrMemPool* mp = pool->rr_mem_pool;
    const int n = pool->get_pool_size();
    const int burst = max_batch_ > 0 ? max_batch_ : 1;
    const bool gpu = app_->device_id >= 0;
    if (gpu) srpc_require_cuda("pull thread")->set_device(app_->device_id);
    std::vector<std::unique_ptr<P2pRpcRr>> rr((size_t)n);
    for (auto& r : rr) r.reset(new P2pRpcRr(nullptr, app_->req_size));
    std::vector<g_params> stubs((size_t)n);
    std::vector<P2pRpcRr*> rp((size_t)burst);
    std::vector<g_params*> sp((size_t)burst);
    std::vector<volatile uint32_t*> hs((size_t)burst), ds((size_t)burst);
    int pi = 0;
    uint64_t seq = 0;
    IdleBackoff backoff;
    while (!pull_quit_.load(std::memory_order_acquire)) {
      int k = 0;
      while (k < burst && __atomic_load_n(pool->get_app_rr((pi + k) % n)->h_state, __ATOMIC_ACQUIRE) == (uint32_t)APP_RR_STATUS::RX_DESCRIBED) k++;
      if (k == 0) {
        backoff.empty();
        continue;
      }
      backoff.busy();
      int good = 0;
      for (int j = 0; j < k; j++) {
        const int slot = (pi + j) % n;
        const SrpcSlotDesc* d = mp->get_slot_desc(slot);
        P2pRpcRr* r = rr[(size_t)slot].get();
        r->clear_bufs();
        // The descriptors come from another process: nothing in them is trusted.  A request may name at most as many
        // bytes as a ring slot holds, every fragment must lie inside a mapped region.
        const uint32_t nf = d->n_frags;
        bool ok = nf > 0 && nf <= mp->desc_per_slot() && nf <= MAX_BI_SIZE;
        uint64_t total = 0;
        for (uint32_t f = 0; ok && f < nf; f++) {
          const uint32_t region = (uint32_t)(d->frag[f].where >> 56);
          const uint64_t off = d->frag[f].where & ((1ull << 56) - 1);
          total += d->frag[f].len;
          if (d->frag[f].len == 0 || total > app_->req_size || region >= (uint32_t)n_regions_.load(std::memory_order_acquire) ||
              off + d->frag[f].len > regions_[region].bytes) {
            ok = false;
            break;
          }
          const uint8_t* base = (const uint8_t*)(gpu ? regions_[region].dev : regions_[region].host);
          r->payload_bufs->burst_items[f] = (uintptr_t)(base + off);
          r->payload_bufs->item_size[f] = d->frag[f].len;
        }
        volatile uint32_t* hstate = pool->get_app_rr(slot)->h_state;
        if (!ok) {
          // Hand the slot on anyway (the app answers with whatever the ring holds) rather than stall the ring.
          pull_errors_++;
          srpc_log(SRPC_LOG_ERROR, "pull: slot %d carries a malformed fragment list", slot);
          __atomic_store_n(hstate, (uint32_t)APP_RR_STATUS::RX_COMPLETE, __ATOMIC_RELEASE);
          continue;
        }
        r->payload_bufs->num_items = (uint16_t)nf;
        stubs[(size_t)slot] = pool->window_stub(seq + (uint64_t)j);
        rp[(size_t)good] = r;
        sp[(size_t)good] = &stubs[(size_t)slot];
        hs[(size_t)good] = hstate;
        ds[(size_t)good] = pool->get_app_rr(slot)->d_state;
        good++;
      }
      if (good > 0 &&
          pull_engine_->gather_batch_notify(rp.data(), sp.data(), hs.data(), ds.data(), good, (uint32_t)APP_RR_STATUS::RX_COMPLETE) < 0) {
        pull_errors_ += (uint64_t)good;
        srpc_log(SRPC_LOG_ERROR, "pull: could not fetch %d described request(s)", good);
        for (int j = 0; j < good; j++) __atomic_store_n(hs[(size_t)j], (uint32_t)APP_RR_STATUS::RX_COMPLETE, __ATOMIC_RELEASE);
      }
      pulled_ += (uint64_t)k;
      pi = (pi + k) % n;
      seq += (uint64_t)k;
    }
  }

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
    if (pull_) {
      P2pRpcAppRrMemPool* mp = pool->rr_mem_pool;
      pull_engine_->set_stamp_layout(mp->get_doorbells_host(), mp->get_stamps_host(), mp->get_doorbells_device(), mp->get_stamps_device());
      pull_quit_.store(false);
      puller_ = std::thread([this] { pull_loop(); });
    }
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
    pull_quit_.store(true, std::memory_order_release);
    if (puller_.joinable()) puller_.join();
    app_server_.quit();
    if (worker_.joinable()) worker_.join();
    app_->disable_device_completion();
    app_->use_window_stub = false;
    srpc_shm_free(&tx_arena_);
    for (int i = 0; i < n_regions_.load(); i++) srpc_shm_free(&regions_[i]);
    n_regions_.store(0);
    pull_ = false;
  }
  bool add_region(int fd, uint64_t bytes) {
    const int at = n_regions_.load();
    if (at >= NVL_MAX_REGIONS) return false;
    if (app_->device_id >= 0) srpc_require_cuda("pull regions")->set_device(app_->device_id);
    SrpcSharedMem m;
    if (!srpc_shm_import(fd, bytes, app_->device_id >= 0, &m)) return false;
    regions_[at] = m;
    n_regions_.store(at + 1, std::memory_order_release);
    return true;
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
    int next_fd = 0;
    if (n_fds >= 1 && req.tx_arena.length > 0) {
      if (srpc_shm_import(fds[0], req.tx_arena.length, app_->device_id >= 0, &tx_arena_)) {
        tx_base = (uint64_t)(uintptr_t)tx_arena_.dev;
        tx_bytes = tx_arena_.bytes;
      } else {
        ::close(fds[0]);
        srpc_log(SRPC_LOG_WARN, "batched server: could not map the producer's transmit arena; responses stay in the ring");
      }
      next_fd = 1;
    }
    // Pull mode: map the producer's payload regions (all of them, or the mode stays off).
    pull_ = false;
    if (req.pull && pull_engine_ && req.n_regions > 0 && req.n_regions <= (uint32_t)NVL_MAX_REGIONS && next_fd + (int)req.n_regions <= n_fds) {
      bool ok = true;
      for (uint32_t i = 0; i < req.n_regions; i++) {
        if (!ok || !add_region(fds[next_fd], req.region_bytes[i])) {
          ::close(fds[next_fd]);
          ok = false;
        }
        next_fd++;
      }
      if (!ok) {
        srpc_log(SRPC_LOG_WARN, "batched server: could not map the producer's payload regions; it will push instead");
        for (int i = 0; i < n_regions_.load(); i++) srpc_shm_free(&regions_[i]);
        n_regions_.store(0);
      }
      pull_ = ok;
    }
    for (int i = next_fd; i < n_fds; i++) ::close(fds[i]);
    rep.pull = pull_ ? 1u : 0u;
    rep.tx_arena.length = tx_bytes;  // 0: this side could not map the arena, responses stay in the response ring
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
    int fds[NVL_MAX_FDS], n_fds = 0;
    int r = ch.recv_msg(&msg, sizeof(msg), fds, NVL_MAX_FDS, &n_fds, 0);
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
    } else if (msg.type == BUF_MON_REGION) {
      buf_mon_rr rep{};
      rep.type = BUF_MON_REGION;
      rep.func_id = func_id_;
      rep.status = -1;
      if (pull_ && n_fds >= 1 && add_region(fds[0], msg.region_bytes[0])) {
        rep.status = 0;
        rep.n_regions = (uint32_t)n_regions_.load();
        for (int i = 1; i < n_fds; i++) ::close(fds[i]);
      } else {
        for (int i = 0; i < n_fds; i++) ::close(fds[i]);
      }
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
    int fds[NVL_MAX_FDS], n_fds = 0;
    if (ch.recv_msg(&msg, sizeof(msg), fds, NVL_MAX_FDS, &n_fds, 200) == 1) {
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

  // Engine that fetches described requests (pull mode): normally the app's own scatter-gather engine, with the
  // ingress transform, if any, already set on it.  Without one the server only accepts pushed requests.
  void set_pull_engine(P2pRpcSgEngine* e) { pull_engine_ = e; }
  bool pulling() const { return pull_; }
  uint64_t pulled() const { return pulled_.load(); }
  uint64_t pull_errors() const { return pull_errors_.load(); }
  // Device-side (host-side on the CPU device) base address and size of the producer's i-th payload region.
  bool region(int i, uint64_t* base, uint64_t* bytes) const {
    if (i < 0 || i >= n_regions_.load(std::memory_order_acquire)) return false;
    *base = (uint64_t)(uintptr_t)(app_->device_id >= 0 ? regions_[i].dev : regions_[i].host);
    *bytes = regions_[i].bytes;
    return true;
  }

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

// Ingress side of pull mode: a "gather" only writes where the request's fragments are into the slot's descriptor
// block and marks the slot RX_DESCRIBED; the serving side moves the bytes.  A ticket is done when the serving side has
// taken all its requests out of the regions (their slots have left RX_DESCRIBED), which is when the receive buffers can
// be reused.  Responses that the serving side did not push are fetched by `fetch` (the engine that maps the rings).
class P2pRpcSgDescribeEngine : public P2pRpcSgEngine {
  P2pRpcAppRrMemPool* mp_;
  std::vector<DmaRegion> regions_;
  P2pRpcSgEngine* fetch_;
  bool dev_addr_;  // fragment addresses arrive as the ingress GPU sees them (otherwise as the host does)
  struct Pending {
    int64_t ticket;
    std::vector<uint32_t> slots;
  };
  std::deque<Pending> pending_;
  int64_t ticket_ = 0;
  std::vector<SrpcFragDesc> tmp_;
  // Regions can appear after the handshake (a sender's by-reference buffer): `list_` re-reads the port's regions,
  // `announce_` shares a new one with the serving side.
  std::function<int(DmaRegion*, int)> list_;
  std::function<bool(const DmaRegion&)> announce_;

  bool refresh_regions() {
    if (!list_ || !announce_) return false;
    DmaRegion all[NVL_MAX_REGIONS];
    const int n = list_(all, NVL_MAX_REGIONS);
    bool grew = false;
    for (int i = (int)regions_.size(); i < n; i++) {
      if (all[i].fd < 0 || !announce_(all[i])) return grew;
      regions_.push_back(all[i]);
      grew = true;
    }
    return grew;
  }
  bool locate(uintptr_t addr, size_t len, uint64_t* where) {
    return locate_known(addr, len, where) || (refresh_regions() && locate_known(addr, len, where));
  }
  bool locate_known(uintptr_t addr, size_t len, uint64_t* where) const {
    for (size_t r = 0; r < regions_.size(); r++) {
      const uintptr_t base = (uintptr_t)(dev_addr_ ? regions_[r].dev_base : regions_[r].host_base);
      if (addr >= base && addr + len <= base + regions_[r].bytes) {
        *where = ((uint64_t)r << 56) | (uint64_t)(addr - base);
        return true;
      }
    }
    return false;
  }

 public:
  P2pRpcSgDescribeEngine(P2pRpcAppRrMemPool* mp, const DmaRegion* regions, int n_regions, P2pRpcSgEngine* fetch, bool dev_addr)
      : mp_(mp), regions_(regions, regions + n_regions), fetch_(fetch), dev_addr_(dev_addr) {}
  void set_region_source(std::function<int(DmaRegion*, int)> list, std::function<bool(const DmaRegion&)> announce) {
    list_ = std::move(list);
    announce_ = std::move(announce);
  }
  const char* name() const override { return "describe"; }
  int gather(P2pRpcRr*, g_params*) override { return -1; }  // only the notifying batch form exists
  int scatter(P2pRpcRr* rr, g_params* stub) override { return fetch_ ? fetch_->scatter(rr, stub) : -1; }
  int scatter_batch(P2pRpcRr** rrs, g_params** stubs, int n) override { return fetch_ ? fetch_->scatter_batch(rrs, stubs, n) : -1; }
  int copy_list(const p2p_sk_buf* skb) override { return fetch_ ? fetch_->copy_list(skb) : -1; }

  int64_t gather_batch_notify(P2pRpcRr** rrs, g_params** stubs, volatile uint32_t** h_states, volatile uint32_t** d_states, int n,
                              uint32_t state_value) override {
    (void)stubs;
    (void)d_states;
    (void)state_value;
    const uint32_t cap = mp_->desc_per_slot();
    volatile uint32_t* base = mp_->get_doorbells_host();
    Pending pend;
    for (int i = 0; i < n; i++) {
      const p2p_bufs* fr = rrs[i]->payload_bufs;
      tmp_.clear();
      uintptr_t run_end = 0;
      uint32_t dst = 0;
      for (size_t f = 0; f < fr->num_items; f++) {
        const uintptr_t src = fr->burst_items[f];
        const size_t len = fr->item_size[f];
        if (!tmp_.empty() && src == run_end && (uint64_t)tmp_.back().len + len <= 0xFFFFFFFFull) {
          tmp_.back().len += (uint32_t)len;  // still inside one region: the run started there and is contiguous
        } else {
          SrpcFragDesc d{0, (uint32_t)len, dst};
          if (!locate(src, len, &d.where)) {
            srpc_log(SRPC_LOG_ERROR, "describe: a fragment lies outside the shared regions");
            return -5;
          }
          tmp_.push_back(d);
        }
        run_end = src + len;
        dst += (uint32_t)len;
      }
      // a merged run must not leave its region
      for (const SrpcFragDesc& d : tmp_) {
        const uint32_t r = (uint32_t)(d.where >> 56);
        if ((d.where & ((1ull << 56) - 1)) + d.len > regions_[r].bytes) return -5;
      }
      if (tmp_.empty() || tmp_.size() > cap) return -4;
      const uint32_t slot = (uint32_t)(h_states[i] - base);
      SrpcSlotDesc* sd = mp_->get_slot_desc((int)slot);
      for (size_t k = 0; k < tmp_.size(); k++) sd->frag[k] = tmp_[k];
      sd->n_frags = (uint32_t)tmp_.size();
      pend.slots.push_back(slot);
    }
    std::atomic_thread_fence(std::memory_order_release);
    for (int i = 0; i < n; i++) __atomic_store_n(h_states[i], (uint32_t)APP_RR_STATUS::RX_DESCRIBED, __ATOMIC_RELEASE);
    pend.ticket = ++ticket_;
    pending_.push_back(std::move(pend));
    counters.gathers += (uint64_t)n;
    return ticket_;
  }
  bool ticket_done(int64_t ticket) override {
    volatile uint32_t* base = mp_->get_doorbells_host();
    while (!pending_.empty() && pending_.front().ticket <= ticket) {
      for (uint32_t s : pending_.front().slots)
        if (__atomic_load_n(base + s, __ATOMIC_ACQUIRE) == (uint32_t)APP_RR_STATUS::RX_DESCRIBED) return false;
      pending_.pop_front();
    }
    return true;
  }
};

// GPU engine factory of the CUDA half (null without CUDA).
extern "C" P2pRpcSgEngine* srpc_make_gpu_sg_engine(int device_id, int copy_type);

class NvlRemoteReplica {
  NvlCtrlChannel ch_;
  std::unique_ptr<P2pRpcAppRrPool> pool_;
  std::unique_ptr<P2pRpcSgEngine> engine_;           // what the server's shunter drives
  std::unique_ptr<P2pRpcSgEngine> fetch_engine_;     // pull mode: the engine that maps the rings (response fetches)
  buf_mon_rr info_{};
  int64_t stamp_skew_ns_ = 0;
  std::mutex mu_;

 public:
  // Connects to the batched server listening at `path` and performs the ALLOC handshake.  `ingress_device`: the GPU
  // whose kernels will fill the rings (-1: the CPU engine; only for rings in host memory).  `tx`: this process's
  // transmit arena (may be null or unshareable: responses then stay in the response ring and are fetched from there).
  static std::unique_ptr<NvlRemoteReplica> connect(const std::string& path, uint32_t func_id, int ingress_device, int copy_type,
                                                   const TxArenaInfo* tx, int timeout_ms, std::string* err,
                                                   const Transport* pull_from = nullptr) {
    // Pull mode: `pull_from` is the port whose received payloads the server should fetch by itself.
    DmaRegion regions[NVL_MAX_REGIONS];
    const int n_regions = pull_from ? pull_from->dma_regions(regions, NVL_MAX_REGIONS) : 0;
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
    // Pull mode is asked for when every region can be mapped by another process.
    int out_fds[NVL_MAX_FDS], n_out = 0;
    if (tx_fd >= 0) out_fds[n_out++] = tx_fd;
    bool want_pull = n_regions > 0 && n_regions <= NVL_MAX_REGIONS;
    for (int i = 0; want_pull && i < n_regions; i++) want_pull = regions[i].fd >= 0 && regions[i].bytes > 0;
    if (want_pull) {
      req.pull = 1;
      req.n_regions = (uint32_t)n_regions;
      for (int i = 0; i < n_regions; i++) {
        req.region_bytes[i] = regions[i].bytes;
        out_fds[n_out++] = regions[i].fd;
      }
    }
    if (!r->ch_.send_msg(&req, sizeof(req), n_out ? out_fds : nullptr, n_out)) return fail("ALLOC send failed");
    int fds[NVL_MAX_FDS], n_fds = 0;
    if (r->ch_.recv_msg(&r->info_, sizeof(r->info_), fds, NVL_MAX_FDS, &n_fds, timeout_ms) != 1) return fail("no ALLOC reply");
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
    if (r->info_.pull) {
      // The server fetches by itself: the shunter only describes.  Both stamps then come from the serving device.
      r->fetch_engine_ = std::move(r->engine_);
      auto* de = new P2pRpcSgDescribeEngine(r->pool_->rr_mem_pool, regions, n_regions, r->fetch_engine_.get(), ingress_device >= 0);
      NvlRemoteReplica* self = r.get();
      de->set_region_source([pull_from](DmaRegion* out, int max) { return pull_from->dma_regions(out, max); },
                            [self](const DmaRegion& reg) { return self->add_region(reg); });
      r->engine_.reset(de);
      r->stamp_skew_ns_ = 0;
    }
    return r;
  }
  // (completion stamp - doorbell stamp) exceeds the true latency by this much: the two stamps come from different
  // devices' timers.
  int64_t stamp_skew_ns() const { return stamp_skew_ns_; }

  P2pRpcAppRrPool* pool() { return pool_.get(); }
  P2pRpcSgEngine* engine() { return engine_.get(); }
  const buf_mon_rr& info() const { return info_; }
  bool device_completes() const { return info_.device_completes != 0; }
  bool pulls() const { return info_.pull != 0; }
  // The serving side stores single-fragment responses straight into this process's transmit arena.
  bool pushes_responses() const { return info_.device_completes != 0 && info_.tx_arena.length > 0; }

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
  // Shares one more payload region with the server (pull mode).
  bool add_region(const DmaRegion& reg, int timeout_ms = 3000) {
    std::lock_guard<std::mutex> g(mu_);
    if (!ch_.ok() || reg.fd < 0) return false;
    buf_mon_rr m{};
    m.type = BUF_MON_REGION;
    m.func_id = info_.func_id;
    m.n_regions = 1;
    m.region_bytes[0] = reg.bytes;
    int fd = reg.fd;
    if (!ch_.send_msg(&m, sizeof(m), &fd, 1)) return false;
    return ch_.recv_msg(&m, sizeof(m), nullptr, 0, nullptr, timeout_ms) == 1 && m.type == BUF_MON_REGION && m.status == 0;
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
