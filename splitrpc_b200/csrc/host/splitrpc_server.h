// Server process wiring: receive thread, shunter thread, one worker per replica.
//
// Same three-stage host pipeline as reference
// src/splitrpc_server/p2p_rpc_dpdk_server.cc:45-197 — the receive loop parses
// 64-byte headers and reassembles by token, the shunter moves ready requests
// into app ring slots through a scatter-gather engine and sends finished
// responses, the worker runs the app over the slot ring — generalised to several
// replicas (one app instance per GPU) with flow steering between them, and with
// bounded waits, reassembly timeouts and back-pressure counters instead of
// unbounded spins.  The CPU never reads or writes payload bytes here: it passes
// pointers to the engines.
#pragma once

#include <deque>
#include <thread>

#include "nvl_batched_server.h"
#include "p2p_rpc_async_app_server.h"
#include "p2p_rpc_sg_engine.h"
#include "transport.h"

struct ServerConfig {
  std::string server_uri = "b8:ce:f6:cc:6a:52,192.168.25.1,50051";
  size_t req_size = 1024, resp_size = 1024;
  int server_mode = 0;      // 0 sync fixed batch, 1 async (stream armed), 2 dynamic batching
  int max_batch = 1;        // fixed batch (modes 0/1) or upper bound (mode 2)
  int zerocopy = 0;         // 1 = serve out of the receive buffers (single-fragment requests)
  int rr_pool_size = 4095;
  uint64_t reassembly_timeout_ns = 200000000ull;
  int steer_policy = 0;     // 0 = round robin in runs of max_batch, 1 = least outstanding
  int gather_burst = 64;    // requests per scatter-gather submission
  // 1 = let the serving side store single-fragment responses straight into the transmit arena and complete the slot
  // itself (see RespPushCtx) wherever the arena is reachable from the app's device; 0 = host-driven scatter.
  int device_completion = 1;
};

struct ReplicaStats {
  uint64_t steered = 0, completed = 0, ring_full = 0, pushed = 0;
};

struct ServerStats {
  uint64_t rx_pkts = 0, rx_reqs = 0, tx_resps = 0, tx_pkts = 0, dropped_pkts = 0, expired = 0, ring_full = 0,
           tx_alloc_fail = 0, sg_errors = 0, replicas_lost = 0;
  std::vector<ReplicaStats> replicas;
};

class SplitRpcServer {
  // A replica is a slot ring plus the engine that fills it.  Local: the app lives in this process and a worker thread
  // of this server runs it.  Remote: the ring belongs to a batched server in another process (another GPU); this
  // process holds a mirror of its slot pool and an engine on the ingress GPU that writes into it over NVLink.
  struct Replica {
    P2pRpcAppInfo* app = nullptr;
    P2pRpcAppRrPool* pool = nullptr;
    P2pRpcSgEngine* engine = nullptr;
    NvlRemoteReplica* remote = nullptr;
    bool device_completes = false;         // responses and WORK_COMPLETE arrive without this process's help
    int64_t stamp_skew_ns = 0;             // serving device's stamp timer minus the gather device's
    bool can_push = true;                  // the serving side can reach the transmit arena
    int app_idx = -1;
    int tx_idx = 0;                        // next slot whose response goes out
    std::atomic<int> outstanding{0};
    std::atomic<bool> down{false};         // steering skips a replica marked down
    struct {
      std::atomic<uint64_t> steered{0}, completed{0}, ring_full{0}, pushed{0};  // written by the shunter, read by stats()
    } stats;
    std::thread worker;
  };
  // A gather that the engine finishes by itself: the receive buffers go back to the port once its ticket is done.
  struct Inflight {
    P2pRpcSgEngine* engine;
    int64_t ticket;
    std::vector<uint32_t> rx_slots;
    const std::atomic<bool>* replica_down;  // a replica that died will never take its requests out of the buffers
  };

  Transport* port_;
  ServerConfig cfg_;
  p2p_rpc_conn_info* server_conn_ = nullptr;
  P2pRpcRRPool rr_pool_;
  P2pRpcAsyncAppServer app_server_;
  std::vector<std::unique_ptr<Replica>> replicas_;
  std::thread rx_thread_, shunter_thread_;
  std::atomic<bool> quit_{false};
  std::atomic<bool> running_{false};
  struct LiveStats {
    std::atomic<uint64_t> rx_pkts{0}, rx_reqs{0}, tx_resps{0}, tx_pkts{0}, dropped_pkts{0}, expired{0}, ring_full{0},
        tx_alloc_fail{0}, sg_errors{0}, replicas_lost{0};
  } stats_;
  int rr_cursor_ = 0, rr_run_ = 0;
  size_t resp_frags_;
  TxArenaInfo tx_info_{};
  bool have_tx_info_ = false;
  std::deque<Inflight> inflight_;
  std::mutex lat_mu_;
  std::vector<uint64_t> device_latency_ns_;  // per pushed response: doorbell rung -> response stored (device timers)

  void rx_loop() {
    std::vector<SrpcPkt> pkts(1024);
    uint64_t last_sweep = getCurNs();
    IdleBackoff backoff;
    while (!quit_.load(std::memory_order_acquire)) {
      int n = port_->rx_burst(pkts.data(), (int)pkts.size());
      if (n > 0) backoff.busy();
      else backoff.empty();
      if (n > 0) NVTX_R("rx_burst");
      for (int i = 0; i < n; i++) {
        SrpcPkt& p = pkts[i];
        stats_.rx_pkts++;
        P2pRpcRr* rr = rr_pool_.append_to_rr(p.hdr, (uintptr_t)p.slot + 1, (uintptr_t)port_->rx_dev_ptr(p), p.len);
        if (!rr) {
          stats_.dropped_pkts++;
          port_->release_rx(&p, 1);
          continue;
        }
        if (rr->is_rr_ready()) {
          rr_pool_.mark_rx_ready_rr(rr);
          stats_.rx_reqs++;
        } else if (rr->is_rr_malformed()) {
          // More bytes than the app's request size, or all the bytes with a hole in the sequence numbers:
          // protocol violation, drop the whole request.
          release_rr_rx(rr);
          rr_pool_.drop_partial(rr);
          stats_.dropped_pkts++;
        }
      }
      if (n > 0) NVTX_P();
      uint64_t now = getCurNs();
      if (now - last_sweep > cfg_.reassembly_timeout_ns / 4 + 1) {
        last_sweep = now;
        stats_.expired += rr_pool_.expire_stale(now, cfg_.reassembly_timeout_ns, [this](P2pRpcRr* rr) { release_rr_rx(rr); });
      }
    }
  }

  void release_rr_rx(P2pRpcRr* rr) {
    for (size_t i = 0; i < rr->transport_mbufs->num_items; i++) {
      uintptr_t h = rr->transport_mbufs->burst_items[i];
      if (!h) continue;
      SrpcPkt p;
      p.slot = (uint32_t)(h - 1);
      port_->release_rx(&p, 1);
      rr->transport_mbufs->burst_items[i] = 0;
    }
  }
  // Moves the receive-buffer handles of a record into `out` (they are released later, when the gather is done).
  static void take_rx_slots(P2pRpcRr* rr, std::vector<uint32_t>* out) {
    for (size_t i = 0; i < rr->transport_mbufs->num_items; i++) {
      uintptr_t h = rr->transport_mbufs->burst_items[i];
      if (h) out->push_back((uint32_t)(h - 1));
      rr->transport_mbufs->burst_items[i] = 0;
    }
  }
  void release_rx_slots(const std::vector<uint32_t>& slots) {
    SrpcPkt p;
    for (uint32_t s : slots) {
      p.slot = s;
      port_->release_rx(&p, 1);
    }
  }
  void reap_inflight(bool wait_all) {
    uint64_t t0 = getCurNs();
    while (!inflight_.empty()) {
      Inflight& f = inflight_.front();
      if (!f.engine->ticket_done(f.ticket) && !(f.replica_down && f.replica_down->load(std::memory_order_acquire))) {
        if (!wait_all || getCurNs() - t0 > 2000000000ull) return;
        continue;
      }
      release_rx_slots(f.rx_slots);
      inflight_.pop_front();
    }
  }

  int pick_replica() {
    int n = (int)replicas_.size();
    if (n == 1) return replicas_[0]->down.load() ? -1 : 0;
    if (cfg_.steer_policy == 1) {
      int best = -1, best_out = INT_MAX;
      for (int i = 0; i < n; i++) {
        if (replicas_[i]->down.load()) continue;
        int o = replicas_[i]->outstanding.load(std::memory_order_relaxed);
        if (o < best_out) {
          best_out = o;
          best = i;
        }
      }
      return best;
    }
    // Round robin in runs of max_batch so that a replica receives whole batches.
    for (int tries = 0; tries < n; tries++) {
      if (rr_run_ >= cfg_.max_batch) {
        rr_run_ = 0;
        rr_cursor_ = (rr_cursor_ + 1) % n;
      }
      if (!replicas_[rr_cursor_]->down.load()) {
        rr_run_++;
        return rr_cursor_;
      }
      rr_run_ = cfg_.max_batch;
    }
    return -1;
  }

  // Response side of a record, part 2: reply headers + buffer list over transmit buffers that were reserved before.
  void fill_tx(P2pRpcRr* rr, const SrpcPkt* tx) {
    rr->clear_bufs();
    size_t left = cfg_.resp_size, mtu = rpc_mtu();
    for (size_t i = 0; i < resp_frags_; i++) {
      size_t len = left < mtu ? left : mtu;
      left -= len;
      fill_frag_hdr(tx[i].hdr, &rr->_client_conn_info, rr->req_token, (uint16_t)i, (uint16_t)len, true);
      rr->rr_append_mbuf((uintptr_t)tx[i].slot + 1, (uintptr_t)tx[i].hdr, (uintptr_t)tx[i].payload, len);
    }
  }

  void send_response(P2pRpcRr* rr) {
    std::vector<SrpcPkt> tx(rr->transport_mbufs->num_items);
    for (size_t k = 0; k < tx.size(); k++) {
      tx[k].slot = (uint32_t)(rr->transport_mbufs->burst_items[k] - 1);
      tx[k].hdr = (p2p_rpc_hdr*)rr->hdr_bufs->burst_items[k];
      tx[k].payload = (uint8_t*)rr->payload_bufs->burst_items[k];
      tx[k].len = (uint32_t)rr->payload_bufs->item_size[k];
    }
    if (!tx.empty()) stats_.tx_pkts += (uint64_t)port_->tx_burst(tx.data(), (int)tx.size());
    stats_.tx_resps++;
    rr_pool_.reap_rr(rr);
  }

  void check_remote_replicas() {
    for (auto& rp : replicas_) {
      Replica& rep = *rp;
      if (!rep.remote || rep.down.load()) continue;
      if (!rep.remote->alive()) {
        rep.down.store(true);
        stats_.replicas_lost++;
        srpc_log(SRPC_LOG_WARN, "a remote replica closed its control connection: steering now skips it");
      }
    }
  }

  void shunter_loop() {
    const int burst = cfg_.gather_burst;
    std::vector<P2pRpcRr*> rrs((size_t)burst);
    std::vector<g_params*> stubs((size_t)burst);
    std::vector<P2pRpcAppRr*> slots((size_t)burst);
    std::vector<volatile uint32_t*> h_states((size_t)burst), d_states((size_t)burst);
    std::vector<SrpcPkt> tx((size_t)burst * resp_frags_);
    std::vector<uint8_t> tx_ok((size_t)burst);
    std::vector<P2pRpcRr*> s_rrs;
    std::vector<g_params*> s_stubs;
    P2pRpcRr* pending = nullptr;  // a ready request that found its replica's ring full
    IdleBackoff backoff;
    bool did_work = true;
    uint64_t last_alive_check = getCurNs();
    while (!quit_.load(std::memory_order_acquire)) {
      if (did_work) backoff.busy();
      else backoff.empty();
      did_work = false;
      // ---- RX half: ready requests -> app ring slots
      int target = -1, nb = 0;
      while (nb < burst) {
        P2pRpcRr* rr = pending ? pending : rr_pool_.get_next_rx_ready_rr();
        if (!rr) break;
        int t = pending ? rr->steer_target : pick_replica();
        if (t >= 0 && replicas_[t]->down.load()) t = pick_replica();  // its replica went down while it waited
        pending = nullptr;
        if (t < 0) {  // every replica is down: drop the request
          release_rr_rx(rr);
          rr_pool_.reap_rr(rr);
          stats_.dropped_pkts++;
          continue;
        }
        rr->steer_target = t;
        if (target >= 0 && t != target) {  // one submission serves one replica
          pending = rr;
          break;
        }
        Replica& rep = *replicas_[t];
        // The next producer slot is bound to ring addresses only once it is free.
        P2pRpcAppRrPool* arp = rep.pool;
        P2pRpcAppRr* slot = arp->get_app_rr((int)arp->producer_index());
        if (__atomic_load_n(slot->h_state, __ATOMIC_ACQUIRE) != APP_RR_STATUS::FREE) {
          rep.stats.ring_full++;
          stats_.ring_full++;
          pending = rr;
          break;
        }
        target = t;
        slot = arp->get_next();
        rrs[nb] = rr;
        stubs[nb] = slot->h_stub;
        slots[nb] = slot;
        h_states[nb] = slot->h_state;
        d_states[nb] = slot->d_state;
        slot->rpc_rr = rr;
        rr->app_rr_idx = slot->rr_idx;
        nb++;
      }
      if (nb > 0) {
        did_work = true;
        NVTX_R("gather");
        Replica& rep = *replicas_[target];
        Inflight fl{rep.engine, 0, {}, rep.remote ? &rep.down : nullptr};
        if (!cfg_.zerocopy) {
          // Transmit buffers first: the serving side reads a slot's response destination as soon as it sees the
          // doorbell, so the destination has to be in place before the gather (which rings the doorbell) is launched.
          for (int i = 0; i < nb; i++) {
            take_rx_slots(rrs[i], &fl.rx_slots);
            tx_ok[i] = port_->alloc_tx(&tx[(size_t)i * resp_frags_], (int)resp_frags_) ? 1 : 0;
            if (!tx_ok[i]) stats_.tx_alloc_fail++;
            uint64_t off = P2pRpcAppRrMemPool::kNoTxOffset;
            if (rep.device_completes && rep.can_push && tx_ok[i] && resp_frags_ == 1) off = port_->tx_arena_offset(tx[(size_t)i * resp_frags_]);
            __atomic_store_n(slots[i]->h_tx_off, off, __ATOMIC_RELEASE);
          }
        }
        int64_t ticket = rep.engine->gather_batch_notify(rrs.data(), stubs.data(), h_states.data(), d_states.data(), nb,
                                                         (uint32_t)APP_RR_STATUS::RX_COMPLETE);
        if (ticket < 0) {
          // Nothing was stored into the slot states.  Hand the slots to the consumer anyway (it will answer with
          // whatever the ring holds) rather than stall the ring: the error is counted and logged by the engine.
          stats_.sg_errors++;
          for (int i = 0; i < nb; i++) __atomic_store_n(h_states[i], (uint32_t)APP_RR_STATUS::RX_COMPLETE, __ATOMIC_RELEASE);
        }
        fl.ticket = ticket;
        if (!cfg_.zerocopy) {
          for (int i = 0; i < nb; i++) {
            if (tx_ok[i]) fill_tx(rrs[i], &tx[(size_t)i * resp_frags_]);
            else rrs[i]->clear_bufs();
          }
          inflight_.push_back(std::move(fl));
        }
        rep.outstanding.fetch_add(nb);
        rep.stats.steered += (uint64_t)nb;
        NVTX_P();
      }
      if (!inflight_.empty()) reap_inflight(false);
      // ---- TX half: finished slots -> responses
      for (auto& rep_ptr : replicas_) {
        Replica& rep = *rep_ptr;
        int nt = 0, n_scatter = 0;
        const int pool_n = rep.pool->get_pool_size();
        while (nt < burst) {
          P2pRpcAppRr* slot = rep.pool->get_app_rr((rep.tx_idx + nt) % pool_n);
          if (__atomic_load_n(slot->h_state, __ATOMIC_ACQUIRE) != APP_RR_STATUS::WORK_COMPLETE) break;
          if (!slot->rpc_rr) break;  // completed without ever being filled: leave it to the worker's accounting
          rrs[nt] = (P2pRpcRr*)slot->rpc_rr;
          stubs[nt] = slot->h_stub;
          slots[nt] = slot;
          nt++;
        }
        if (nt == 0) continue;
        did_work = true;
        NVTX_R("tx");
        if (cfg_.zerocopy) {
          send_zerocopy(rep, rrs.data(), slots.data(), nt);
        } else {
          // Responses that the serving side already stored in the transmit arena only need sending; the others are
          // fetched from the response ring by the engine (for a remote replica: a read over NVLink).
          s_rrs.clear();
          s_stubs.clear();
          for (int i = 0; i < nt; i++) {
            bool pushed = rep.device_completes &&
                          __atomic_load_n(slots[i]->h_tx_off, __ATOMIC_ACQUIRE) != P2pRpcAppRrMemPool::kNoTxOffset;
            if (pushed) {
              rep.stats.pushed++;
              // doorbell rung -> response stored, on the timers of the devices that did it
              const uint64_t t_rx = slots[i]->h_stamps[0], t_done = slots[i]->h_stamps[1];
              const int64_t lat = (int64_t)(t_done - t_rx) - rep.stamp_skew_ns;
              if (t_rx && t_done && lat > 0 && lat < 60000000000ll) {
                std::lock_guard<std::mutex> g(lat_mu_);
                if (device_latency_ns_.size() < ((size_t)1 << 21)) device_latency_ns_.push_back((uint64_t)lat);
              }
            } else {
              s_rrs.push_back(rrs[i]);
              s_stubs.push_back(stubs[i]);
              n_scatter++;
            }
          }
          if (n_scatter > 0) {
            int rc = rep.engine->scatter_batch(s_rrs.data(), s_stubs.data(), n_scatter);
            if (rc != 0) stats_.sg_errors++;
          }
          for (int i = 0; i < nt; i++) send_response(rrs[i]);
        }
        for (int i = 0; i < nt; i++) {
          slots[i]->rpc_rr = nullptr;
          slots[i]->h_stamps[0] = slots[i]->h_stamps[1] = 0;
          __atomic_store_n(slots[i]->h_tx_off, P2pRpcAppRrMemPool::kNoTxOffset, __ATOMIC_RELAXED);
          __atomic_store_n(slots[i]->h_state, (uint32_t)APP_RR_STATUS::FREE, __ATOMIC_RELEASE);
        }
        rep.tx_idx = (rep.tx_idx + nt) % pool_n;
        rep.outstanding.fetch_sub(nt);
        rep.stats.completed += (uint64_t)nt;
        NVTX_P();
      }
      if (!did_work) {
        uint64_t now = getCurNs();
        if (now - last_alive_check > 20000000ull) {
          last_alive_check = now;
          check_remote_replicas();
        }
      }
    }
    reap_inflight(true);
  }

  // Zero-copy replies: the app answered in the receive buffer; build the reply
  // header by swapping the request header in place and send header + the first
  // resp_size bytes of the same buffer back.
  void send_zerocopy(Replica&, P2pRpcRr** rrs, P2pRpcAppRr** slots, int n) {
    for (int i = 0; i < n; i++) {
      P2pRpcRr* rr = rrs[i];
      p2p_rpc_hdr h;
      fill_frag_hdr(&h, &rr->_client_conn_info, rr->req_token, 0, (uint16_t)cfg_.resp_size, true);
      const uint8_t* payload = port_->rx_host_ptr((uint32_t)(rr->transport_mbufs->burst_items[0] - 1));
      uint32_t len = (uint32_t)cfg_.resp_size;
      stats_.tx_pkts += (uint64_t)port_->tx_copy(&h, &payload, &len, 1);
      stats_.tx_resps++;
      release_rr_rx(rr);
      rr_pool_.reap_rr(rr);
      (void)slots;
    }
  }

 public:
  SplitRpcServer(Transport* port, const ServerConfig& cfg)
      : port_(port), cfg_(cfg), rr_pool_(cfg.rr_pool_size), resp_frags_(num_fragments(cfg.resp_size, rpc_mtu())) {
    have_tx_info_ = port_->tx_arena_info(&tx_info_);
    server_conn_ = initialize_src_conn_info(cfg.server_uri);
    rr_pool_.setup_and_init_rr_pool(server_conn_, cfg.req_size);
  }
  ~SplitRpcServer() {
    stop();
    release_conn_info(server_conn_);
  }

  // Adds a local replica: an app instance (its own slot ring) and the engine that
  // fills that ring.  Returns the replica index.
  int add_replica(P2pRpcAppInfo* app, P2pRpcSgEngine* engine) {
    auto r = std::make_unique<Replica>();
    r->app = app;
    r->pool = app->app_rr_pool;
    r->engine = engine;
    r->app_idx = app_server_.register_app(app);
    app->app_rr_pool->init_pool();
    // Completion by the serving side: possible when responses fit one fragment and the app's device can store into
    // the transmit arena (any host arena for a CPU app; a pinned/registered one for a GPU app).
    if (cfg_.device_completion && !cfg_.zerocopy && resp_frags_ == 1 && have_tx_info_) {
      if (app->device_id < 0) {
        app->enable_device_completion((uint64_t)(uintptr_t)tx_info_.host_base, tx_info_.bytes);
        r->device_completes = true;
      } else if (tx_info_.gpu_visible) {
        app->enable_device_completion((uint64_t)(uintptr_t)tx_info_.dev_base, tx_info_.bytes);
        r->device_completes = true;
      }
    }
    {
      P2pRpcAppRrMemPool* mp = app->app_rr_pool->rr_mem_pool;
      engine->set_stamp_layout(mp->get_doorbells_host(), mp->get_stamps_host(), mp->get_doorbells_device(), mp->get_stamps_device());
    }
    replicas_.push_back(std::move(r));
    return (int)replicas_.size() - 1;
  }
  // Adds a replica that is served by a batched server in another process.  The caller keeps `remote` alive.
  int add_remote_replica(NvlRemoteReplica* remote) {
    auto r = std::make_unique<Replica>();
    r->remote = remote;
    r->pool = remote->pool();
    r->engine = remote->engine();
    r->device_completes = remote->device_completes();
    r->stamp_skew_ns = remote->stamp_skew_ns();
    r->can_push = remote->pushes_responses();
    {
      P2pRpcAppRrMemPool* mp = r->pool->rr_mem_pool;
      r->engine->set_stamp_layout(mp->get_doorbells_host(), mp->get_stamps_host(), mp->get_doorbells_device(), mp->get_stamps_device());
    }
    replicas_.push_back(std::move(r));
    return (int)replicas_.size() - 1;
  }
  const TxArenaInfo* tx_arena() const { return have_tx_info_ ? &tx_info_ : nullptr; }
  Transport* port() const { return port_; }
  size_t num_replicas() const { return replicas_.size(); }
  P2pRpcAsyncAppServer& app_server() { return app_server_; }
  P2pRpcRRPool& rr_pool() { return rr_pool_; }
  void mark_replica_down(int idx, bool down) { replicas_[idx]->down.store(down); }

  void start() {
    if (running_.exchange(true)) return;
    quit_.store(false);
    app_server_.reset_quit();
    for (auto& rp : replicas_) {
      Replica* r = rp.get();
      if (!r->app) continue;  // remote replicas run their own worker
      r->app->app_ctx->curr_batch_size = cfg_.max_batch;
      r->app->app_ctx->next_batch_size = cfg_.max_batch;
      r->worker = std::thread([this, r] {
        switch (cfg_.server_mode) {
          case 1: app_server_.async_worker_loop(r->app_idx); break;
          case 2: app_server_.dynamic_batching_sync_worker_loop(r->app_idx, cfg_.max_batch); break;
          default: app_server_.sync_worker_loop(r->app_idx); break;
        }
      });
    }
    rx_thread_ = std::thread([this] { rx_loop(); });
    shunter_thread_ = std::thread([this] { shunter_loop(); });
  }

  void stop() {
    if (!running_.exchange(false)) return;
    quit_.store(true, std::memory_order_release);
    app_server_.quit();
    if (rx_thread_.joinable()) rx_thread_.join();
    if (shunter_thread_.joinable()) shunter_thread_.join();
    for (auto& rp : replicas_)
      if (rp->worker.joinable()) rp->worker.join();
  }

  ServerStats stats() {
    ServerStats s;
    s.rx_pkts = stats_.rx_pkts; s.rx_reqs = stats_.rx_reqs; s.tx_resps = stats_.tx_resps; s.tx_pkts = stats_.tx_pkts;
    s.dropped_pkts = stats_.dropped_pkts; s.expired = stats_.expired; s.ring_full = stats_.ring_full;
    s.tx_alloc_fail = stats_.tx_alloc_fail; s.sg_errors = stats_.sg_errors; s.replicas_lost = stats_.replicas_lost;
    for (auto& rp : replicas_) {
      ReplicaStats r;
      r.steered = rp->stats.steered.load(std::memory_order_relaxed);
      r.completed = rp->stats.completed.load(std::memory_order_relaxed);
      r.ring_full = rp->stats.ring_full.load(std::memory_order_relaxed);
      r.pushed = rp->stats.pushed.load(std::memory_order_relaxed);
      s.replicas.push_back(r);
    }
    return s;
  }
  // Device-timed service latency of the responses that the serving side pushed: from the moment the gather rang the
  // slot's doorbell to the moment the response was stored, both stamped by the GPUs (or CPU threads) that did it.
  std::vector<uint64_t> device_latency_ns() {
    std::lock_guard<std::mutex> g(lat_mu_);
    return device_latency_ns_;
  }
  void clear_device_latency() {
    std::lock_guard<std::mutex> g(lat_mu_);
    device_latency_ns_.clear();
  }
  WorkerStats worker_stats(int replica) {
    Replica& r = *replicas_[replica];
    if (r.app) return app_server_.stats(r.app_idx);
    WorkerStats w;  // remote: ask its server
    if (r.remote) r.remote->query_stats(&w.num_req, &w.num_batches);
    return w;
  }
};
