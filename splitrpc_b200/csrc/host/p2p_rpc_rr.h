// Transport-side request/response records and their pools.
//
// A P2pRpcRr tracks one in-flight RPC on the network side of the server: the
// client's token and reply template, and per fragment the transport buffer, the
// header pointer and the payload pointer/length, indexed by sequence number
// (reference src/p2p_rpc_rr_ng.h:13-127).  P2pRpcRRPool owns the records: a
// token -> record map used only by the receive thread, and three MPMC rings
// (free, rx_ready, tx_ready) that hand records between the receive, shunter and
// transmit stages (reference src/p2p_rpc_rr_pool_ng.h:12-188).
//
// Added over the original: every record stamps its first-fragment time so that
// expire_stale() can reclaim requests that lost a fragment instead of leaking
// them, duplicate fragments are detected, and pool exhaustion grows the pool or
// reports failure instead of exiting the process.
#pragma once

#include <functional>
#include <unordered_map>
#include <vector>

#include "mpmc_ring.h"
#include "p2p_rpc.h"

enum P2P_RPC_RR_STATES { RR_CREATE, RR_PROCESS, RR_READY, RR_FINISH, RR_UNUSED };

class P2pRpcRr {
 public:
  uint64_t req_token = 0;
  size_t payload_size = 0;      // bytes received so far (request) or to send (response)
  size_t max_payload_size = 0;  // fixed request size of the app
  p2p_rpc_conn_info _client_conn_info{};
  uint32_t rr_state = RR_CREATE;
  uint64_t first_frag_ns = 0;
  int steer_target = 0;         // replica chosen by flow steering
  int app_rr_idx = -1;          // slot of the app ring this request was placed in

  p2p_hbufs* transport_mbufs;   // opaque transport buffer handles
  p2p_hbufs* hdr_bufs;          // header pointers
  p2p_bufs* payload_bufs;       // payload pointers + sizes
  p2p_sk_buf* payload_sk_bufs;  // coalesced copy list built by the SG engine

  explicit P2pRpcRr(const p2p_rpc_conn_info* tmpl = nullptr, size_t max_payload = 0)
      : max_payload_size(max_payload),
        transport_mbufs(new p2p_hbufs()),
        hdr_bufs(new p2p_hbufs()),
        payload_bufs(new p2p_bufs()),
        payload_sk_bufs(new p2p_sk_buf()) {
    if (tmpl) _client_conn_info = *tmpl;
    clear_bufs();
  }
  ~P2pRpcRr() {
    delete transport_mbufs;
    delete hdr_bufs;
    delete payload_bufs;
    delete payload_sk_bufs;
  }
  P2pRpcRr(const P2pRpcRr&) = delete;
  P2pRpcRr& operator=(const P2pRpcRr&) = delete;

  void clear_bufs() {
    // Entries that were in use go back to zero, so that an index nobody filled can never be read as a stale
    // pointer or length.
    for (uint16_t i = 0; i < transport_mbufs->num_items; i++) transport_mbufs->burst_items[i] = 0;
    for (uint16_t i = 0; i < hdr_bufs->num_items; i++) hdr_bufs->burst_items[i] = 0;
    for (uint16_t i = 0; i < payload_bufs->num_items; i++) {
      payload_bufs->burst_items[i] = 0;
      payload_bufs->item_size[i] = 0;
    }
    n_frags_ = 0;
    transport_mbufs->num_items = 0;
    hdr_bufs->num_items = 0;
    payload_bufs->num_items = 0;
    payload_sk_bufs->num_items = 0;
    payload_size = 0;
    seen_.assign(seen_.size(), 0);
  }

  void reset() {
    clear_bufs();
    req_token = 0;
    rr_state = RR_CREATE;
    first_frag_ns = 0;
    app_rr_idx = -1;
  }

  // Appends a buffer at the next index (used when building a response).
  void rr_append_mbuf(uintptr_t mbuf, uintptr_t hdr, uintptr_t payload, size_t size) {
    place(mbuf, hdr, payload, size, transport_mbufs->num_items);
    payload_size += size;
  }

  // Places a received fragment at its sequence number.  Returns false (and leaves
  // the record untouched) for an out-of-range or repeated sequence number and for
  // an empty fragment of a non-empty request.
  bool rr_emplace_mbuf(uintptr_t mbuf, uintptr_t hdr, uintptr_t payload, size_t size, int seq_num) {
    if (seq_num < 0 || seq_num >= MAX_BI_SIZE) return false;
    if (size == 0 && max_payload_size > 0) return false;
    if ((size_t)seq_num >= seen_.size()) seen_.resize((size_t)seq_num + 1, 0);
    if (seen_[seq_num]) return false;
    seen_[seq_num] = 1;
    place(mbuf, hdr, payload, size, (uint16_t)seq_num);
    payload_size += size;
    n_frags_++;
    return true;
  }

  // Ready = every byte of the fixed-size request has arrived AND the fragments
  // fill indices 0..n-1 without a hole.  The byte count alone is not enough: a
  // fragment with a skipped sequence number raises num_items past an index that
  // nobody filled, and a copy list built from that index would be garbage.
  bool is_rr_ready() const { return payload_size == max_payload_size && n_frags_ == payload_bufs->num_items; }
  // All the bytes are there (or more) but the sequence numbers leave a hole: the
  // sender broke the framing rule and the record can never become ready.
  bool is_rr_malformed() const {
    return payload_size > max_payload_size || (payload_size == max_payload_size && n_frags_ != payload_bufs->num_items);
  }

  void rr_print_bufs() const {
    std::printf("rr %p token=%lu: %u fragments, %zu/%zu bytes\n", (const void*)this, (unsigned long)req_token,
                (unsigned)payload_bufs->num_items, payload_size, max_payload_size);
    print_bufs(payload_bufs);
  }

 private:
  std::vector<uint8_t> seen_;
  uint16_t n_frags_ = 0;  // distinct fragments accepted since clear_bufs()
  void place(uintptr_t mbuf, uintptr_t hdr, uintptr_t payload, size_t size, uint16_t idx) {
    transport_mbufs->burst_items[idx] = mbuf;
    hdr_bufs->burst_items[idx] = hdr;
    payload_bufs->burst_items[idx] = payload;
    payload_bufs->item_size[idx] = size;
    uint16_t n = (uint16_t)(idx + 1);
    if (transport_mbufs->num_items < n) transport_mbufs->num_items = n;
    if (hdr_bufs->num_items < n) hdr_bufs->num_items = n;
    if (payload_bufs->num_items < n) payload_bufs->num_items = n;
  }
};

static inline P2pRpcRr* rr_clone_alloc(const P2pRpcRr* rr) {
  return new P2pRpcRr(&rr->_client_conn_info, rr->max_payload_size);
}

struct RrPoolCounters {
  uint64_t allocated = 0, grown = 0, dropped_zero_token = 0, dropped_bad_seq = 0, dropped_dup = 0, expired = 0,
           rx_ready = 0, reaped = 0;
};

class P2pRpcRRPool {
 public:
  static constexpr int kDefaultPoolSize = 4095;

  explicit P2pRpcRRPool(int pool_size = kDefaultPoolSize)
      : pool_size_(pool_size), free_(ring_cap(pool_size)), rx_ready_(ring_cap(pool_size)), tx_ready_(ring_cap(pool_size)) {}

  ~P2pRpcRRPool() {
    if (!cache_.empty())
      srpc_log(SRPC_LOG_WARN, "rr pool destroyed with %zu partially received requests", cache_.size());
    for (P2pRpcRr* r : all_) delete r;
  }

  // Creates the records; every record starts as a copy of the server's header
  // template and expects `req_size` payload bytes.
  void setup_and_init_rr_pool(const p2p_rpc_conn_info* server_conn, size_t req_size) {
    if (server_conn) server_conn_ = *server_conn;
    req_size_ = req_size;
    for (int i = 0; i < pool_size_; i++) add_record();
  }

  size_t get_req_size() const { return req_size_; }
  size_t num_partial() const { return cache_.size(); }
  size_t num_free() const { return free_.size(); }
  const RrPoolCounters& counters() const { return ctr_; }

  // Receive-thread only.  Finds the record of the header's token or takes a free
  // one; returns nullptr for token 0 (protocol: such packets are dropped).
  P2pRpcRr* get_rr(p2p_rpc_hdr* hdr) {
    uint64_t token = hdr->req_token;
    if (token == 0) {
      ctr_.dropped_zero_token++;
      return nullptr;
    }
    // The fragments of a request mostly arrive back to back: remember the last record and skip the hash lookup.
    if (last_rr_ && last_token_ == token) return last_rr_;
    auto it = cache_.find(token);
    if (it != cache_.end()) {
      last_token_ = token;
      last_rr_ = it->second;
      return it->second;
    }
    P2pRpcRr* rr = alloc_rr();
    if (!rr) return nullptr;
    rr->req_token = token;
    rr->rr_state = RR_PROCESS;
    rr->first_frag_ns = getCurNs();
    set_conn_info(&rr->_client_conn_info, hdr);
    cache_.emplace(token, rr);
    last_token_ = token;
    last_rr_ = rr;
    return rr;
  }

  // Receive-thread only.  Looks up/creates the record and places one fragment.
  // Returns the record when the fragment was accepted, nullptr when dropped.
  P2pRpcRr* append_to_rr(p2p_rpc_hdr* hdr, uintptr_t mbuf, uintptr_t payload, size_t len) {
    if (hdr->seq_num >= MAX_BI_SIZE) {
      ctr_.dropped_bad_seq++;
      return nullptr;
    }
    P2pRpcRr* rr = get_rr(hdr);
    if (!rr) return nullptr;
    if (!rr->rr_emplace_mbuf(mbuf, (uintptr_t)hdr, payload, len, hdr->seq_num)) {
      ctr_.dropped_dup++;
      return nullptr;
    }
    return rr;
  }

  void mark_rx_ready_rr(P2pRpcRr* rr) {
    forget(rr);
    cache_.erase(rr->req_token);
    rr->rr_state = RR_READY;
    ctr_.rx_ready++;
    while (!rx_ready_.push(rr)) cpu_relax();
  }
  P2pRpcRr* get_next_rx_ready_rr() {
    P2pRpcRr* rr = nullptr;
    return rx_ready_.pop(rr) ? rr : nullptr;
  }
  // The original's spellings of the two dequeues (reference src/p2p_rpc_rr_pool_ng.h:163-187) and of the record list.
  P2pRpcRr* consume_rx_ready_rr() { return get_next_rx_ready_rr(); }
  int get_next_rx_ready_rr(P2pRpcRr** next_rr) {
    *next_rr = get_next_rx_ready_rr();
    return *next_rr ? 1 : 0;
  }
  P2pRpcRr* consume_tx_ready_rr() { return get_next_tx_ready_rr(); }
  std::vector<P2pRpcRr*>& get_rr_pool_container() { return all_; }
  P2pRpcRr** get_rr_pool() { return all_.data(); }
  int get_pool_size() const { return pool_size_; }
  void mark_tx_ready_rr(P2pRpcRr* rr) {
    rr->rr_state = RR_FINISH;
    while (!tx_ready_.push(rr)) cpu_relax();
  }
  P2pRpcRr* get_next_tx_ready_rr() {
    P2pRpcRr* rr = nullptr;
    return tx_ready_.pop(rr) ? rr : nullptr;
  }

  // Takes a record that is not tied to a token (client side, response building).
  P2pRpcRr* alloc_rr() {
    P2pRpcRr* rr = nullptr;
    if (free_.pop(rr)) return rr;
    std::lock_guard<std::mutex> g(grow_mu_);
    if (free_.pop(rr)) return rr;
    if ((int)all_.size() >= max_records_) return nullptr;
    ctr_.grown++;
    return add_record(false);
  }

  // Returns a finished record to the free ring.
  void reap_rr(P2pRpcRr* rr) {
    rr->reset();
    rr->_client_conn_info = server_conn_;
    ctr_.reaped++;
    while (!free_.push(rr)) cpu_relax();
  }

  // Receive-thread only.  Reclaims requests whose first fragment is older than
  // `timeout_ns`; `release` is called once per reclaimed record so the transport
  // can free the fragments it still holds.
  size_t expire_stale(uint64_t now_ns, uint64_t timeout_ns, const std::function<void(P2pRpcRr*)>& release) {
    size_t n = 0;
    for (auto it = cache_.begin(); it != cache_.end();) {
      P2pRpcRr* rr = it->second;
      if (now_ns - rr->first_frag_ns > timeout_ns) {
        forget(rr);
        if (release) release(rr);
        it = cache_.erase(it);
        reap_rr(rr);
        ctr_.expired++;
        n++;
      } else {
        ++it;
      }
    }
    return n;
  }

  // Receive-thread only.  Forgets a partially received request.
  void drop_partial(P2pRpcRr* rr) {
    forget(rr);
    cache_.erase(rr->req_token);
    reap_rr(rr);
  }

  void set_max_records(int n) { max_records_ = n < (1 << 16) ? n : (1 << 16); }

  static inline void cpu_relax() {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }

 private:
  // Rings hold every record the pool may ever own (max_records_ <= 65536).
  static size_t ring_cap(int pool) { (void)pool; return (size_t)1 << 17; }
  P2pRpcRr* add_record(bool to_free = true) {
    P2pRpcRr* rr = new P2pRpcRr(&server_conn_, req_size_);
    all_.push_back(rr);
    ctr_.allocated++;
    if (to_free) free_.push(rr);
    return rr;
  }

  void forget(const P2pRpcRr* rr) {
    if (last_rr_ == rr) last_rr_ = nullptr;
  }
  uint64_t last_token_ = 0;       // receive thread only: the record the previous fragment belonged to
  P2pRpcRr* last_rr_ = nullptr;
  int pool_size_;
  int max_records_ = 1 << 16;
  size_t req_size_ = 0;
  p2p_rpc_conn_info server_conn_{};
  std::vector<P2pRpcRr*> all_;
  std::unordered_map<uint64_t, P2pRpcRr*> cache_;
  MpmcRing<P2pRpcRr*> free_, rx_ready_, tx_ready_;
  std::mutex grow_mu_;
  RrPoolCounters ctr_;
};
