// Public types of the original's client-side and socket-side API, kept so that code written against them compiles
// against this library: the typed buffer pool, the first-generation request/response record with its pool, and the
// kernel-UDP record with its pool.  They are thin: storage and queues come from this library's own pieces (mapped
// pinned memory instead of gdrcopy, MpmcRing instead of DPDK rings / moodycamel queues), every loop is bounded and the
// pools are safe to use from several threads where the originals note that they are not.
//
//   BufItemPool<T>            reference src/p2p_buf_pool.h:12-78
//   p2p_rpc_rr + rr_* helpers reference src/p2p_rpc_rr.h:13-223
//   p2p_rpc_v1::P2pRpcRRPool  reference src/p2p_rpc_rr_pool.h:54-184 (same class name as the current pool in the
//                             original, which keeps the two in different headers; here the older one has a namespace)
//   UdpRpcHdr, UdpRr, UdpRrPool   reference src/udp_rr.h:23-446
#pragma once

#include <netinet/in.h>
#include <unistd.h>
#include <sys/time.h>
#include <sys/socket.h>
#include <arpa/inet.h>
#include <limits>
#include <random>

#include <atomic>
#include <memory>
#include <chrono>
#include <ctime>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "mpmc_ring.h"
#include "p2p_rpc.h"
#include "p2p_rpc_app.h"
#include "p2p_rpc_async_app_server.h"

// ------------------------------------------------------------------ typed buffer pool
// type -1: plain host memory.  type >= 0: memory that both the CPU and GPU `type` address (the original maps GPU
// memory into the CPU with gdrcopy; here it is mapped pinned host memory, which serves the same purpose for stubs and
// doorbells).  get_dev_ptr() returns the device-side address of a pool (the host address for host pools).
template <class T>
class BufItemPool {
  struct Info {
    T* dev = nullptr;
    size_t num = 0;
    bool mapped = false;
  };
  static std::unordered_map<T*, Info>& table() {
    static std::unordered_map<T*, Info> t;
    return t;
  }
  static std::mutex& mu() {
    static std::mutex m;
    return m;
  }

 public:
  static T* create_buf_item_pool(int num, int type = -1) {
    if (num <= 0) return nullptr;
    Info info;
    info.num = (size_t)num;
    T* h = nullptr;
    if (type >= 0) {
      const SrpcDeviceOps* ops = srpc_cuda_ops();
      void *hp = nullptr, *dp = nullptr;
      if (!ops || ops->set_device(type) != 0 || ops->host_alloc_mapped(sizeof(T) * (size_t)num, &hp, &dp) != 0) return nullptr;
      h = static_cast<T*>(hp);
      info.dev = static_cast<T*>(dp);
      info.mapped = true;
    } else {
      void* p = nullptr;
      if (posix_memalign(&p, 64, sizeof(T) * (size_t)num) != 0) return nullptr;
      h = static_cast<T*>(p);
      info.dev = h;
    }
    std::memset((void*)h, 0, sizeof(T) * (size_t)num);
    std::lock_guard<std::mutex> g(mu());
    table()[h] = info;
    return h;
  }
  static void delete_buf_item_pool(T* h, int type = -1) {
    (void)type;
    Info info;
    {
      std::lock_guard<std::mutex> g(mu());
      auto it = table().find(h);
      if (it == table().end()) return;
      info = it->second;
      table().erase(it);
    }
    if (info.mapped) {
      if (const SrpcDeviceOps* ops = srpc_cuda_ops()) ops->host_free(h);
    } else {
      free((void*)h);
    }
  }
  static T* get_dev_ptr(T* h) {
    std::lock_guard<std::mutex> g(mu());
    auto it = table().find(h);
    return it == table().end() ? nullptr : it->second.dev;
  }
};

// ------------------------------------------------------------------ helper names of the original
// (reference src/utils/config_utils.h:34-40,83-96, src/utils/time_utils.h:42-47,72-78, src/p2p_rpc_app_rr_mem_pool.h:29)
static inline std::string getBasePath() { return get_p2p_path(); }
static inline std::string getDatasetBasePath() { return get_dataset_path(); }
static inline size_t get_rpc_mtu() { return rpc_mtu(); }
static inline int16_t is_zerocopy_mode() { return (int16_t)get_zerocopy_mode(); }
// wall-clock time in ns with microsecond resolution (getCurNs is the monotonic clock)
static inline uint64_t getAbsCurNs() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::system_clock::now().time_since_epoch()).count() *
         1000ull;
}
static inline std::string getCurTsAsString() {
  const std::time_t t = std::time(nullptr);
  std::tm tm{};
  localtime_r(&t, &tm);
  char buf[64];
  std::strftime(buf, sizeof(buf), "%d-%m-%Y %H-%M-%S", &tm);
  return buf;
}
// The original keeps a second ring-memory class without the double mapping; here the double mapping is a property of
// the ring allocation inside the one class (and absent where the platform cannot provide it).
using P2pRpcAppRrSimpleMemPool = P2pRpcAppRrMemPool;

// ------------------------------------------------------------------ first-generation record
enum RR_STATUS : uint32_t { RR_V1_UNUSED = 0, RR_V1_INUSE = 1 };

struct p2p_rpc_rr {
  uint64_t req_token = 0;
  uint8_t *req_payload = nullptr, *resp_payload = nullptr;
  size_t req_size = 0, resp_size = 0;
  size_t max_req_size = 0, max_resp_size = 0;
  int req_device_id = -2, resp_device_id = -2;
  volatile uint32_t* state = nullptr;
  uint32_t rr_state = RR_V1_UNUSED;
  p2p_rpc_conn_info _client_conn_info{};
  p2p_hbufs* transport_mbufs = nullptr;
  p2p_hbufs* hdr_bufs = nullptr;
  p2p_bufs* payload_bufs = nullptr;
  p2p_sk_buf* payload_sk_bufs = nullptr;
};

static inline p2p_rpc_rr* rr_base_alloc() {
  p2p_rpc_rr* rr = new p2p_rpc_rr;
  rr->transport_mbufs = new p2p_hbufs();
  rr->hdr_bufs = new p2p_hbufs();
  rr->payload_bufs = new p2p_bufs();
  rr->payload_sk_bufs = new p2p_sk_buf();
  return rr;
}
static inline void rr_base_free(p2p_rpc_rr* rr) {
  if (!rr) return;
  delete rr->transport_mbufs;
  delete rr->hdr_bufs;
  delete rr->payload_bufs;
  delete rr->payload_sk_bufs;
  delete rr;
}
static inline p2p_rpc_rr* rr_proto_alloc(const p2p_rpc_conn_info* conn, size_t req_size, size_t resp_size) {
  p2p_rpc_rr* rr = rr_base_alloc();
  rr->max_req_size = req_size;
  rr->max_resp_size = resp_size;
  if (conn) rr->_client_conn_info = *conn;
  return rr;
}
static inline p2p_rpc_rr* rr_clone_alloc(const p2p_rpc_rr* src) {
  p2p_rpc_rr* rr = rr_proto_alloc(&src->_client_conn_info, src->max_req_size, src->max_resp_size);
  rr->req_device_id = src->req_device_id;
  rr->resp_device_id = src->resp_device_id;
  return rr;
}
// Places one buffer at index `idx` of the record's three parallel lists.  Out-of-range indices are ignored.
static inline void rr_merge_mbuf(p2p_rpc_rr* rr, uintptr_t transport_mbuf, uintptr_t hdr_buf, uintptr_t payload_buf, size_t item_size,
                                 int idx) {
  if (idx < 0 || idx >= MAX_BI_SIZE) return;
  rr->transport_mbufs->burst_items[idx] = transport_mbuf;
  rr->hdr_bufs->burst_items[idx] = hdr_buf;
  rr->payload_bufs->burst_items[idx] = payload_buf;
  rr->payload_bufs->item_size[idx] = item_size;
  const uint16_t n = (uint16_t)(idx + 1);
  if (rr->transport_mbufs->num_items < n) rr->transport_mbufs->num_items = n;
  if (rr->hdr_bufs->num_items < n) rr->hdr_bufs->num_items = n;
  if (rr->payload_bufs->num_items < n) rr->payload_bufs->num_items = n;
}
static inline void rr_append_req_mbuf(p2p_rpc_rr* rr, uintptr_t m, uintptr_t h, uintptr_t p, size_t sz) {
  rr->req_size += sz;
  rr_merge_mbuf(rr, m, h, p, sz, rr->transport_mbufs->num_items);
}
static inline void rr_append_resp_mbuf(p2p_rpc_rr* rr, uintptr_t m, uintptr_t h, uintptr_t p, size_t sz) {
  rr->resp_size += sz;
  rr_merge_mbuf(rr, m, h, p, sz, rr->transport_mbufs->num_items);
}
static inline void rr_merge_req_mbuf(p2p_rpc_rr* rr, uintptr_t m, uintptr_t h, uintptr_t p, size_t sz, int seq_num) {
  rr->req_size += sz;
  rr_merge_mbuf(rr, m, h, p, sz, seq_num);
}
static inline void rr_merge_resp_mbuf(p2p_rpc_rr* rr, uintptr_t m, uintptr_t h, uintptr_t p, size_t sz, int seq_num) {
  rr->resp_size += sz;
  rr_merge_mbuf(rr, m, h, p, sz, seq_num);
}
static inline void rr_clear_bufs(p2p_rpc_rr* rr) {
  rr->transport_mbufs->num_items = rr->hdr_bufs->num_items = rr->payload_bufs->num_items = 0;
  rr->payload_sk_bufs->num_items = 0;
  rr->req_size = rr->resp_size = 0;
}
static inline void rr_print_bufs(const p2p_rpc_rr* rr) {
  std::printf("rr %p token=%lu: %u buffers\n", (const void*)rr, (unsigned long)rr->req_token, (unsigned)rr->payload_bufs->num_items);
  print_bufs(rr->payload_bufs);
}

// Payload memory by device id, with the original's names (reference src/p2p_rpc_rr_pool.h:15-50): -1 host memory,
// >= 0 memory that GPU addresses too (mapped pinned), anything else none.
static inline uint8_t* alloc_cpu_mem(size_t mem_size) { return mem_size ? BufItemPool<uint8_t>::create_buf_item_pool((int)mem_size, -1) : nullptr; }
static inline void free_cpu_mem(uint8_t* mem) {
  if (mem) BufItemPool<uint8_t>::delete_buf_item_pool(mem);
}
static inline uint8_t* alloc_mem(size_t mem_size, int device_id) {
  if (device_id < -1 || mem_size == 0) return nullptr;
  return BufItemPool<uint8_t>::create_buf_item_pool((int)mem_size, device_id);
}
static inline void free_mem(uint8_t* mem, int device_id) {
  if (mem && device_id >= -1) BufItemPool<uint8_t>::delete_buf_item_pool(mem);
}

namespace p2p_rpc_v1 {

// Pool of first-generation records that also owns each record's request and response payload memory: host memory
// (device id -1), memory a GPU can address (device id >= 0, mapped pinned) or none (-2).
class P2pRpcRRPool {
  int pool_size_;
  std::unordered_map<uint64_t, p2p_rpc_rr*> rr_cache_;
  MpmcRing<p2p_rpc_rr*> free_;
  std::vector<p2p_rpc_rr*> rr_pool_;
  std::mutex mu_;

  // A record with its own request and response memory on the named devices.
  static p2p_rpc_rr* alloc_new_rr(const p2p_rpc_conn_info* src_conn_info, size_t req_size, size_t resp_size, int req_device_id = -2,
                                  int resp_device_id = -2) {
    p2p_rpc_rr* rr = rr_proto_alloc(src_conn_info, req_size, resp_size);
    rr->req_payload = alloc_mem(req_size, req_device_id);
    rr->resp_payload = alloc_mem(resp_size, resp_device_id);
    rr->req_device_id = req_device_id;
    rr->resp_device_id = resp_device_id;
    return rr;
  }

 public:
  explicit P2pRpcRRPool(int pool_size = 1023) : pool_size_(pool_size), free_((size_t)1 << 12) {}
  ~P2pRpcRRPool() {
    for (p2p_rpc_rr* rr : rr_pool_) {
      if (rr->req_payload) BufItemPool<uint8_t>::delete_buf_item_pool(rr->req_payload);
      if (rr->resp_payload) BufItemPool<uint8_t>::delete_buf_item_pool(rr->resp_payload);
      rr_base_free(rr);
    }
  }
  int get_pool_size() const { return pool_size_; }
  std::vector<p2p_rpc_rr*>& get_rr_pool() { return rr_pool_; }
  std::vector<p2p_rpc_rr*>& get_rr_pool_container() { return rr_pool_; }

  void setup_and_init_rr_pool(const p2p_rpc_conn_info* src_conn_info, size_t req_size, size_t resp_size, int device_id) {
    for (int i = 0; i < pool_size_; i++) {
      p2p_rpc_rr* rr = alloc_new_rr(src_conn_info, req_size, resp_size, device_id, device_id);
      rr_pool_.push_back(rr);
      free_.push(rr);
    }
  }
  // Record of the header's token; a new one is taken from the free ring.  nullptr when the pool is exhausted.
  p2p_rpc_rr* get_rr(p2p_rpc_hdr* rpc_hdr) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = rr_cache_.find(rpc_hdr->req_token);
    if (it != rr_cache_.end()) return it->second;
    p2p_rpc_rr* rr = nullptr;
    if (!free_.pop(rr)) return nullptr;
    rr->req_token = rpc_hdr->req_token;
    rr->rr_state = RR_V1_INUSE;
    set_conn_info(&rr->_client_conn_info, rpc_hdr);
    rr_cache_[rr->req_token] = rr;
    return rr;
  }
  p2p_rpc_rr* consume_rr() {
    p2p_rpc_rr* rr = nullptr;
    if (!free_.pop(rr)) return nullptr;
    rr->rr_state = RR_V1_INUSE;
    return rr;
  }
  void reap_rr(p2p_rpc_rr* rr) {
    {
      std::lock_guard<std::mutex> g(mu_);
      rr_cache_.erase(rr->req_token);
    }
    rr_clear_bufs(rr);
    rr->req_token = 0;
    rr->rr_state = RR_V1_UNUSED;
    free_.push(rr);
  }
  size_t num_free() const { return free_.size(); }
};

// First-generation synchronous app server (reference src/p2p_rpc_app_server.h:31-284): records are submitted on a
// ring; one worker per app instance takes a record, points the instance's stub at the record's request and response
// buffers, runs the app, waits for it, and hands the record to the completion ring that the owner registered.  Each
// instance is a P2pRpcAppInfo (stub, doorbell, stream), so the callbacks are the same ones the current server takes.
class P2pRpcAppServer {
 public:
  using Ring = MpmcRing<p2p_rpc_rr*>;
  P2pRpcAppServer(AppInitCB init, AppRunCB run, AppCleanupCB cleanup, AppCompleteCB complete, int num_instances, int device_id,
                  size_t req_size, size_t resp_size, size_t queue_len = 1024, void* internal = nullptr)
      : sub_queue_(queue_len) {
    for (int i = 0; i < (num_instances < 1 ? 1 : num_instances); i++)
      apps_.emplace_back(new P2pRpcAppInfo(init, run, cleanup, complete, device_id, req_size, resp_size, 1, internal, 1, 1));
  }
  ~P2pRpcAppServer() { stop(); }
  bool init_ok() const {
    for (auto& a : apps_)
      if (!a->init_ok) return false;
    return true;
  }
  int num_instances() const { return (int)apps_.size(); }
  void register_cq(Ring* cq) { cq_ = cq; }
  bool enqueue_work(p2p_rpc_rr* rr) { return sub_queue_.push(rr); }

  // Points the instance's stub at the record and starts the app; does not wait.
  void do_work(p2p_rpc_rr* rr, int instance = 0) {
    P2pRpcAppInfo* a = apps_[instance].get();
    a->app_ctx->h_stub->req = rr->req_payload;
    a->app_ctx->h_stub->resp = rr->resp_payload;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    a->stage_window(0, 1, false);
    a->app_run(a->app_ctx);
  }
  bool sync(int instance = 0) {
    P2pRpcAppInfo* a = apps_[instance].get();
    bool ok = a->app_ctx->WaitForAppRunComplete();
    if (a->app_complete) a->app_complete(a->app_ctx);
    return ok;
  }
  bool do_work_sync(p2p_rpc_rr* rr, int instance = 0) {
    do_work(rr, instance);
    return sync(instance);
  }

  void start() {
    if (!workers_.empty()) return;
    stop_.store(false);
    for (int i = 0; i < num_instances(); i++) workers_.emplace_back([this, i] { rpc_handler(i); });
  }
  void stop() {
    stop_.store(true);
    for (auto& t : workers_)
      if (t.joinable()) t.join();
    workers_.clear();
  }
  // The worker loop of one instance on the caller's thread, until stop() (the original's name for it; start() runs one
  // per instance on threads of its own).
  void HandleRpcs(int instance = 0) {
    stop_.store(false);
    rpc_handler(instance);
  }
  uint64_t num_serviced() const { return serviced_.load(); }
  uint64_t num_failed() const { return failed_.load(); }

 private:
  void rpc_handler(int instance) {
    IdleBackoff backoff;
    p2p_rpc_rr* rr = nullptr;
    while (!stop_.load(std::memory_order_acquire)) {
      if (!sub_queue_.pop(rr)) {
        backoff.empty();
        continue;
      }
      backoff.busy();
      if (!do_work_sync(rr, instance)) failed_.fetch_add(1);
      serviced_.fetch_add(1);
      if (cq_)
        while (!cq_->push(rr) && !stop_.load(std::memory_order_acquire)) std::this_thread::yield();
    }
  }
  std::vector<std::unique_ptr<P2pRpcAppInfo>> apps_;
  Ring sub_queue_;
  Ring* cq_ = nullptr;
  std::vector<std::thread> workers_;
  std::atomic<bool> stop_{false};
  std::atomic<uint64_t> serviced_{0}, failed_{0};
};

}  // namespace p2p_rpc_v1

// ------------------------------------------------------------------ kernel-UDP records
// UdpRpcHdr, the datagram header of the socket path, is defined with the wire format (p2p_rpc.h).
static constexpr size_t UDP_RPC_HEADER_LEN = sizeof(UdpRpcHdr);
static inline uint64_t get_req_token(const UdpRpcHdr* h) { return h->req_token; }
static inline uint16_t get_seq_num(const UdpRpcHdr* h) { return h->seq_num; }

enum UDP_RR_STATES : uint32_t { UDP_RR_CREATE, UDP_RR_PROCESS, UDP_RR_READY, UDP_RR_FINISH, UDP_RR_UNUSED };

// One RPC on the socket path.  A request or response is held twice: as one contiguous payload and as a list of
// datagram buffers (header + up to MTU payload bytes each); req_to_bufs / bufs_to_req and resp_to_bufs / bufs_to_resp
// convert between the two.
class UdpRr {
  static void alloc_bufs(p2p_bufs* b, size_t total) {
    const size_t mtu = rpc_mtu();
    size_t n = num_fragments(total, mtu), left = total;
    if (n > MAX_BI_SIZE) n = MAX_BI_SIZE;
    b->num_items = (uint16_t)n;
    for (size_t i = 0; i < n; i++) {
      size_t len = left < mtu ? left : mtu;
      left -= len;
      b->burst_items[i] = (uintptr_t) new uint8_t[UDP_RPC_HEADER_LEN + len];
      b->item_size[i] = UDP_RPC_HEADER_LEN + len;
    }
  }
  static void release_bufs(p2p_bufs* b) {
    for (size_t i = 0; i < b->num_items; i++) delete[] (uint8_t*)b->burst_items[i];
    b->num_items = 0;
  }
  static size_t payload_to_bufs(const uint8_t* payload, size_t size, p2p_bufs* b, uint64_t token) {
    size_t off = 0;
    for (size_t i = 0; i < b->num_items && off < size; i++) {
      uint8_t* buf = (uint8_t*)b->burst_items[i];
      UdpRpcHdr* h = (UdpRpcHdr*)buf;
      std::memset(h, 0, sizeof(*h));
      h->req_token = token;
      h->seq_num = (uint16_t)i;
      size_t len = b->item_size[i] - UDP_RPC_HEADER_LEN;
      if (len > size - off) len = size - off;
      std::memcpy(buf + UDP_RPC_HEADER_LEN, payload + off, len);
      off += len;
    }
    return off;
  }
  static size_t bufs_to_payload(const p2p_bufs* b, uint8_t* payload, size_t cap) {
    size_t off = 0;
    for (size_t i = 0; i < b->num_items; i++) {
      size_t len = b->item_size[i] - UDP_RPC_HEADER_LEN;
      if (off + len > cap) len = cap - off;
      std::memcpy(payload + off, (const uint8_t*)b->burst_items[i] + UDP_RPC_HEADER_LEN, len);
      off += len;
    }
    return off;
  }

 public:
  uint64_t req_token = 0;
  size_t rr_idx = 0;
  uint8_t *req_payload = nullptr, *resp_payload = nullptr;
  size_t req_size = 0, resp_size = 0;
  int req_device_id = -1, resp_device_id = -1;
  size_t max_req_size, max_resp_size;
  p2p_bufs* req_bufs;
  p2p_bufs* resp_bufs;
  uint32_t rr_state = UDP_RR_CREATE;
  sockaddr_in si_server{}, si_other{};
  int my_sock = -1;

  explicit UdpRr(size_t _max_req_size = 0, size_t _max_resp_size = 0)
      : max_req_size(_max_req_size), max_resp_size(_max_resp_size), req_bufs(new p2p_bufs()), resp_bufs(new p2p_bufs()) {}
  ~UdpRr() {
    release_req_bufs();
    release_resp_bufs();
    delete req_bufs;
    delete resp_bufs;
  }
  UdpRr(const UdpRr&) = delete;

  void alloc_req_bufs() { alloc_bufs(req_bufs, max_req_size); }
  void alloc_resp_bufs() { alloc_bufs(resp_bufs, max_resp_size); }
  void release_req_bufs() { release_bufs(req_bufs); }
  void release_resp_bufs() { release_bufs(resp_bufs); }
  // Records a received datagram (header + payload, `item_size` bytes in all) at its sequence number.
  void rr_merge_req_buf(uintptr_t buf, size_t item_size, int seq_num) {
    if (seq_num < 0 || seq_num >= MAX_BI_SIZE || item_size < UDP_RPC_HEADER_LEN) return;
    req_bufs->burst_items[seq_num] = buf;
    req_bufs->item_size[seq_num] = item_size;
    if (req_bufs->num_items < seq_num + 1) req_bufs->num_items = (uint16_t)(seq_num + 1);
    req_size += item_size - UDP_RPC_HEADER_LEN;
  }
  void rr_merge_resp_buf(uintptr_t buf, size_t item_size, int seq_num) {
    if (seq_num < 0 || seq_num >= MAX_BI_SIZE || item_size < UDP_RPC_HEADER_LEN) return;
    resp_bufs->burst_items[seq_num] = buf;
    resp_bufs->item_size[seq_num] = item_size;
    if (resp_bufs->num_items < seq_num + 1) resp_bufs->num_items = (uint16_t)(seq_num + 1);
    resp_size += item_size - UDP_RPC_HEADER_LEN;
  }
  size_t req_to_bufs() { return payload_to_bufs(req_payload, max_req_size, req_bufs, req_token); }
  size_t bufs_to_req() { return bufs_to_payload(req_bufs, req_payload, max_req_size); }
  size_t resp_to_bufs() { return payload_to_bufs(resp_payload, max_resp_size, resp_bufs, req_token); }
  size_t bufs_to_resp() { return bufs_to_payload(resp_bufs, resp_payload, max_resp_size); }
  bool is_req_ready() const { return req_size == max_req_size; }
  bool is_resp_ready() const { return resp_size == max_resp_size; }
  void rr_print_req_bufs() const { print_bufs("req", req_bufs); }
  void rr_print_resp_bufs() const { print_bufs("resp", resp_bufs); }

 private:
  void print_bufs(const char* what, const p2p_bufs* b) const {
    std::printf("UdpRr %p token %lu %s buffers: %u\n", (const void*)this, (unsigned long)req_token, what, (unsigned)b->num_items);
    for (size_t i = 0; i < b->num_items; i++)
      std::printf("  [%zu] %p, %zu bytes\n", i, (const void*)b->burst_items[i], (size_t)b->item_size[i]);
  }
};

// Pool of socket-path records over one request arena and one response arena (its own, or the caller's: the original's
// SmartNIC proxy hands in a registered staging region).  Records move free -> (by token) in process -> process queue
// -> ready queue -> free.
class UdpRrPool {
  std::unordered_map<uint64_t, UdpRr*> rr_cache_;
  std::vector<UdpRr*> rr_pool_;
  int pool_size_;
  size_t req_size_ = 0, resp_size_ = 0;
  uint8_t *req_arena_internal_ = nullptr, *resp_arena_internal_ = nullptr;
  MpmcRing<UdpRr*> ready_, process_, free_;
  std::mutex mu_;

 public:
  explicit UdpRrPool(int pool_size = MAX_WI_SIZE - 1)
      : pool_size_(pool_size), ready_((size_t)1 << 12), process_((size_t)1 << 12), free_((size_t)1 << 12) {}
  ~UdpRrPool() {
    for (UdpRr* rr : rr_pool_) delete rr;
    delete[] req_arena_internal_;
    delete[] resp_arena_internal_;
  }
  UdpRr** get_rr_pool() { return rr_pool_.data(); }
  int get_pool_size() const { return pool_size_; }

  void setup_and_init_rr_pool_with_preallocation(uint8_t* req_arena, size_t req_size, uint8_t* resp_arena, size_t resp_size) {
    req_size_ = req_size;
    resp_size_ = resp_size;
    for (int i = 0; i < pool_size_; i++) {
      UdpRr* rr = new UdpRr(req_size, resp_size);
      rr->req_payload = req_arena + (size_t)i * req_size;
      rr->resp_payload = resp_arena + (size_t)i * resp_size;
      rr->rr_state = UDP_RR_UNUSED;
      rr->rr_idx = (size_t)i;
      rr_pool_.push_back(rr);
      free_.push(rr);
    }
  }
  void setup_and_init_rr_pool(size_t req_size, size_t resp_size) {
    req_arena_internal_ = new uint8_t[req_size * (size_t)pool_size_]();
    resp_arena_internal_ = new uint8_t[resp_size * (size_t)pool_size_]();
    setup_and_init_rr_pool_with_preallocation(req_arena_internal_, req_size, resp_arena_internal_, resp_size);
  }
  // nullptr when no record is free (the original spins forever here).
  UdpRr* consume_rr() {
    UdpRr* rr = nullptr;
    return free_.pop(rr) ? rr : nullptr;
  }
  UdpRr* get_rr(const UdpRpcHdr* hdr) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = rr_cache_.find(hdr->req_token);
    if (it != rr_cache_.end()) return it->second;
    UdpRr* rr = consume_rr();
    if (!rr) return nullptr;
    rr->req_token = hdr->req_token;
    rr->rr_state = UDP_RR_PROCESS;
    rr->req_size = rr->resp_size = 0;
    rr_cache_[rr->req_token] = rr;
    return rr;
  }
  void reap_rr(UdpRr* rr) {
    rr->req_token = 0;
    rr->rr_state = UDP_RR_UNUSED;
    free_.push(rr);
  }
  void mark_process_rr(UdpRr* rr) {
    {
      std::lock_guard<std::mutex> g(mu_);
      rr_cache_.erase(rr->req_token);
    }
    rr->rr_state = UDP_RR_READY;
    process_.push(rr);
  }
  UdpRr* consume_process_rr() {
    UdpRr* rr = nullptr;
    return process_.pop(rr) ? rr : nullptr;
  }
  void mark_ready_rr(UdpRr* rr) { ready_.push(rr); }
  // All bytes of the record are there: out of the by-token table and into the ready queue in one step.
  void complete_rr(UdpRr* rr) {
    {
      std::lock_guard<std::mutex> g(mu_);
      rr_cache_.erase(rr->req_token);
    }
    rr->rr_state = UDP_RR_READY;
    ready_.push(rr);
  }
  UdpRr* consume_ready_rr() {
    UdpRr* rr = nullptr;
    return ready_.pop(rr) ? rr : nullptr;
  }
  int get_next_rx_ready_rr(UdpRr** next_rr) {
    *next_rr = consume_process_rr();
    return *next_rr ? 1 : 0;
  }
};

// ------------------------------------------------------------------ socket helpers of the kernel-UDP path
// (reference src/transport/udp_rx_tx.h:15-100, src/transport/udp_transport.h:16-170).  A datagram is a UdpRpcHdr and up
// to rpc_mtu() payload bytes.  The receive helpers take one datagram, file it under its token's record and hand out
// a record once all of its bytes are there; unlike the original they drop a datagram when the pool has no free record
// and they test a response for completeness with the response size.
static inline size_t udp_rpc_max_mtu() { return rpc_mtu() + UDP_RPC_HEADER_LEN; }
#define UDP_RPC_MAX_MTU (udp_rpc_max_mtu())

// A bound datagram socket (2 MB buffers; with `timeout` a receive returns after 100 ms without data); -1 on failure.
static inline int initUdpSock(sockaddr_in* si_me, bool timeout = true) {
  int s = ::socket(AF_INET, SOCK_DGRAM, IPPROTO_UDP);
  if (s < 0) return -1;
  int sz = 2 << 20;
  setsockopt(s, SOL_SOCKET, SO_RCVBUF, &sz, sizeof(sz));
  setsockopt(s, SOL_SOCKET, SO_SNDBUF, &sz, sizeof(sz));
  if (timeout) {
    timeval tv{0, 100000};
    setsockopt(s, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  }
  if (::bind(s, (sockaddr*)si_me, sizeof(*si_me)) != 0) {
    ::close(s);
    return -1;
  }
  return s;
}
// One datagram of at most `len` bytes; its length, or -1 when none arrived (time-out) or the call failed.
static inline int getData(int udp_sock, sockaddr_in* si_other, void* data, size_t len) {
  socklen_t slen = sizeof(*si_other);
  const ssize_t r = ::recvfrom(udp_sock, data, len, 0, (sockaddr*)si_other, &slen);
  return r < 0 ? -1 : (int)r;
}
// `len` bytes in datagrams of at most `seg_size` bytes.
static inline void sendData(int udp_sock, sockaddr_in* si_other, void* out, size_t len, size_t seg_size) {
  const uint8_t* p = (const uint8_t*)out;
  while (len > 0) {
    const size_t n = len < seg_size ? len : seg_size;
    if (::sendto(udp_sock, p, n, 0, (sockaddr*)si_other, sizeof(*si_other)) < 0) return;
    p += n;
    len -= n;
  }
}
static inline int udp_rr_send_req(int udp_sock, UdpRr* rr) {
  for (size_t i = 0; i < rr->req_bufs->num_items; i++)
    sendData(udp_sock, &rr->si_other, (void*)rr->req_bufs->burst_items[i], rr->req_bufs->item_size[i], UDP_RPC_MAX_MTU);
  return (int)rr->req_size;
}
static inline int udp_rr_send_resp(int udp_sock, UdpRr* rr) {
  for (size_t i = 0; i < rr->resp_bufs->num_items; i++)
    sendData(udp_sock, &rr->si_other, (void*)rr->resp_bufs->burst_items[i], rr->resp_bufs->item_size[i], UDP_RPC_MAX_MTU);
  return (int)rr->resp_size;
}
// Takes one datagram into its record; `as_resp` selects the response side.  The record owns the buffer from then on.
static inline UdpRr* udp_rr_take_datagram(int udp_sock, UdpRrPool* rr_pool, bool as_resp) {
  uint8_t* buf = new uint8_t[UDP_RPC_MAX_MTU];
  sockaddr_in si_other{};
  const int len = getData(udp_sock, &si_other, buf, UDP_RPC_MAX_MTU);
  UdpRr* rr = nullptr;
  if (len >= (int)UDP_RPC_HEADER_LEN) {
    const UdpRpcHdr* h = (const UdpRpcHdr*)buf;
    if (h->seq_num < MAX_BI_SIZE) rr = rr_pool->get_rr(h);
    if (rr) {
      rr->si_other = si_other;
      if (as_resp) rr->rr_merge_resp_buf((uintptr_t)buf, (size_t)len, h->seq_num);
      else rr->rr_merge_req_buf((uintptr_t)buf, (size_t)len, h->seq_num);
      return rr;
    }
  }
  delete[] buf;
  return nullptr;
}
static inline int udp_rr_recv_req(int udp_sock, UdpRr** new_call_id, UdpRrPool* rr_pool) {
  if (UdpRr* rr = udp_rr_take_datagram(udp_sock, rr_pool, false))
    if (rr->is_req_ready()) rr_pool->complete_rr(rr);
  *new_call_id = rr_pool->consume_ready_rr();
  return *new_call_id ? 1 : 0;
}
static inline int udp_rr_recv_resp(int udp_sock, UdpRr** new_call_id, UdpRrPool* rr_pool) {
  if (UdpRr* rr = udp_rr_take_datagram(udp_sock, rr_pool, true))
    if (rr->is_resp_ready()) rr_pool->complete_rr(rr);
  *new_call_id = rr_pool->consume_ready_rr();
  return *new_call_id ? 1 : 0;
}
// Two-thread form: the listener files datagrams and queues complete requests for the processor, which flattens their
// buffers into the request payload and marks them ready.  Both leave when `force_quit` is set.
static inline void udp_rr_recv_req_listener(int udp_sock, UdpRrPool* rr_pool, const std::atomic<bool>& force_quit) {
  while (!force_quit.load(std::memory_order_acquire))
    if (UdpRr* rr = udp_rr_take_datagram(udp_sock, rr_pool, false))
      if (rr->is_req_ready()) rr_pool->mark_process_rr(rr);
}
static inline void udp_rr_recv_req_processor(UdpRrPool* rr_pool, const std::atomic<bool>& force_quit) {
  IdleBackoff backoff;
  while (!force_quit.load(std::memory_order_acquire)) {
    UdpRr* rr = rr_pool->consume_process_rr();
    if (!rr) {
      backoff.empty();
      continue;
    }
    backoff.busy();
    rr->bufs_to_req();
    rr->release_req_bufs();
    rr_pool->mark_ready_rr(rr);
  }
}

// ------------------------------------------------------------------ small utilities of the original
// (reference src/utils/debug_utils.h:12-60, src/utils/random_utils.h:10-32)
static inline void hexDump(const char* desc, const void* addr, int len) {
  const unsigned char* pc = (const unsigned char*)addr;
  if (desc) std::printf("%s:\n", desc);
  for (int i = 0; i < len; i += 16) {
    std::printf("  %04x ", i);
    for (int j = 0; j < 16; j++) {
      if (i + j < len) std::printf(" %02x", pc[i + j]);
      else std::printf("   ");
    }
    std::printf("  ");
    for (int j = 0; j < 16 && i + j < len; j++) std::printf("%c", pc[i + j] >= 0x20 && pc[i + j] <= 0x7e ? pc[i + j] : '.');
    std::printf("\n");
  }
}
inline std::mt19937_64& srpc_global_generator() {
  static std::mt19937_64 g;
  return g;
}
static inline void seedGenerator(unsigned int seed) { srpc_global_generator().seed(seed); }
static inline void seedGeneratorRand() {
  std::random_device rd;
  srpc_global_generator().seed(rd());
}
static inline double uniform01() {
  return std::generate_canonical<double, std::numeric_limits<double>::digits>(srpc_global_generator());
}
static inline int uniformint(int min, int max) {
  std::uniform_int_distribution<int> dist(min, max);
  return dist(srpc_global_generator());
}
