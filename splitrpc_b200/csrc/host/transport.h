// Packet transports behind one interface.
//
// The server only ever sees packets as {header pointer, payload pointer, length}
// triples with the header and the payload in separate buffers ("header/data
// split", reference src/transport/dpdk_init.cc:79-98): headers land in host
// memory that the CPU parses, payloads land in a buffer arena the GPU can read.
// Three back-ends implement the interface:
//   LoopbackPort  in-process link that plays the NIC: the sender's tx_burst
//                 writes header and payload into the receiver's arenas exactly
//                 like a DMA engine would, with optional fault injection;
//   UdpPort       kernel UDP sockets (reference src/transport/udp_rx_tx.h:15-93),
//                 22-byte header on the wire;
//   DpdkPort      placeholder for a DPDK + GPUDirect RDMA port (reference
//                 src/transport/dpdk_init.cc:309-398); not buildable without
//                 DPDK, creation reports that.
#pragma once

#include <netinet/in.h>
#include <sched.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>

#include <vector>

#include "cpu_batch_pool.h"
#include "mpmc_ring.h"
#include "p2p_rpc.h"

struct SrpcPkt {
  p2p_rpc_hdr* hdr = nullptr;   // 64-byte header in host memory
  uint8_t* payload = nullptr;   // payload location (host view when it is host memory)
  uint32_t len = 0;             // payload bytes
  uint32_t slot = 0;            // arena slot index (transport bookkeeping)
};

struct TransportCounters {
  std::atomic<uint64_t> rx_pkts{0}, tx_pkts{0}, rx_bytes{0}, tx_bytes{0}, tx_dropped{0}, rx_runts{0},
      arena_full{0}, injected_faults{0};
};

// Memory the payload arena of a port lives in.  `host` is what the emulated NIC
// (or the socket layer) writes through; `dev` is the address the GPU uses for the
// same bytes (equal to host for plain host memory).
struct ArenaMem {
  uint8_t* host = nullptr;
  uint8_t* dev = nullptr;
  size_t bytes = 0;
  std::function<void()> release;  // frees the memory when the arena dies
  int fd = -1;                    // memfd behind the mapping when other processes may map the arena too
  bool gpu_visible = false;       // `dev` is an address that this process's GPUs can read and write
};

// A port's transmit arena seen as one region that a serving GPU (of this or of another process) stores responses
// into: the stand-in for a NIC's registered transmit ring.
struct TxArenaInfo {
  uint8_t* host_base = nullptr;
  uint8_t* dev_base = nullptr;
  size_t bytes = 0;
  size_t slot_bytes = 0;
  int fd = -1;
  bool gpu_visible = false;
};

static inline ArenaMem make_malloc_arena(size_t bytes) {
  ArenaMem m;
  void* p = nullptr;
  if (posix_memalign(&p, 4096, bytes) != 0) std::abort();
  std::memset(p, 0, bytes);
  m.host = m.dev = (uint8_t*)p;
  m.bytes = bytes;
  m.release = [p] { free(p); };
  return m;
}

// Fixed-size slots handed out in ring order, so the fragments of one message
// occupy consecutive slots and adjacent payloads coalesce into one copy.  Headers
// live in a parallel host array with the same slot index.
class PktArena {
  ArenaMem mem_;
  size_t slot_bytes_, n_slots_;
  std::unique_ptr<p2p_rpc_hdr[]> hdrs_;
  std::unique_ptr<std::atomic<uint8_t>[]> busy_;
  std::atomic<uint64_t> next_{0};
  std::mutex claim_mu_;

 public:
  PktArena(ArenaMem mem, size_t slot_bytes) : mem_(std::move(mem)), slot_bytes_(slot_bytes) {
    n_slots_ = mem_.bytes / slot_bytes_;
    hdrs_.reset(new p2p_rpc_hdr[n_slots_]);
    busy_.reset(new std::atomic<uint8_t>[n_slots_]);
    for (size_t i = 0; i < n_slots_; i++) busy_[i].store(0);
  }
  ~PktArena() {
    if (mem_.release) mem_.release();
  }
  size_t num_slots() const { return n_slots_; }
  size_t slot_bytes() const { return slot_bytes_; }
  uint8_t* host_base() const { return mem_.host; }
  uint8_t* dev_base() const { return mem_.dev; }
  size_t bytes() const { return mem_.bytes; }
  uint8_t* host_ptr(uint32_t slot) const { return mem_.host + (size_t)slot * slot_bytes_; }
  uint8_t* dev_ptr(uint32_t slot) const { return mem_.dev + (size_t)slot * slot_bytes_; }
  p2p_rpc_hdr* hdr_ptr(uint32_t slot) const { return &hdrs_[slot]; }
  int fd() const { return mem_.fd; }
  bool gpu_visible() const { return mem_.gpu_visible; }
  uint8_t* to_dev(const uint8_t* host) const { return mem_.dev + (host - mem_.host); }
  uint8_t* to_host(const uint8_t* dev) const { return mem_.host + (dev - mem_.dev); }

  // Claims n consecutive slots (they may wrap around the end of the arena).
  // Fails without side effects when any of them is still in use.
  bool claim(uint32_t n, uint32_t* first) {
    std::lock_guard<std::mutex> g(claim_mu_);
    uint64_t start = next_.load(std::memory_order_relaxed);
    if (n > n_slots_) return false;
    for (uint32_t i = 0; i < n; i++)
      if (busy_[(start + i) % n_slots_].load(std::memory_order_acquire)) return false;
    for (uint32_t i = 0; i < n; i++) busy_[(start + i) % n_slots_].store(1, std::memory_order_relaxed);
    next_.store(start + n, std::memory_order_relaxed);
    *first = (uint32_t)(start % n_slots_);
    return true;
  }
  void release(uint32_t slot) { busy_[slot % n_slots_].store(0, std::memory_order_release); }
  size_t in_use() const {
    size_t c = 0;
    for (size_t i = 0; i < n_slots_; i++) c += busy_[i].load(std::memory_order_relaxed);
    return c;
  }
};

// A range of host memory in which the payloads of received packets may lie (the receive arena, or a buffer that a
// sender hands over by reference), as this process and its GPUs address it.  fd >= 0: a memfd that another process
// can map too, which is what lets a replica in another process fetch a request's fragments by itself.
struct DmaRegion {
  uint8_t* host_base = nullptr;
  uint8_t* dev_base = nullptr;
  size_t bytes = 0;
  int fd = -1;
  bool gpu_visible = false;
};

class Transport {
 public:
  TransportCounters counters;
  virtual ~Transport() = default;
  // Receiving side: the regions received payloads can be in (region 0 is the receive arena).  Returns how many.
  virtual int dma_regions(DmaRegion* out, int max) const {
    (void)out;
    (void)max;
    return 0;
  }
  // Sending side: memory whose contents tx_ref() can hand to the peer without a copy and that the peer can share with
  // other processes.  false: the port has none (the caller uses memory of its own).
  virtual bool alloc_dma_region(size_t bytes, DmaRegion* out) {
    (void)bytes;
    (void)out;
    return false;
  }
  // Receives up to `max` packets; never blocks.
  virtual int rx_burst(SrpcPkt* out, int max) = 0;
  // Hands buffers of received packets back to the port.
  virtual void release_rx(const SrpcPkt* pkts, int n) = 0;
  // Reserves n transmit buffers (consecutive slots); payload pointers are
  // device-view addresses a GPU may write.  Returns false when the arena is full.
  virtual bool alloc_tx(SrpcPkt* out, int n) = 0;
  // Sends packets whose headers and payloads were filled in place in buffers from
  // alloc_tx.  Returns how many were accepted; the buffers are released.
  virtual int tx_burst(const SrpcPkt* pkts, int n) = 0;
  // Sends packets whose payload lives anywhere in host memory (client side).
  virtual int tx_copy(const p2p_rpc_hdr* hdrs, const uint8_t* const* payloads, const uint32_t* lens, int n) = 0;
  // Sends packets whose payloads already sit in memory the receiver's GPU can read (registered, pinned): only
  // headers and descriptors move, the payload is handed over by reference, like a NIC sending from registered
  // memory.  The caller keeps the payload unchanged until the reply arrives.  Default: falls back to tx_copy.
  virtual int tx_ref(const p2p_rpc_hdr* hdrs, const uint8_t* const* payloads, const uint32_t* lens, int n) {
    return tx_copy(hdrs, payloads, lens, n);
  }
  virtual const char* name() const = 0;
  // Device-view address of a received payload (identity for host arenas).
  virtual uint8_t* rx_dev_ptr(const SrpcPkt& p) const { return p.payload; }
  virtual uint8_t* tx_host_ptr(const SrpcPkt& p) const { return p.payload; }
  // Host-view address of the payload buffer of receive slot `slot`.
  virtual uint8_t* rx_host_ptr(uint32_t slot) const = 0;
  // Describes the transmit arena; false when the port has none that others could write into.
  virtual bool tx_arena_info(TxArenaInfo* out) const {
    (void)out;
    return false;
  }
  // Byte offset of a transmit buffer (from alloc_tx) inside the transmit arena.
  virtual uint64_t tx_arena_offset(const SrpcPkt& p) const {
    (void)p;
    return ~0ull;
  }
};

// ------------------------------------------------------------------ loopback
// Host-side fault injector of the loopback link.  Probabilities are per packet;
// reorder swaps a packet with its successor in the same burst; truncate shortens
// the payload by `truncate_bytes`.
struct LoopbackFaults {
  double drop = 0, duplicate = 0, reorder = 0, truncate = 0;
  uint32_t truncate_bytes = 1;
  bool zero_token = false;       // stamp token 0 on every packet
  int force_seq = -1;            // overwrite seq_num (e.g. with an out-of-range value)
  uint64_t seed = 99;
};

class LoopbackPort;

class LoopbackLink {
 public:
  LoopbackFaults faults_to_server, faults_to_client;
};

class LoopbackPort : public Transport {
  static constexpr uint32_t kExternalSlot = 0xFFFFFFFFu;  // packet whose payload is not an arena slot
  // Header ring for by-reference packets: as deep as the receive ring, so a header lives at least until its packet
  // has been taken out of the ring.
  uint32_t ext_hdrs_n_;
  std::unique_ptr<p2p_rpc_hdr[]> ext_hdrs_;
  uint32_t ext_next_ = 0;
  std::unique_ptr<PktArena> rx_arena_, tx_arena_;
  MpmcRing<SrpcPkt> rx_ring_;
  LoopbackPort* peer_ = nullptr;
  LoopbackFaults faults_;  // applied to packets this port SENDS
  SrpcRng rng_;
  std::mutex tx_mu_;
  // Buffers that the peer's senders fill and hand over by reference (they belong to the port that receives them).
  std::function<ArenaMem(size_t)> region_factory_;
  static constexpr int kMaxRefRegions = 7;
  std::unique_ptr<ArenaMem> ref_regions_[kMaxRefRegions];
  std::atomic<int> n_ref_regions_{0};  // entries below it never change: readers need no lock
  std::mutex region_mu_;

  // The emulated DMA, in two steps: write one packet's header and payload into the peer's receive arena (any thread),
  // then make it visible in the peer's receive ring (the sending thread, in order).
  bool dma_write(const p2p_rpc_hdr* hdr, const uint8_t* payload_host, uint32_t len, uint32_t slot) {
    PktArena* a = peer_->rx_arena_.get();
    if (len > a->slot_bytes()) return false;
    std::memcpy(a->hdr_ptr(slot), hdr, RPC_HEADER_LEN);
    if (len) std::memcpy(a->host_ptr(slot), payload_host, len);
    return true;
  }
  bool dma_publish(uint32_t len, uint32_t slot, bool written) {
    PktArena* a = peer_->rx_arena_.get();
    if (!written) {
      a->release(slot);
      counters.tx_dropped++;
      return false;
    }
    SrpcPkt p;
    p.hdr = a->hdr_ptr(slot);
    p.payload = a->host_ptr(slot);
    p.len = len;
    p.slot = slot;
    std::atomic_thread_fence(std::memory_order_release);
    if (!peer_->rx_ring_.push(p)) {
      a->release(slot);
      counters.tx_dropped++;
      return false;
    }
    return true;
  }
  // Copy lanes of the emulated DMA engine: bursts of eight packets or more are written by this many threads (the
  // sender among them).  One lane is the sender alone.
  std::unique_ptr<CpuBatchPool> dma_pool_;
  struct DmaJob {
    p2p_rpc_hdr hdr;
    const uint8_t* payload;
    uint32_t len, slot;
    bool written;
  };
  std::vector<DmaJob> dma_jobs_;  // scratch of send_list (under tx_mu_)

  int send_list(const p2p_rpc_hdr* const* hdrs, const uint8_t* const* payloads, const uint32_t* lens, int n) {
    std::lock_guard<std::mutex> g(tx_mu_);
    // Fault injection happens "on the wire", before delivery.
    std::vector<int> order;
    order.reserve((size_t)n * 2);
    for (int i = 0; i < n; i++) {
      if (faults_.drop > 0 && rng_.uniform() < faults_.drop) {
        counters.injected_faults++;
        continue;
      }
      order.push_back(i);
      if (faults_.duplicate > 0 && rng_.uniform() < faults_.duplicate) {
        counters.injected_faults++;
        order.push_back(i);
      }
    }
    if (faults_.reorder > 0)
      for (size_t i = 0; i + 1 < order.size(); i++)
        if (rng_.uniform() < faults_.reorder) {
          std::swap(order[i], order[i + 1]);
          counters.injected_faults++;
          i++;
        }
    if (order.empty()) return n;
    uint32_t first = 0;
    PktArena* a = peer_->rx_arena_.get();
    if (!a->claim((uint32_t)order.size(), &first)) {
      counters.arena_full++;
      return 0;
    }
    dma_jobs_.resize(order.size());
    for (size_t k = 0; k < order.size(); k++) {
      int i = order[k];
      DmaJob& j = dma_jobs_[k];
      j.slot = (uint32_t)((first + k) % a->num_slots());
      j.hdr = *hdrs[i];
      j.payload = payloads[i];
      j.len = lens[i];
      j.written = false;
      if (faults_.zero_token) j.hdr.req_token = 0;
      if (faults_.force_seq >= 0) j.hdr.seq_num = (uint16_t)faults_.force_seq;
      if (faults_.truncate > 0 && rng_.uniform() < faults_.truncate) {
        j.len = j.len > faults_.truncate_bytes ? j.len - faults_.truncate_bytes : 0;
        counters.injected_faults++;
      }
    }
    auto write_one = [this](int k) {
      DmaJob& j = dma_jobs_[(size_t)k];
      j.written = dma_write(&j.hdr, j.payload, j.len, j.slot);
    };
    if (dma_pool_ && dma_jobs_.size() >= 8) dma_pool_->run((int)dma_jobs_.size(), write_one);
    else
      for (size_t k = 0; k < dma_jobs_.size(); k++) write_one((int)k);
    for (const DmaJob& j : dma_jobs_)
      if (dma_publish(j.len, j.slot, j.written)) {
        counters.tx_pkts++;
        counters.tx_bytes += j.len;
      }
    return n;
  }

 public:
  LoopbackPort(ArenaMem rx_mem, ArenaMem tx_mem, size_t slot_bytes, size_t ring_depth = 65536)
      : ext_hdrs_n_(pow2_at_least(2 * ring_depth)),
        ext_hdrs_(new p2p_rpc_hdr[ext_hdrs_n_]),
        rx_arena_(new PktArena(std::move(rx_mem), slot_bytes)),
        tx_arena_(new PktArena(std::move(tx_mem), slot_bytes)),
        rx_ring_(pow2_at_least(ring_depth)) {}
  static uint32_t pow2_at_least(size_t n) {
    uint32_t p = 1;
    while (p < n && p < (1u << 30)) p <<= 1;
    return p;
  }

  ~LoopbackPort() override {
    for (int i = 0; i < n_ref_regions_.load(); i++)
      if (ref_regions_[i]->release) ref_regions_[i]->release();
  }
  void set_dma_lanes(int lanes) {
    std::lock_guard<std::mutex> g(tx_mu_);
    dma_pool_.reset(lanes > 1 ? new CpuBatchPool(lanes - 1) : nullptr);
  }
  static void connect(LoopbackPort* a, LoopbackPort* b) {
    a->peer_ = b;
    b->peer_ = a;
  }
  // How this port makes memory of the kind its receive arena is made of (set by whoever built the arenas).
  void set_region_factory(std::function<ArenaMem(size_t)> f) { region_factory_ = std::move(f); }
  int dma_regions(DmaRegion* out, int max) const override {
    int n = 0;
    auto put = [&](uint8_t* h, uint8_t* d, size_t bytes, int fd, bool vis) {
      if (n < max) out[n++] = DmaRegion{h, d, bytes, fd, vis};
    };
    put(rx_arena_->host_base(), rx_arena_->dev_base(), rx_arena_->bytes(), rx_arena_->fd(), rx_arena_->gpu_visible());
    const int nr = n_ref_regions_.load(std::memory_order_acquire);
    for (int i = 0; i < nr; i++) {
      const ArenaMem* m = ref_regions_[i].get();
      put(m->host, m->dev, m->bytes, m->fd, m->gpu_visible);
    }
    return n;
  }
  bool alloc_dma_region(size_t bytes, DmaRegion* out) override {
    if (!peer_ || !peer_->region_factory_) return false;
    auto m = std::make_unique<ArenaMem>(peer_->region_factory_(bytes));
    if (!m->host) return false;
    std::lock_guard<std::mutex> g(peer_->region_mu_);
    const int at = peer_->n_ref_regions_.load();
    if (at >= kMaxRefRegions) {
      if (m->release) m->release();
      return false;
    }
    *out = DmaRegion{m->host, m->dev, m->bytes, m->fd, m->gpu_visible};
    peer_->ref_regions_[at] = std::move(m);
    peer_->n_ref_regions_.store(at + 1, std::memory_order_release);
    return true;
  }
  void set_faults(const LoopbackFaults& f) {
    faults_ = f;
    rng_ = SrpcRng(f.seed);
  }
  LoopbackPort* peer() const { return peer_; }
  PktArena* rx_arena() { return rx_arena_.get(); }
  PktArena* tx_arena() { return tx_arena_.get(); }

  int rx_burst(SrpcPkt* out, int max) override {
    int n = 0;
    while (n < max && rx_ring_.pop(out[n])) {
      counters.rx_bytes += out[n].len;
      n++;
    }
    counters.rx_pkts += (uint64_t)n;
    return n;
  }
  void release_rx(const SrpcPkt* pkts, int n) override {
    for (int i = 0; i < n; i++)
      if (pkts[i].slot != kExternalSlot) rx_arena_->release(pkts[i].slot);
  }
  int tx_ref(const p2p_rpc_hdr* hdrs, const uint8_t* const* payloads, const uint32_t* lens, int n) override {
    if (!peer_) return 0;
    std::lock_guard<std::mutex> g(tx_mu_);
    for (int i = 0; i < n; i++) {
      SrpcPkt p;
      p.hdr = &peer_->ext_hdrs_[peer_->ext_next_++ & (peer_->ext_hdrs_n_ - 1)];
      std::memcpy(p.hdr, &hdrs[i], RPC_HEADER_LEN);
      p.payload = const_cast<uint8_t*>(payloads[i]);
      p.len = lens[i];
      p.slot = kExternalSlot;
      std::atomic_thread_fence(std::memory_order_release);
      if (!peer_->rx_ring_.push(p)) {
        counters.tx_dropped++;
        return i;
      }
      counters.tx_pkts++;
      counters.tx_bytes += lens[i];
    }
    return n;
  }
  bool alloc_tx(SrpcPkt* out, int n) override {
    uint32_t first = 0;
    if (!tx_arena_->claim((uint32_t)n, &first)) {
      counters.arena_full++;
      return false;
    }
    for (int i = 0; i < n; i++) {
      uint32_t s = (uint32_t)((first + i) % tx_arena_->num_slots());
      out[i].slot = s;
      out[i].hdr = tx_arena_->hdr_ptr(s);
      out[i].payload = tx_arena_->dev_ptr(s);
      out[i].len = 0;
    }
    return true;
  }
  int tx_burst(const SrpcPkt* pkts, int n) override {
    if (!peer_) return 0;
    std::vector<const p2p_rpc_hdr*> hdrs((size_t)n);
    std::vector<const uint8_t*> pl((size_t)n);
    std::vector<uint32_t> lens((size_t)n);
    for (int i = 0; i < n; i++) {
      hdrs[i] = pkts[i].hdr;
      pl[i] = tx_arena_->host_ptr(pkts[i].slot);
      lens[i] = pkts[i].len;
    }
    int sent = send_list(hdrs.data(), pl.data(), lens.data(), n);
    for (int i = 0; i < n; i++) tx_arena_->release(pkts[i].slot);
    return sent;
  }
  int tx_copy(const p2p_rpc_hdr* hdrs, const uint8_t* const* payloads, const uint32_t* lens, int n) override {
    if (!peer_) return 0;
    std::vector<const p2p_rpc_hdr*> hp((size_t)n);
    for (int i = 0; i < n; i++) hp[i] = &hdrs[i];
    return send_list(hp.data(), payloads, lens, n);
  }
  // Payloads handed over by reference live in one of this port's regions, or in pinned memory whose device address
  // equals its host address.
  uint8_t* rx_dev_ptr(const SrpcPkt& p) const override {
    if (p.slot != kExternalSlot) return rx_arena_->to_dev(p.payload);
    const int nr = n_ref_regions_.load(std::memory_order_acquire);
    for (int i = 0; i < nr; i++) {
      const ArenaMem* m = ref_regions_[i].get();
      if (p.payload >= m->host && p.payload < m->host + m->bytes) return m->dev + (p.payload - m->host);
    }
    return p.payload;
  }
  uint8_t* tx_host_ptr(const SrpcPkt& p) const override { return tx_arena_->to_host(p.payload); }
  bool tx_arena_info(TxArenaInfo* out) const override {
    out->host_base = tx_arena_->host_base();
    out->dev_base = tx_arena_->dev_base();
    out->bytes = tx_arena_->bytes();
    out->slot_bytes = tx_arena_->slot_bytes();
    out->fd = tx_arena_->fd();
    out->gpu_visible = tx_arena_->gpu_visible();
    return true;
  }
  uint64_t tx_arena_offset(const SrpcPkt& p) const override { return (uint64_t)p.slot * tx_arena_->slot_bytes(); }
  uint8_t* rx_host_ptr(uint32_t slot) const override { return rx_arena_->host_ptr(slot); }
  const char* name() const override { return "loopback"; }
};

// ------------------------------------------------------------------ kernel UDP
// Datagram = 22-byte UdpRpcHdr + payload.  The 64-byte in-memory header is
// synthesised on receive (source address recorded in the L3/L4 fields) so the
// layers above are transport agnostic.
class UdpPort : public Transport {
  int fd_ = -1;
  std::unique_ptr<PktArena> rx_arena_, tx_arena_;
  static constexpr int kBatch = 32;
  std::deque<uint32_t> posted_;  // receive slots handed to the kernel, oldest first
  mmsghdr rx_msgs_[kBatch], tx_msgs_[kBatch];
  iovec rx_iov_[2 * kBatch], tx_iov_[2 * kBatch];
  sockaddr_in rx_from_[kBatch], tx_to_[kBatch];
  uint32_t tx_len_[kBatch];
  std::mutex tx_mu_;
  sockaddr_in default_dst_{};
  bool has_dst_ = false;

 public:
  UdpPort(const char* bind_ip, int bind_port, size_t slot_bytes, size_t n_slots = 4096)
      : UdpPort(bind_ip, bind_port, slot_bytes, make_malloc_arena(slot_bytes * n_slots), make_malloc_arena(slot_bytes * n_slots)) {}
  // Arenas supplied by the caller: pinned, GPU-mapped (and shareable) memory when a GPU gathers from the receive arena
  // and serving GPUs store responses into the transmit arena.
  UdpPort(const char* bind_ip, int bind_port, size_t slot_bytes, ArenaMem rx_mem, ArenaMem tx_mem)
      : rx_arena_(new PktArena(std::move(rx_mem), slot_bytes)),
        tx_arena_(new PktArena(std::move(tx_mem), slot_bytes)) {
    fd_ = ::socket(AF_INET, SOCK_DGRAM | SOCK_NONBLOCK, 0);
    int sz = 2 << 20;
    setsockopt(fd_, SOL_SOCKET, SO_RCVBUF, &sz, sizeof(sz));
    setsockopt(fd_, SOL_SOCKET, SO_SNDBUF, &sz, sizeof(sz));
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons((uint16_t)bind_port);
    inet_pton(AF_INET, bind_ip, &a.sin_addr);
    if (::bind(fd_, (sockaddr*)&a, sizeof(a)) != 0) {
      srpc_log(SRPC_LOG_ERROR, "UdpPort: bind %s:%d failed", bind_ip, bind_port);
      ::close(fd_);
      fd_ = -1;
    }
  }
  ~UdpPort() override {
    if (fd_ >= 0) ::close(fd_);
  }
  bool ok() const { return fd_ >= 0; }
  int bound_port() const {
    sockaddr_in a{};
    socklen_t l = sizeof(a);
    getsockname(fd_, (sockaddr*)&a, &l);
    return ntohs(a.sin_port);
  }
  void set_destination(const char* ip, int port) {
    default_dst_.sin_family = AF_INET;
    default_dst_.sin_port = htons((uint16_t)port);
    inet_pton(AF_INET, ip, &default_dst_.sin_addr);
    has_dst_ = true;
  }

  // Receive: up to kBatch arena slots are kept posted like the descriptors of a NIC receive queue; one recvmmsg
  // fills as many of them as datagrams are waiting, and the kernel scatters every datagram straight into its places
  // (22 header bytes into the slot's header, the rest into the slot's payload): header/data split without a staging
  // copy.  Slots that stay empty remain posted for the next call.
  int rx_burst(SrpcPkt* out, int max) override {
    const int want = max < kBatch ? max : kBatch;
    while ((int)posted_.size() < want) {
      uint32_t slot = 0;
      if (!rx_arena_->claim(1, &slot)) {
        counters.arena_full++;
        break;
      }
      std::memset(rx_arena_->hdr_ptr(slot), 0, sizeof(p2p_rpc_hdr));
      posted_.push_back(slot);
    }
    const int np = (int)posted_.size() < want ? (int)posted_.size() : want;
    if (np == 0) return 0;
    for (int i = 0; i < np; i++) {
      const uint32_t slot = posted_[(size_t)i];
      rx_iov_[2 * i] = iovec{get_req_tail(rx_arena_->hdr_ptr(slot)), RPC_HEADER_TAIL_LEN};
      rx_iov_[2 * i + 1] = iovec{rx_arena_->host_ptr(slot), rx_arena_->slot_bytes()};
      std::memset(&rx_msgs_[i], 0, sizeof(mmsghdr));
      rx_msgs_[i].msg_hdr.msg_iov = &rx_iov_[2 * i];
      rx_msgs_[i].msg_hdr.msg_iovlen = 2;
      rx_msgs_[i].msg_hdr.msg_name = &rx_from_[i];
      rx_msgs_[i].msg_hdr.msg_namelen = sizeof(sockaddr_in);
    }
    const int r = ::recvmmsg(fd_, rx_msgs_, (unsigned)np, MSG_DONTWAIT, nullptr);
    if (r <= 0) return 0;
    int n = 0;
    for (int i = 0; i < r; i++) {
      const uint32_t slot = posted_[(size_t)i];
      const size_t got = rx_msgs_[i].msg_len;
      if (got < RPC_HEADER_TAIL_LEN || (rx_msgs_[i].msg_hdr.msg_flags & MSG_TRUNC)) {
        counters.rx_runts++;
        rx_arena_->release(slot);
        continue;
      }
      p2p_rpc_hdr* h = rx_arena_->hdr_ptr(slot);
      get_ip_header(h)->src_ip = rx_from_[i].sin_addr.s_addr;
      get_udp_header(h)->src_port = rx_from_[i].sin_port;
      const uint32_t len = (uint32_t)(got - RPC_HEADER_TAIL_LEN);
      out[n].hdr = h;
      out[n].payload = rx_arena_->host_ptr(slot);
      out[n].len = len;
      out[n].slot = slot;
      counters.rx_bytes += len;
      n++;
    }
    posted_.erase(posted_.begin(), posted_.begin() + r);
    counters.rx_pkts += (uint64_t)n;
    return n;
  }
  void release_rx(const SrpcPkt* pkts, int n) override {
    for (int i = 0; i < n; i++) rx_arena_->release(pkts[i].slot);
  }
  bool alloc_tx(SrpcPkt* out, int n) override {
    uint32_t first = 0;
    if (!tx_arena_->claim((uint32_t)n, &first)) return false;
    for (int i = 0; i < n; i++) {
      uint32_t s = (uint32_t)((first + i) % tx_arena_->num_slots());
      out[i].slot = s;
      out[i].hdr = tx_arena_->hdr_ptr(s);
      out[i].payload = tx_arena_->dev_ptr(s);
      out[i].len = 0;
    }
    return true;
  }
  // Transmit: sendmmsg over {22 header bytes, payload} pairs, one system call per burst of up to kBatch datagrams and
  // no staging copy.
  sockaddr_in destination_of(const p2p_rpc_hdr* h) const {
    sockaddr_in to = default_dst_;
    const ipv4_hdr* ip = get_ip_header(const_cast<p2p_rpc_hdr*>(h));
    const udp_hdr* u = get_udp_header(const_cast<p2p_rpc_hdr*>(h));
    if (!has_dst_ || (ip->dst_ip != 0 && u->dst_port != 0)) {
      to.sin_family = AF_INET;
      to.sin_addr.s_addr = ip->dst_ip;
      to.sin_port = u->dst_port;
    }
    return to;
  }
  template <class At>
  int send_many(int n, At&& at) {  // at(i, &hdr, &payload, &len)
    std::lock_guard<std::mutex> g(tx_mu_);
    int sent_total = 0;
    for (int base = 0; base < n; base += kBatch) {
      const int m = n - base < kBatch ? n - base : kBatch;
      int k = 0;
      for (int i = 0; i < m; i++) {
        const p2p_rpc_hdr* h = nullptr;
        const uint8_t* payload = nullptr;
        uint32_t len = 0;
        at(base + i, &h, &payload, &len);
        if (len > rx_arena_->slot_bytes()) {
          counters.tx_dropped++;
          continue;
        }
        tx_to_[k] = destination_of(h);
        tx_iov_[2 * k] = iovec{const_cast<uint8_t*>(reinterpret_cast<const uint8_t*>(h)) + UDP_HEADER_LEN, RPC_HEADER_TAIL_LEN};
        tx_iov_[2 * k + 1] = iovec{const_cast<uint8_t*>(payload), len};
        std::memset(&tx_msgs_[k], 0, sizeof(mmsghdr));
        tx_msgs_[k].msg_hdr.msg_iov = &tx_iov_[2 * k];
        tx_msgs_[k].msg_hdr.msg_iovlen = len ? 2 : 1;
        tx_msgs_[k].msg_hdr.msg_name = &tx_to_[k];
        tx_msgs_[k].msg_hdr.msg_namelen = sizeof(sockaddr_in);
        tx_len_[k] = len;
        k++;
      }
      int done = 0;
      for (int tries = 0; done < k && tries < 100; tries++) {
        const int r = ::sendmmsg(fd_, tx_msgs_ + done, (unsigned)(k - done), MSG_DONTWAIT);
        if (r > 0) {
          for (int i = 0; i < r; i++) counters.tx_bytes += tx_len_[done + i];
          done += r;
        } else {
          sched_yield();  // socket buffer full: let the receiver drain
        }
      }
      counters.tx_pkts += (uint64_t)done;
      counters.tx_dropped += (uint64_t)(k - done);
      sent_total += done;
    }
    return sent_total;
  }
  int tx_burst(const SrpcPkt* pkts, int n) override {
    const int s = send_many(n, [&](int i, const p2p_rpc_hdr** h, const uint8_t** p, uint32_t* len) {
      *h = pkts[i].hdr;
      *p = tx_arena_->host_ptr(pkts[i].slot);
      *len = pkts[i].len;
    });
    for (int i = 0; i < n; i++) tx_arena_->release(pkts[i].slot);
    return s;
  }
  int tx_copy(const p2p_rpc_hdr* hdrs, const uint8_t* const* payloads, const uint32_t* lens, int n) override {
    return send_many(n, [&](int i, const p2p_rpc_hdr** h, const uint8_t** p, uint32_t* len) {
      *h = &hdrs[i];
      *p = payloads[i];
      *len = lens[i];
    });
  }
  bool tx_arena_info(TxArenaInfo* out) const override {
    out->host_base = tx_arena_->host_base();
    out->dev_base = tx_arena_->dev_base();
    out->bytes = tx_arena_->bytes();
    out->slot_bytes = tx_arena_->slot_bytes();
    out->fd = tx_arena_->fd();
    out->gpu_visible = tx_arena_->gpu_visible();
    return true;
  }
  uint64_t tx_arena_offset(const SrpcPkt& p) const override { return (uint64_t)p.slot * tx_arena_->slot_bytes(); }
  uint8_t* rx_host_ptr(uint32_t slot) const override { return rx_arena_->host_ptr(slot); }
  uint8_t* rx_dev_ptr(const SrpcPkt& p) const override { return rx_arena_->to_dev(p.payload); }
  uint8_t* tx_host_ptr(const SrpcPkt& p) const override { return tx_arena_->to_host(p.payload); }
  int dma_regions(DmaRegion* out, int max) const override {
    if (max < 1) return 0;
    out[0] = DmaRegion{rx_arena_->host_base(), rx_arena_->dev_base(), rx_arena_->bytes(), rx_arena_->fd(), rx_arena_->gpu_visible()};
    return 1;
  }
  const char* name() const override { return "udp"; }
};

// ------------------------------------------------------------------ DPDK placeholder
enum MEM_ALLOC_TYPES { HOST_MEM_ONLY = 0, DEV_MEM_ONLY = 1, BUFFER_SPLIT = 2 };

struct dpdk_ctx {
  int nic_port = 0, queue_id = 0, mem_alloc_type = HOST_MEM_ONLY, device_id = 0, zerocopy_mode = 0;
};

// A DPDK port needs libdpdk and a NIC.  The port itself is DpdkPort (dpdk_port.h), compiled only into builds made with
// SPLITRPC_WITH_DPDK=1; this entry point of the original's name reports that a build without it has none.
static inline Transport* init_dpdk_ctx(const dpdk_ctx&) {
  srpc_log(SRPC_LOG_ERROR, "DPDK transport requested but this build has no DPDK; use the loopback or UDP transport");
  return nullptr;
}
