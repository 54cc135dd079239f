// DPDK port with header/data split: the NIC writes the first 64 bytes of every packet (Ethernet/IP/UDP + RPC header)
// into a host mempool and the payload into an external-memory mempool that lives in the caller's arena (pinned,
// GPU-mapped, optionally shared), so received payloads are where the scatter-gather kernels read them and the CPU never
// touches them.  Transmit chains a header mbuf and a payload mbuf whose data sits in the transmit arena, where the
// serving GPU stored the response.
//
// The role is that of the original's DPDK initialisation and rx/tx glue (reference src/transport/dpdk_init.cc,
// src/transport/dpdk_transport_ng.cc).  It is compiled only when the build defines SPLITRPC_WITH_DPDK and the DPDK
// headers are present; machines without DPDK and a NIC (this includes every machine this package has been run on) get
// init_dpdk_ctx() == nullptr from transport.h.  Nothing here has been run against hardware.
#pragma once

#if defined(SPLITRPC_WITH_DPDK) && __has_include(<rte_ethdev.h>)
#define SPLITRPC_HAVE_DPDK 1

#include <rte_eal.h>
#include <rte_ethdev.h>
#include <rte_mbuf.h>
#include <rte_mempool.h>

#include <vector>

#include "transport.h"

class DpdkPort : public Transport {
  uint16_t port_id_;
  uint16_t queue_id_;
  size_t slot_bytes_;
  ArenaMem rx_mem_, tx_mem_;
  rte_mempool* hdr_pool_ = nullptr;      // 64-byte header segments, host memory
  rte_mempool* rx_data_pool_ = nullptr;  // payload segments inside rx_mem_
  rte_mempool* tx_data_pool_ = nullptr;  // payload segments inside tx_mem_
  std::vector<rte_mbuf*> rx_held_;       // mbuf chains of packets handed to the server, indexed by SrpcPkt::slot
  std::vector<uint32_t> rx_free_;
  std::vector<rte_mbuf*> tx_held_;
  std::vector<uint32_t> tx_free_;
  std::mutex mu_;
  bool ok_ = false;

  static constexpr uint16_t kDesc = 4096;
  static constexpr unsigned kHdrRoom = RTE_PKTMBUF_HEADROOM + 128;

  // A mempool whose data buffers are slices of `mem` (registered with DPDK and mapped for the device's DMA).
  rte_mempool* make_ext_pool(const char* name, ArenaMem& mem, unsigned n, int socket) {
    const size_t page = 4096;
    if (rte_extmem_register(mem.host, mem.bytes, nullptr, 0, page) != 0) return nullptr;
    rte_eth_dev_info info;
    if (rte_eth_dev_info_get(port_id_, &info) != 0) return nullptr;
    if (rte_dev_dma_map(info.device, mem.host, RTE_BAD_IOVA, mem.bytes) != 0) return nullptr;
    rte_pktmbuf_extmem ext;
    ext.buf_ptr = mem.host;
    ext.buf_iova = RTE_BAD_IOVA;
    ext.buf_len = mem.bytes;
    ext.elt_size = (uint16_t)slot_bytes_;
    return rte_pktmbuf_pool_create_extbuf(name, n, 0, 0, (uint16_t)slot_bytes_, socket, &ext, 1);
  }

 public:
  DpdkPort(uint16_t port_id, uint16_t queue_id, size_t slot_bytes, ArenaMem rx_mem, ArenaMem tx_mem)
      : port_id_(port_id), queue_id_(queue_id), slot_bytes_(slot_bytes), rx_mem_(std::move(rx_mem)), tx_mem_(std::move(tx_mem)) {
    const int socket = rte_eth_dev_socket_id(port_id_);
    const unsigned n_rx = (unsigned)(rx_mem_.bytes / slot_bytes_), n_tx = (unsigned)(tx_mem_.bytes / slot_bytes_);
    hdr_pool_ = rte_pktmbuf_pool_create("srpc_hdr", 2 * (n_rx + n_tx), 256, 0, kHdrRoom, socket);
    rx_data_pool_ = make_ext_pool("srpc_rx_data", rx_mem_, n_rx, socket);
    tx_data_pool_ = make_ext_pool("srpc_tx_data", tx_mem_, n_tx, socket);
    if (!hdr_pool_ || !rx_data_pool_ || !tx_data_pool_) {
      srpc_log(SRPC_LOG_ERROR, "DpdkPort: mempool set-up failed");
      return;
    }
    rte_eth_conf conf{};
    conf.rxmode.offloads = RTE_ETH_RX_OFFLOAD_BUFFER_SPLIT | RTE_ETH_RX_OFFLOAD_SCATTER;
    conf.txmode.offloads = RTE_ETH_TX_OFFLOAD_MULTI_SEGS;
    if (rte_eth_dev_configure(port_id_, 1, 1, &conf) != 0) return;
    // two receive segments per packet: RPC_HEADER_LEN bytes into the header pool, the rest into the payload pool
    rte_eth_rxseg rx_seg[2] = {};
    rx_seg[0].split.mp = hdr_pool_;
    rx_seg[0].split.length = RPC_HEADER_LEN;
    rx_seg[0].split.offset = 0;
    rx_seg[1].split.mp = rx_data_pool_;
    rx_seg[1].split.length = 0;  // the remainder
    rx_seg[1].split.offset = 0;
    rte_eth_dev_info info;
    rte_eth_dev_info_get(port_id_, &info);
    rte_eth_rxconf rxc = info.default_rxconf;
    rxc.offloads = conf.rxmode.offloads;
    rxc.rx_seg = rx_seg;
    rxc.rx_nseg = 2;
    if (rte_eth_rx_queue_setup(port_id_, queue_id_, kDesc, (unsigned)socket, &rxc, nullptr) != 0) return;
    rte_eth_txconf txc = info.default_txconf;
    txc.offloads = conf.txmode.offloads;
    if (rte_eth_tx_queue_setup(port_id_, queue_id_, kDesc, (unsigned)socket, &txc) != 0) return;
    if (rte_eth_dev_start(port_id_) != 0) return;
    rte_eth_promiscuous_enable(port_id_);
    rx_held_.assign(n_rx, nullptr);
    tx_held_.assign(n_tx, nullptr);
    for (uint32_t i = 0; i < n_rx; i++) rx_free_.push_back(n_rx - 1 - i);
    for (uint32_t i = 0; i < n_tx; i++) tx_free_.push_back(n_tx - 1 - i);
    ok_ = true;
  }
  ~DpdkPort() override {
    if (ok_) {
      rte_eth_dev_stop(port_id_);
      rte_eth_dev_close(port_id_);
    }
    if (rx_mem_.release) rx_mem_.release();
    if (tx_mem_.release) tx_mem_.release();
  }
  bool ok() const { return ok_; }
  const char* name() const override { return "dpdk"; }

  int rx_burst(SrpcPkt* out, int max) override {
    rte_mbuf* m[64];
    if (max > 64) max = 64;
    const uint16_t got = rte_eth_rx_burst(port_id_, queue_id_, m, (uint16_t)max);
    int n = 0;
    std::lock_guard<std::mutex> g(mu_);
    for (uint16_t i = 0; i < got; i++) {
      rte_mbuf* h = m[i];
      rte_mbuf* d = h->next;
      if (h->data_len < RPC_HEADER_LEN || rx_free_.empty()) {  // a runt, or more packets in flight than slots
        (h->data_len < RPC_HEADER_LEN ? counters.rx_runts : counters.arena_full)++;
        rte_pktmbuf_free(h);
        continue;
      }
      const uint32_t slot = rx_free_.back();
      rx_free_.pop_back();
      rx_held_[slot] = h;
      out[n].hdr = rte_pktmbuf_mtod(h, p2p_rpc_hdr*);
      out[n].payload = d ? rte_pktmbuf_mtod(d, uint8_t*) : nullptr;
      out[n].len = d ? d->data_len : 0;
      out[n].slot = slot;
      counters.rx_bytes += out[n].len;
      n++;
    }
    counters.rx_pkts += (uint64_t)n;
    return n;
  }
  void release_rx(const SrpcPkt* pkts, int n) override {
    std::lock_guard<std::mutex> g(mu_);
    for (int i = 0; i < n; i++) {
      const uint32_t s = pkts[i].slot;
      if (s < rx_held_.size() && rx_held_[s]) {
        rte_pktmbuf_free(rx_held_[s]);  // frees the header and the payload segment
        rx_held_[s] = nullptr;
        rx_free_.push_back(s);
      }
    }
  }
  bool alloc_tx(SrpcPkt* out, int n) override {
    std::lock_guard<std::mutex> g(mu_);
    if ((int)tx_free_.size() < n) {
      counters.arena_full++;
      return false;
    }
    for (int i = 0; i < n; i++) {
      rte_mbuf* h = rte_pktmbuf_alloc(hdr_pool_);
      rte_mbuf* d = rte_pktmbuf_alloc(tx_data_pool_);
      if (!h || !d) {
        if (h) rte_pktmbuf_free(h);
        if (d) rte_pktmbuf_free(d);
        for (int k = 0; k < i; k++) {
          rte_pktmbuf_free(tx_held_[out[k].slot]);
          tx_held_[out[k].slot] = nullptr;
          tx_free_.push_back(out[k].slot);
        }
        counters.arena_full++;
        return false;
      }
      h->next = d;
      h->nb_segs = 2;
      const uint32_t slot = tx_free_.back();
      tx_free_.pop_back();
      tx_held_[slot] = h;
      out[i].slot = slot;
      out[i].hdr = rte_pktmbuf_mtod(h, p2p_rpc_hdr*);
      uint8_t* host = rte_pktmbuf_mtod(d, uint8_t*);
      out[i].payload = tx_mem_.dev + (host - tx_mem_.host);  // what a GPU writes
      out[i].len = 0;
    }
    return true;
  }
  int tx_burst(const SrpcPkt* pkts, int n) override {
    rte_mbuf* m[64];
    int sent = 0;
    for (int base = 0; base < n; base += 64) {
      const int cnt = n - base < 64 ? n - base : 64;
      {
        std::lock_guard<std::mutex> g(mu_);
        for (int i = 0; i < cnt; i++) {
          const SrpcPkt& p = pkts[base + i];
          rte_mbuf* h = tx_held_[p.slot];
          tx_held_[p.slot] = nullptr;
          tx_free_.push_back(p.slot);
          h->data_len = RPC_HEADER_LEN;
          h->next->data_len = (uint16_t)p.len;
          h->pkt_len = RPC_HEADER_LEN + p.len;
          m[i] = h;
        }
      }
      uint16_t done = rte_eth_tx_burst(port_id_, queue_id_, m, (uint16_t)cnt);
      for (int i = done; i < cnt; i++) {
        rte_pktmbuf_free(m[i]);
        counters.tx_dropped++;
      }
      sent += done;
    }
    counters.tx_pkts += (uint64_t)sent;
    return sent;
  }
  int tx_copy(const p2p_rpc_hdr* hdrs, const uint8_t* const* payloads, const uint32_t* lens, int n) override {
    int sent = 0;
    for (int i = 0; i < n; i++) {
      SrpcPkt p;
      if (!alloc_tx(&p, 1)) break;
      std::memcpy(p.hdr, &hdrs[i], RPC_HEADER_LEN);
      std::memcpy(tx_host_ptr(p), payloads[i], lens[i]);
      p.len = lens[i];
      sent += tx_burst(&p, 1);
    }
    return sent;
  }
  uint8_t* rx_dev_ptr(const SrpcPkt& p) const override { return rx_mem_.dev + (p.payload - rx_mem_.host); }
  uint8_t* tx_host_ptr(const SrpcPkt& p) const override { return tx_mem_.host + (p.payload - tx_mem_.dev); }
  uint8_t* rx_host_ptr(uint32_t slot) const override {
    rte_mbuf* h = slot < rx_held_.size() ? rx_held_[slot] : nullptr;
    return h && h->next ? rte_pktmbuf_mtod(h->next, uint8_t*) : nullptr;
  }
  bool tx_arena_info(TxArenaInfo* out) const override {
    out->host_base = tx_mem_.host;
    out->dev_base = tx_mem_.dev;
    out->bytes = tx_mem_.bytes;
    out->slot_bytes = slot_bytes_;
    out->fd = tx_mem_.fd;
    out->gpu_visible = tx_mem_.gpu_visible;
    return true;
  }
  uint64_t tx_arena_offset(const SrpcPkt& p) const override { return (uint64_t)(p.payload - tx_mem_.dev); }
  int dma_regions(DmaRegion* out, int max) const override {
    if (max < 1) return 0;
    out[0] = DmaRegion{rx_mem_.host, rx_mem_.dev, rx_mem_.bytes, rx_mem_.fd, rx_mem_.gpu_visible};
    return 1;
  }
};

// Brings up the environment abstraction layer once and opens the port.  `make_mem(bytes)` supplies the arenas
// (pinned, GPU-mapped memory for a GPU server).
static inline Transport* srpc_open_dpdk_port(int nic_port, int queue_id, size_t slot_bytes, size_t n_slots,
                                             const std::function<ArenaMem(size_t)>& make_mem) {
  static bool eal = false;
  if (!eal) {
    const char* argv[] = {"splitrpc", "--proc-type=auto", nullptr};
    if (rte_eal_init(2, const_cast<char**>(argv)) < 0) {
      srpc_log(SRPC_LOG_ERROR, "DPDK: rte_eal_init failed");
      return nullptr;
    }
    eal = true;
  }
  if (!rte_eth_dev_is_valid_port((uint16_t)nic_port)) {
    srpc_log(SRPC_LOG_ERROR, "DPDK: no such port %d", nic_port);
    return nullptr;
  }
  auto* p = new DpdkPort((uint16_t)nic_port, (uint16_t)queue_id, slot_bytes, make_mem(slot_bytes * n_slots), make_mem(slot_bytes * n_slots));
  if (!p->ok()) {
    delete p;
    return nullptr;
  }
  return p;
}

#endif  // SPLITRPC_WITH_DPDK
