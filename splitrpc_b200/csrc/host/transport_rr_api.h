// The record-level transport calls of the original (reference src/transport/dpdk_transport_ng.h:20-370:
// get_requests_zc / send_requests_zc, rr_recv / rr_recv_sync, rr_alloc_mbufs / rr_release_mbufs / rr_realloc_mbufs,
// rr_set_hdr / rr_swap_hdr, rr_send) over any `Transport`, so that a serve loop written against them runs on the
// loopback port, on kernel UDP or on a DPDK port alike.  The server of this package (splitrpc_server.h) does the same
// steps in bulk and pipelined; these are the one-record-at-a-time forms.
//
// The context argument is the port itself (the original passes its DPDK context).  A packet buffer is named by its
// arena slot: handle = slot + 1, so that 0 stays "no buffer", as in the server.
#pragma once
#include <atomic>
#include <cstring>

#include "p2p_rpc_rr.h"
#include "transport.h"

// ---- bursts
// Receives up to MAX_BI_SIZE packets: handles, header addresses, payload addresses (as the consumer of the payload sees
// them: device-side addresses when the arena is GPU-visible) and payload lengths.  Returns the number of packets.
static inline int get_requests_zc(Transport* port, p2p_hbufs* mbufs, p2p_hbufs* hdr_bufs, p2p_bufs* payload_bufs) {
  SrpcPkt pkts[MAX_BI_SIZE];
  const int n = port->rx_burst(pkts, MAX_BI_SIZE);
  for (int i = 0; i < n; i++) {
    mbufs->burst_items[i] = (uintptr_t)pkts[i].slot + 1;
    hdr_bufs->burst_items[i] = (uintptr_t)pkts[i].hdr;
    payload_bufs->burst_items[i] = (uintptr_t)port->rx_dev_ptr(pkts[i]);
    payload_bufs->item_size[i] = pkts[i].len;
  }
  mbufs->num_items = hdr_bufs->num_items = payload_bufs->num_items = (uint16_t)(n > 0 ? n : 0);
  return n > 0 ? n : 0;
}
static inline int get_requests_zc_blocking(Transport* port, p2p_hbufs* mbufs, p2p_hbufs* hdr_bufs, p2p_bufs* payload_bufs,
                                           const std::atomic<bool>& cancel) {
  IdleBackoff backoff;
  for (;;) {
    const int n = get_requests_zc(port, mbufs, hdr_bufs, payload_bufs);
    if (n > 0 || cancel.load(std::memory_order_acquire)) return n;
    backoff.empty();
  }
}
static inline void release_rx_handles(Transport* port, const uintptr_t* handles, int n) {
  for (int i = 0; i < n; i++) {
    if (!handles[i]) continue;
    SrpcPkt p;
    p.slot = (uint32_t)(handles[i] - 1);
    port->release_rx(&p, 1);
  }
}

// ---- receive into records
// One burst: every packet goes to the record of its token; complete records move to the pool's ready queue.  Packets
// the pool refuses (token 0, bad or repeated sequence number, no free record) are released at once.
static inline int rr_recv(Transport* port, P2pRpcRRPool* rr_pool) {
  p2p_hbufs mbufs, hdrs;
  p2p_bufs payloads;
  const int n = get_requests_zc(port, &mbufs, &hdrs, &payloads);
  for (int i = 0; i < n; i++) {
    p2p_rpc_hdr* h = (p2p_rpc_hdr*)hdrs.burst_items[i];
    P2pRpcRr* rr = rr_pool->append_to_rr(h, mbufs.burst_items[i], payloads.burst_items[i], payloads.item_size[i]);
    if (!rr) {
      release_rx_handles(port, &mbufs.burst_items[i], 1);
      continue;
    }
    if (rr->is_rr_ready()) {
      rr_pool->mark_rx_ready_rr(rr);
    } else if (rr->is_rr_malformed()) {
      release_rx_handles(port, rr->transport_mbufs->burst_items, rr->transport_mbufs->num_items);
      rr_pool->drop_partial(rr);
    }
  }
  return n;
}
// Polls until a request is complete (1, *new_call_id set) or `cancel` is raised (0).
static inline int rr_recv_sync(Transport* port, P2pRpcRr** new_call_id, P2pRpcRRPool& rr_pool, const std::atomic<bool>& cancel) {
  IdleBackoff backoff;
  for (;;) {
    if ((*new_call_id = rr_pool.consume_rx_ready_rr()) != nullptr) return 1;
    if (cancel.load(std::memory_order_acquire)) return 0;
    if (rr_recv(port, &rr_pool) > 0) backoff.busy();
    else backoff.empty();
  }
}

// ---- buffers of a record
// The received packets of a record go back to the port; the lists are emptied.
static inline void rr_release_mbufs(Transport* port, P2pRpcRr* rr) {
  release_rx_handles(port, rr->transport_mbufs->burst_items, rr->transport_mbufs->num_items);
  rr->clear_bufs();
}
// Transmit buffers for `payload_size` bytes (one per rpc_mtu() bytes) appended to the (empty) lists of the record:
// handle, header slot, payload address as the producer of the payload sees it, and length.  Returns how many, 0 when
// the transmit arena has no room.
static inline int rr_alloc_mbufs(Transport* port, P2pRpcRr* rr, size_t payload_size) {
  const size_t mtu = rpc_mtu();
  const int n = (int)num_fragments(payload_size, mtu);
  if (n > MAX_BI_SIZE) return 0;
  SrpcPkt tx[MAX_BI_SIZE];
  if (!port->alloc_tx(tx, n)) return 0;
  rr->clear_bufs();
  size_t left = payload_size;
  for (int i = 0; i < n; i++) {
    const size_t len = left < mtu ? left : mtu;
    left -= len;
    rr->rr_append_mbuf((uintptr_t)tx[i].slot + 1, (uintptr_t)tx[i].hdr, (uintptr_t)tx[i].payload, len);
  }
  return n;
}
static inline int rr_realloc_mbufs(Transport* port, P2pRpcRr* rr, size_t new_payload_size) {
  rr_release_mbufs(port, rr);
  return rr_alloc_mbufs(port, rr, new_payload_size);
}

// ---- headers
// Writes the header of every transmit buffer of the record from a connection template: token and sequence number,
// lengths and UDP checksum field per fragment.  Returns the number of headers.
static inline int rr_set_hdr(const p2p_rpc_conn_info* tx_conn_info, P2pRpcRr* rr, size_t payload_size) {
  const size_t mtu = rpc_mtu();
  for (uint16_t i = 0; i < rr->hdr_bufs->num_items; i++) {
    const size_t len = payload_size < mtu ? payload_size : mtu;
    payload_size -= len;
    fill_frag_hdr((p2p_rpc_hdr*)rr->hdr_bufs->burst_items[i], tx_conn_info, rr->req_token, i, (uint16_t)len, true);
  }
  return rr->hdr_bufs->num_items;
}
// Turns received headers into reply headers in place (addresses and ports swapped, lengths and checksum for
// `payload_size` payload bytes per packet).
static inline int swap_hdrs_on_cpu(p2p_hbufs* /*transport_mbufs*/, p2p_hbufs* hdr, size_t payload_size) {
  for (uint16_t i = 0; i < hdr->num_items; i++) {
    p2p_rpc_hdr* h = (p2p_rpc_hdr*)hdr->burst_items[i];
    swap_eth_hdr(h);
    add_ip_udp_len(h, (uint16_t)((RPC_HEADER_LEN - UDP_HEADER_LEN) + payload_size));
    add_udp_cksum(h);
  }
  return 1;
}
static inline int swap_sockperf_hdrs_on_cpu(p2p_hbufs* transport_mbufs, p2p_hbufs* hdr, size_t payload_size) {
  for (uint16_t i = 0; i < hdr->num_items; i++) set_sockperf_header((p2p_rpc_hdr*)hdr->burst_items[i]);
  return swap_hdrs_on_cpu(transport_mbufs, hdr, payload_size);
}
static inline int rr_swap_hdr(Transport* /*port*/, P2pRpcRr* rr, size_t payload_size) {
  return swap_hdrs_on_cpu(rr->transport_mbufs, rr->hdr_bufs, payload_size);
}

// ---- transmit
// Sends the transmit buffers listed in the record (headers and payloads are already in place).  Returns the number of
// packets sent; the buffers belong to the port again.
static inline int send_requests_zc(Transport* port, P2pRpcRr* rr) {
  SrpcPkt tx[MAX_BI_SIZE];
  const int n = rr->transport_mbufs->num_items;
  for (int i = 0; i < n; i++) {
    tx[i].slot = (uint32_t)(rr->transport_mbufs->burst_items[i] - 1);
    tx[i].hdr = (p2p_rpc_hdr*)rr->hdr_bufs->burst_items[i];
    tx[i].payload = (uint8_t*)rr->payload_bufs->burst_items[i];
    tx[i].len = (uint32_t)rr->payload_bufs->item_size[i];
  }
  const int sent = port->tx_burst(tx, n);
  rr->clear_bufs();
  return sent;
}
// Sends the record's response and gives the record back to the pool.  1 when every packet went out.
static inline int rr_send(Transport* port, P2pRpcRr* rr, P2pRpcRRPool& rr_pool) {
  const int want = rr->hdr_bufs->num_items;
  const int sent = send_requests_zc(port, rr);
  rr_pool.reap_rr(rr);
  return sent == want ? 1 : 0;
}
