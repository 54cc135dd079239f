// The 64-byte SplitRPC packet header, connection templates and buffer lists.
//
// Wire contract (reference src/p2p_rpc.h:10-21, src/udp_rr.h:23-34):
//   bytes  0..41  Ethernet + IPv4 + UDP headers (network byte order)
//   bytes 42..49  req_token   (uint64, host byte order, opaque, echoed by the server)
//   bytes 50..57  sock_perf_header (int64; the reply clears its low 32 bits)
//   bytes 58..59  seq_num     (uint16 fragment index)
//   bytes 60..63  padding
// A request of S bytes travels as ceil(S / RPC_MTU) packets that share one token
// and carry seq_num 0,1,2,...; each has min(remaining, RPC_MTU) payload bytes.
#pragma once

#include <cstddef>
#include <sstream>

#include "config_utils.h"
#include "eth_common.h"

struct p2p_rpc_hdr {
  uint8_t pkt_hdr_t[UDP_HEADER_LEN];
  uint64_t req_token;
  int64_t sock_perf_header;
  uint16_t seq_num;
  uint8_t _pad[4];
} __attribute__((packed));

static_assert(sizeof(p2p_rpc_hdr) == 64, "RPC header is exactly one 64-byte line");
static_assert(offsetof(p2p_rpc_hdr, req_token) == 42, "token at byte 42");
static_assert(offsetof(p2p_rpc_hdr, sock_perf_header) == 50, "sockperf word at byte 50");
static_assert(offsetof(p2p_rpc_hdr, seq_num) == 58, "sequence number at byte 58");

static constexpr size_t RPC_HEADER_LEN = sizeof(p2p_rpc_hdr);
static constexpr size_t RPC_HEADER_TAIL_LEN = RPC_HEADER_LEN - UDP_HEADER_LEN;  // 22
static inline size_t max_frame_len() { return rpc_mtu() + RPC_HEADER_LEN; }
#define MAX_MTU (max_frame_len())

// Header of the kernel-UDP-socket path: the same tail without the L2-L4 prefix.
struct UdpRpcHdr {
  uint64_t req_token;
  int64_t sock_perf_header;
  uint16_t seq_num;
  uint8_t _pad[4];
} __attribute__((packed));
static_assert(sizeof(UdpRpcHdr) == RPC_HEADER_TAIL_LEN, "socket-path header is the 22-byte tail");

SRPC_HD static inline eth_hdr* get_eth_header(p2p_rpc_hdr* h) { return reinterpret_cast<eth_hdr*>(h->pkt_hdr_t); }
SRPC_HD static inline ipv4_hdr* get_ip_header(p2p_rpc_hdr* h) {
  return reinterpret_cast<ipv4_hdr*>(h->pkt_hdr_t + sizeof(eth_hdr));
}
SRPC_HD static inline udp_hdr* get_udp_header(p2p_rpc_hdr* h) {
  return reinterpret_cast<udp_hdr*>(h->pkt_hdr_t + sizeof(eth_hdr) + sizeof(ipv4_hdr));
}
SRPC_HD static inline uint64_t get_req_token(const p2p_rpc_hdr* h) { return h->req_token; }
SRPC_HD static inline uint16_t get_seq_num(const p2p_rpc_hdr* h) { return h->seq_num; }
SRPC_HD static inline void* get_req_tail(p2p_rpc_hdr* h) { return reinterpret_cast<uint8_t*>(h) + UDP_HEADER_LEN; }

// A reply is marked by a zero low word in the sockperf field.
SRPC_HD static inline void set_sockperf_header(p2p_rpc_hdr* h) {
  h->sock_perf_header = (int64_t)((uint64_t)h->sock_perf_header & 0xFFFFFFFF00000000ull);
}

SRPC_HD static inline void add_ip_udp_len(p2p_rpc_hdr* h, uint16_t payload_len) {
  get_ip_header(h)->tot_len = srpc_bswap16((uint16_t)(sizeof(ipv4_hdr) + sizeof(udp_hdr) + payload_len));
  get_udp_header(h)->len = srpc_bswap16((uint16_t)(sizeof(udp_hdr) + payload_len));
}

SRPC_HD static inline void add_udp_cksum(p2p_rpc_hdr* h) {
  get_udp_header(h)->check = ipv4_pseudo_csum(get_ip_header(h));
}

// Turns a received header into an echo header in place: source and destination
// MAC, IP and port trade places and both checksum fields are cleared (the caller
// recomputes them).  Reference: src/p2p_rpc.h:64-83.
SRPC_HD static inline void swap_eth_hdr(p2p_rpc_hdr* h) {
  eth_hdr* e = get_eth_header(h);
  for (int i = 0; i < 6; i++) {
    uint8_t t = e->src_mac_.addr[i];
    e->src_mac_.addr[i] = e->dst_mac_.addr[i];
    e->dst_mac_.addr[i] = t;
  }
  ipv4_hdr* ip = get_ip_header(h);
  uint32_t tip = ip->src_ip;
  ip->src_ip = ip->dst_ip;
  ip->dst_ip = tip;
  ip->check = 0;
  udp_hdr* u = get_udp_header(h);
  uint16_t tp = u->src_port;
  u->src_port = u->dst_port;
  u->dst_port = tp;
  u->check = 0;
}

static inline size_t num_fragments(size_t size, size_t mtu) { return size == 0 ? 1 : (size + mtu - 1) / mtu; }

// ------------------------------------------------------------------ conn info
// A peer is described by a pre-built header; sending a packet is a 64-byte copy
// of the template plus the per-packet fields.
struct p2p_rpc_conn_info {
  p2p_rpc_hdr hdr_template;
};

static inline p2p_rpc_conn_info* alloc_conn_info() {
  auto* c = new p2p_rpc_conn_info;
  std::memset(c, 0, sizeof(*c));
  return c;
}
static inline void release_conn_info(p2p_rpc_conn_info* c) { delete c; }

static inline p2p_rpc_conn_info* init_conn_info(int src_port, int dst_port, const char* src_ip, const char* dst_ip,
                                                mac_addr src_mac, mac_addr dst_mac) {
  p2p_rpc_conn_info* c = alloc_conn_info();
  gen_eth_header_template(get_eth_header(&c->hdr_template), &src_mac, &dst_mac);
  gen_ipv4_header_template(get_ip_header(&c->hdr_template), ipv4_from_str(src_ip), ipv4_from_str(dst_ip));
  gen_udp_header_template(get_udp_header(&c->hdr_template), src_port, dst_port);
  return c;
}

static inline std::vector<std::string> srpc_split(const std::string& s, char sep) {
  std::vector<std::string> out;
  std::stringstream ss(s);
  std::string tok;
  while (std::getline(ss, tok, sep)) out.push_back(tok);
  return out;
}

// Server URI "mac,ip,port": the destination half stays blank until a request arrives.
static inline p2p_rpc_conn_info* initialize_src_conn_info(const std::string& uri) {
  auto f = srpc_split(uri, ',');
  if (f.size() < 3) {
    srpc_log(SRPC_LOG_ERROR, "server URI must be 'mac,ip,port', got '%s'", uri.c_str());
    return nullptr;
  }
  mac_addr m = mac_from_string(f[0]);
  return init_conn_info(std::stoi(f[2]), 0, f[1].c_str(), "0.0.0.0", m, m);
}

// Client URI "src_mac,src_ip,src_port,dst_mac,dst_ip,dst_port".
static inline p2p_rpc_conn_info* initialize_client_conn_info(const std::string& uri) {
  auto f = srpc_split(uri, ',');
  if (f.size() < 6) {
    srpc_log(SRPC_LOG_ERROR, "client URI needs 6 comma separated fields, got '%s'", uri.c_str());
    return nullptr;
  }
  return init_conn_info(std::stoi(f[2]), std::stoi(f[5]), f[1].c_str(), f[4].c_str(), mac_from_string(f[0]),
                        mac_from_string(f[3]));
}

// Makes `conn` a reply template for the sender of `recv`: RPC tail copied, and the
// destination MAC/IP/port taken from the request's source fields.
static inline void set_conn_info(p2p_rpc_conn_info* conn, p2p_rpc_hdr* recv) {
  std::memcpy(get_req_tail(&conn->hdr_template), get_req_tail(recv), RPC_HEADER_TAIL_LEN);
  get_udp_header(&conn->hdr_template)->dst_port = get_udp_header(recv)->src_port;
  get_ip_header(&conn->hdr_template)->dst_ip = get_ip_header(recv)->src_ip;
  get_eth_header(&conn->hdr_template)->dst_mac_ = get_eth_header(recv)->src_mac_;
}

// Fills the header of fragment `seq` of a message: template copy, token, sequence
// number, lengths and the partial UDP checksum.
static inline void fill_frag_hdr(p2p_rpc_hdr* dst, const p2p_rpc_conn_info* conn, uint64_t token, uint16_t seq,
                                 uint16_t payload_len, bool is_reply) {
  std::memcpy(dst, &conn->hdr_template, RPC_HEADER_LEN);
  dst->req_token = token;
  dst->seq_num = seq;
  if (is_reply) set_sockperf_header(dst);
  add_ip_udp_len(dst, (uint16_t)(payload_len + RPC_HEADER_TAIL_LEN));
  add_udp_cksum(dst);
}

// ------------------------------------------------------------------ buffer lists
static constexpr uint16_t MAX_BI_SIZE = 1024;  // fragments per message (upper bound of seq_num)
static constexpr uint16_t MAX_WI_SIZE = 1024;

struct p2p_hbufs {
  uintptr_t burst_items[MAX_BI_SIZE];
  uint16_t num_items;
};

struct p2p_bufs {
  uintptr_t burst_items[MAX_BI_SIZE];
  size_t item_size[MAX_BI_SIZE];
  uint16_t num_items;
};

// Copy list handed to a scatter-gather engine: item i copies len[i] bytes from
// i_buf[i] to o_buf[i].
struct p2p_sk_buf {
  uintptr_t i_buf[MAX_BI_SIZE];
  uintptr_t o_buf[MAX_BI_SIZE];
  size_t len[MAX_BI_SIZE];
  size_t num_items;
};

static inline void print_bufs(const p2p_bufs* b) {
  std::printf("bufs %p: %u items\n", (const void*)b, (unsigned)b->num_items);
  for (size_t i = 0; i < b->num_items; i++)
    std::printf("  [%zu] ptr=%p size=%zu\n", i, (void*)b->burst_items[i], b->item_size[i]);
}
static inline void print_skb(const p2p_sk_buf* s) {
  std::printf("skb %p: %zu items\n", (const void*)s, s->num_items);
  for (size_t i = 0; i < s->num_items; i++)
    std::printf("  [%zu] %p -> %p (%zu B)\n", i, (void*)s->i_buf[i], (void*)s->o_buf[i], s->len[i]);
}
