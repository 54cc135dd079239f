// L2-L4 header structs and helpers for the SplitRPC wire format.
//
// The on-wire layout is fixed by the protocol (reference: src/eth_common.h:13-48):
// a 14-byte Ethernet header, a 20-byte IPv4 header (no options) and an 8-byte UDP
// header, 42 bytes in total, all fields in network byte order.  This file only
// keeps the layout and the arithmetic (pseudo-header checksum, reference
// src/eth_common.h:97-135); the code is organised around small value types and
// free functions that work both on the host and, where marked, on the device.
#pragma once

#include <arpa/inet.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#if defined(__CUDACC__)
#define SRPC_HD __host__ __device__
#else
#define SRPC_HD
#endif

struct mac_addr {
  uint8_t addr[6];
} __attribute__((packed));

struct eth_hdr {
  mac_addr dst_mac_;
  mac_addr src_mac_;
  uint16_t eth_type_;
} __attribute__((packed));

// Byte 0 holds version (high nibble) and ihl (low nibble); byte 1 holds dscp/ecn.
struct ipv4_hdr {
  uint8_t ihl : 4;
  uint8_t version : 4;
  uint8_t ecn : 2;
  uint8_t dscp : 6;
  uint16_t tot_len;
  uint16_t id;
  uint16_t frag_off;
  uint8_t ttl;
  uint8_t protocol;
  uint16_t check;
  uint32_t src_ip;
  uint32_t dst_ip;
} __attribute__((packed));

struct udp_hdr {
  uint16_t src_port;
  uint16_t dst_port;
  uint16_t len;
  uint16_t check;
} __attribute__((packed));

static_assert(sizeof(eth_hdr) == 14, "ethernet header is 14 bytes on the wire");
static_assert(sizeof(ipv4_hdr) == 20, "ipv4 header is 20 bytes on the wire");
static_assert(sizeof(udp_hdr) == 8, "udp header is 8 bytes on the wire");

static constexpr int UDP_HEADER_LEN = sizeof(eth_hdr) + sizeof(ipv4_hdr) + sizeof(udp_hdr);
static_assert(UDP_HEADER_LEN == 42, "L2-L4 prefix is 42 bytes");
static constexpr uint16_t ETHER_TYPE_IPV4 = 0x0800;
static constexpr uint8_t SRPC_IPPROTO_UDP = 17;

SRPC_HD static inline uint16_t srpc_bswap16(uint16_t v) { return (uint16_t)((v << 8) | (v >> 8)); }

static inline void gen_eth_header_template(eth_hdr* h, const mac_addr* src, const mac_addr* dst) {
  h->dst_mac_ = *dst;
  h->src_mac_ = *src;
  h->eth_type_ = htons(ETHER_TYPE_IPV4);
}

// IP addresses are given in host byte order.  tot_len starts at the two header
// sizes; the payload length is added when a packet is built.
static inline void gen_ipv4_header_template(ipv4_hdr* h, uint32_t src_ip, uint32_t dst_ip) {
  std::memset(h, 0, sizeof(*h));
  h->version = 4;
  h->ihl = 5;
  h->ecn = 1;
  h->dscp = 0;
  h->tot_len = htons(sizeof(ipv4_hdr) + sizeof(udp_hdr));
  h->ttl = 128;
  h->protocol = SRPC_IPPROTO_UDP;
  h->src_ip = htonl(src_ip);
  h->dst_ip = htonl(dst_ip);
}

static inline void gen_udp_header_template(udp_hdr* h, int src_port, int dst_port) {
  h->src_port = htons((uint16_t)src_port);
  h->dst_port = htons((uint16_t)dst_port);
  h->len = htons(sizeof(ipv4_hdr) + sizeof(udp_hdr));
  h->check = 0;
}

// One's-complement sum of the IPv4 pseudo header {src, dst, 0, proto, udp_len},
// folded to 16 bits and NOT inverted: a NIC with UDP checksum offload expects the
// partial sum in the checksum field and finishes it over the UDP header+payload.
// udp_len is tot_len minus (version*4), which for IPv4 equals tot_len - 16 in the
// protocol's convention (reference src/eth_common.h:113-115) and is kept as is so
// that both ends compute identical bytes.
SRPC_HD static inline uint16_t ipv4_pseudo_csum(const ipv4_hdr* ip) {
  uint16_t words[6];
  uint32_t s = ip->src_ip, d = ip->dst_ip;
  words[0] = (uint16_t)(s & 0xFFFF);
  words[1] = (uint16_t)(s >> 16);
  words[2] = (uint16_t)(d & 0xFFFF);
  words[3] = (uint16_t)(d >> 16);
  words[4] = (uint16_t)((uint16_t)ip->protocol << 8);  // bytes {0, proto} read as a LE word
  uint16_t tot = srpc_bswap16(ip->tot_len);
  uint16_t l4 = (uint16_t)(tot - (uint16_t)(ip->version * 4u));
  words[5] = srpc_bswap16(l4);
  uint32_t sum = 0;
  for (int i = 0; i < 6; i++) sum += words[i];
  sum = (sum & 0xFFFF) + (sum >> 16);
  sum = (sum & 0xFFFF) + (sum >> 16);
  return (uint16_t)sum;
}

// Standard IPv4 header checksum (inverted one's-complement sum of the 10 header
// words with the check field taken as zero).  The NIC normally fills this in; the
// loopback transport has no NIC, so software computes it when asked to.
SRPC_HD static inline uint16_t ipv4_header_csum(const ipv4_hdr* ip) {
  const uint8_t* b = reinterpret_cast<const uint8_t*>(ip);
  uint32_t sum = 0;
  for (int i = 0; i < 20; i += 2) {
    if (i == 10) continue;
    sum += (uint32_t)b[i] | ((uint32_t)b[i + 1] << 8);
  }
  sum = (sum & 0xFFFF) + (sum >> 16);
  sum = (sum & 0xFFFF) + (sum >> 16);
  return (uint16_t)~sum;
}

// Host-byte-order address from dotted-quad text; 0 on parse failure.
static inline uint32_t ipv4_from_str(const char* ip) {
  in_addr a{};
  if (inet_pton(AF_INET, ip, &a) != 1) {
    std::fprintf(stderr, "splitrpc: bad IPv4 address '%s'\n", ip);
    return 0;
  }
  return ntohl(a.s_addr);
}

// Takes a network-byte-order address.
static inline std::string ipv4_to_string(uint32_t ipv4_addr_be) {
  char buf[INET_ADDRSTRLEN] = {0};
  in_addr a{};
  a.s_addr = ipv4_addr_be;
  if (!inet_ntop(AF_INET, &a, buf, sizeof(buf))) return std::string();
  return std::string(buf);
}

static inline mac_addr mac_from_string(const std::string& s) {
  mac_addr m{};
  unsigned v[6] = {0, 0, 0, 0, 0, 0};
  if (std::sscanf(s.c_str(), "%x:%x:%x:%x:%x:%x", &v[0], &v[1], &v[2], &v[3], &v[4], &v[5]) != 6)
    std::fprintf(stderr, "splitrpc: bad MAC address '%s'\n", s.c_str());
  for (int i = 0; i < 6; i++) m.addr[i] = (uint8_t)v[i];
  return m;
}

static inline std::string mac_to_string(const mac_addr& m) {
  char buf[20];
  std::snprintf(buf, sizeof(buf), "%02x:%02x:%02x:%02x:%02x:%02x", m.addr[0], m.addr[1], m.addr[2],
                m.addr[3], m.addr[4], m.addr[5]);
  return std::string(buf);
}
