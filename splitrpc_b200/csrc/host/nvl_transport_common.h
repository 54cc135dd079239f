// Control plane between an ingress (proxy) process and the serving processes of other GPUs.
//
// The original splits a deployment into a SmartNIC-side proxy and a host-side batched GPU server that talk over an RDMA
// connection: the proxy asks for buffers with a `buf_mon` ALLOC message, the server answers with the address, length
// and key of three remotely accessible regions (request ring, response ring, doorbell array), and from then on payload
// and doorbells are written by the NIC without the server's CPU (reference
// src/splitrpc_rdma_transport/gpu_rdma_common.h:57-97 message structs, gpu_rdma_batched_server.cc:279-377 handshake).
// On an NVLink machine the "remote" side is another GPU of the same box, so the connection is a Unix-domain socket and a
// region travels as a file descriptor (SCM_RIGHTS) instead of an rkey: a CUDA virtual-memory allocation exported as a
// POSIX descriptor for the rings, a memfd for host-resident control words.  Message names and fields follow the
// original so that code written against it reads the same.
#pragma once

#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstring>
#include <string>

#include "p2p_rpc_app.h"

// BUF_MON_REGION: one more payload region of a producer that is already being served in pull mode (its descriptor
// travels with the message, its size in region_bytes[0]); the reply carries status 0 and the region's index.
enum buf_mon_type : uint32_t { BUF_MON_ALLOC = 1, BUF_MON_RELEASE = 2, BUF_MON_STATS = 3, BUF_MON_REGION = 4 };
enum req_mon_type : uint32_t { REQ_MON_COMPLETE = 1 };

// One shareable region.  `stag` is the position of its descriptor among the descriptors that travel with the message
// (the role an rkey plays for an RDMA region); `address` is only meaningful inside the owner.
struct nvl_buffer_attr {
  uint64_t address = 0;
  uint64_t length = 0;
  uint32_t stag = 0;
  uint32_t _pad = 0;
};

// Parameters of the deserialising gather that the owner of a request ring expects producers to apply.
struct nvl_ingress_transform {
  uint32_t kind = 0;  // SG_TRANSFORM_*
  uint32_t _pad = 0;
  float params[6] = {0, 0, 0, 0, 0, 0};
};

// ALLOC request: proxy -> server.  Carries the proxy's transmit arena (descriptor 0) when responses are to be stored
// there by the serving GPU.  ALLOC reply: server -> proxy with the three regions of the app's slot ring (descriptors
// 0..2 = request ring, response ring, control block).
static constexpr int NVL_MAX_REGIONS = 8;
static constexpr int NVL_MAX_FDS = 12;
struct buf_mon_rr {
  uint32_t type = 0;
  uint32_t func_id = 0;
  uint32_t queue_size = 0;      // slots of the ring
  int32_t status = 0;           // reply: 0 ok, negative = refused
  uint64_t req_size = 0, resp_size = 0;
  int32_t device_id = -1;       // reply: GPU that owns the rings (-1 = host memory); request: the proxy's GPU
  uint32_t server_mode = 0;     // reply: worker mode of the server (0 sync, 1 stream armed, 2 dynamic batching)
  uint32_t max_batch = 0;
  uint32_t device_completes = 0;  // reply: 1 = the serving side stores responses and WORK_COMPLETE itself
  nvl_buffer_attr req_buf, resp_buf, ctl_buf;  // reply
  nvl_buffer_attr tx_arena;                    // request
  nvl_ingress_transform transform;             // reply
  uint64_t stat_served = 0, stat_batches = 0;  // BUF_MON_STATS reply
  int64_t timer_offset_ns = 0;  // reply: the serving device's stamp timer minus the machine's steady clock
  // Pull mode.  Request: pull = 1 and the host memory regions in which the producer's received payloads lie (their
  // descriptors follow the transmit arena's in the message); the producer will only DESCRIBE requests (fragment list
  // in the slot's descriptor block, state RX_DESCRIBED) and the serving side fetches the bytes over its own link to
  // host memory.  Reply: pull = 1 when the server mapped the regions and runs a fetch thread; 0 = push as usual.
  uint32_t pull = 0;
  uint32_t n_regions = 0;
  uint64_t region_bytes[NVL_MAX_REGIONS] = {};
};

// Per-request notification (host path, kept for parity with the original's SEND_WITH_IMM of a slot index; the
// device-completes path needs none).
struct req_mon_rr {
  uint32_t type = 0;
  uint32_t func_id = 0;
  uint32_t rr_idx = 0;
};

// Unix-domain stream socket that moves fixed-size messages together with file descriptors.
class NvlCtrlChannel {
  int fd_ = -1;

 public:
  NvlCtrlChannel() = default;
  explicit NvlCtrlChannel(int fd) : fd_(fd) {}
  ~NvlCtrlChannel() { close_fd(); }
  NvlCtrlChannel(const NvlCtrlChannel&) = delete;
  NvlCtrlChannel& operator=(const NvlCtrlChannel&) = delete;
  NvlCtrlChannel(NvlCtrlChannel&& o) noexcept : fd_(o.fd_) { o.fd_ = -1; }
  NvlCtrlChannel& operator=(NvlCtrlChannel&& o) noexcept {
    if (this != &o) {
      close_fd();
      fd_ = o.fd_;
      o.fd_ = -1;
    }
    return *this;
  }
  bool ok() const { return fd_ >= 0; }
  int fd() const { return fd_; }
  void close_fd() {
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
  }

  static bool make_addr(const std::string& path, sockaddr_un* a, socklen_t* len) {
    std::memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    if (path.empty() || path.size() >= sizeof(a->sun_path)) return false;
    std::memcpy(a->sun_path, path.data(), path.size());
    *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + path.size() + 1);
    return true;
  }

  // Listening socket at `path` (an existing socket file of a dead process is replaced).
  static int listen_at(const std::string& path) {
    sockaddr_un a;
    socklen_t len;
    if (!make_addr(path, &a, &len)) return -1;
    int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    ::unlink(path.c_str());
    if (::bind(fd, (sockaddr*)&a, len) != 0 || ::listen(fd, 8) != 0) {
      ::close(fd);
      return -1;
    }
    return fd;
  }
  // Waits up to timeout_ms for a connection on a listening socket; -1 when none arrived.
  static int accept_on(int listen_fd, int timeout_ms) {
    pollfd p{listen_fd, POLLIN, 0};
    if (::poll(&p, 1, timeout_ms) <= 0) return -1;
    return ::accept4(listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
  }
  // Connects to `path`, retrying until timeout_ms has passed (the server may still be starting).
  static int connect_to(const std::string& path, int timeout_ms) {
    sockaddr_un a;
    socklen_t len;
    if (!make_addr(path, &a, &len)) return -1;
    uint64_t t0 = getCurNs();
    for (;;) {
      int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (fd < 0) return -1;
      if (::connect(fd, (sockaddr*)&a, len) == 0) return fd;
      ::close(fd);
      if ((getCurNs() - t0) / 1000000ull > (uint64_t)timeout_ms) return -1;
      ::usleep(2000);
    }
  }

  // Sends `n` bytes and up to 4 descriptors in one message.
  bool send_msg(const void* buf, size_t n, const int* fds = nullptr, int n_fds = 0) {
    if (fd_ < 0 || n_fds > 4) return false;
    iovec iov{const_cast<void*>(buf), n};
    msghdr m{};
    m.msg_iov = &iov;
    m.msg_iovlen = 1;
    alignas(cmsghdr) char ctl[CMSG_SPACE(4 * sizeof(int))];
    if (n_fds > 0) {
      std::memset(ctl, 0, sizeof(ctl));
      m.msg_control = ctl;
      m.msg_controllen = CMSG_SPACE(n_fds * sizeof(int));
      cmsghdr* c = CMSG_FIRSTHDR(&m);
      c->cmsg_level = SOL_SOCKET;
      c->cmsg_type = SCM_RIGHTS;
      c->cmsg_len = CMSG_LEN(n_fds * sizeof(int));
      std::memcpy(CMSG_DATA(c), fds, n_fds * sizeof(int));
    }
    for (;;) {
      ssize_t r = ::sendmsg(fd_, &m, MSG_NOSIGNAL);
      if (r == (ssize_t)n) return true;
      if (r < 0 && errno == EINTR) continue;
      return false;
    }
  }

  // Receives exactly `n` bytes and the descriptors that came with them.  Returns 1 on success, 0 when timeout_ms passed
  // without a message, -1 when the peer closed or the message was malformed.
  int recv_msg(void* buf, size_t n, int* fds, int max_fds, int* n_fds, int timeout_ms) {
    if (n_fds) *n_fds = 0;
    if (fd_ < 0) return -1;
    pollfd p{fd_, POLLIN, 0};
    int pr = ::poll(&p, 1, timeout_ms);
    if (pr == 0) return 0;
    if (pr < 0) return errno == EINTR ? 0 : -1;
    iovec iov{buf, n};
    msghdr m{};
    m.msg_iov = &iov;
    m.msg_iovlen = 1;
    alignas(cmsghdr) char ctl[CMSG_SPACE(4 * sizeof(int))];
    m.msg_control = ctl;
    m.msg_controllen = sizeof(ctl);
    ssize_t r = ::recvmsg(fd_, &m, MSG_WAITALL | MSG_CMSG_CLOEXEC);
    if (r != (ssize_t)n) return -1;
    for (cmsghdr* c = CMSG_FIRSTHDR(&m); c; c = CMSG_NXTHDR(&m, c)) {
      if (c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) continue;
      int k = (int)((c->cmsg_len - CMSG_LEN(0)) / sizeof(int));
      for (int i = 0; i < k; i++) {
        int f;
        std::memcpy(&f, CMSG_DATA(c) + i * sizeof(int), sizeof(int));
        if (fds && n_fds && *n_fds < max_fds) fds[(*n_fds)++] = f;
        else ::close(f);
      }
    }
    return 1;
  }
};
