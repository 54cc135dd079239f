// The client-side interface of the original load generator over this package's (reference
// src/lib_loadgen/base_client.h:19-178, udp_app_client.h:20-291, p2p_rpc_app_client.h:27-291): drivers written
// against `BaseClient` (configure with the Set... calls, CreateRequest / SchedRequest per call, a listener thread in
// CompleteReqListener, PostProcessResponses at the end) run unchanged on any `Transport`.
//
// The original has one client class per transport (kernel UDP, raw DPDK, gRPC); here the transport is an object, so
// one class covers them: `TransportAppClient`, with `UdpAppClient` and `DpdkZcUdpClient` as names for it.  The
// settings are collected by the setters and the engine (`P2pRpcAppClient`, loadgen.h) is built from them by
// PreProcessRequests().  A request tag is the 1-based call number cast to a pointer; tag 0 means "no more calls".
#pragma once
#include <climits>
#include <memory>
#include <string>

#include "loadgen.h"

class BaseClient {
 public:
  std::atomic<uint32_t> n_r_create{0}, n_r_sent{0}, n_r_recv{0};
  StatsManager* StatsCollector;
  uint64_t startTimeNs = 0, endTimeNs = 0;
  bool closedLoop = false;
  std::atomic<bool> exit_flag{false};  // (a plain volatile flag in the original: a data race between the driver and the listener)
  bool verify_run = false;
  uint32_t maxRequests = UINT_MAX, n_r_warmup = 0;
  app_req_cb req_cb;
  app_resp_cb resp_cb;
  size_t max_req_size = 1024, max_resp_size = 1024;

  explicit BaseClient(StatsManager* stats) : StatsCollector(stats) {
    if (StatsCollector) StatsCollector->addMeasurementType("sojournTime");
  }
  virtual ~BaseClient() = default;

  void SetMaxRequests(uint32_t n) { maxRequests = n; }
  // tags are call numbers 1 .. maxRequests
  bool isValidToken(void* call_tag) const {
    const uintptr_t v = (uintptr_t)call_tag;
    return v >= 1 && v <= (uintptr_t)maxRequests;
  }
  void SetMaxPayloadSize(size_t req_size, size_t resp_size) {
    max_req_size = req_size;
    max_resp_size = resp_size;
  }
  void SetClosedLoop() { closedLoop = true; }
  void SetWarmupRequests(uint32_t n) { n_r_warmup = n; }
  void SetReqRespCb(app_req_cb rq, app_resp_cb rs) {
    if (rq) req_cb = std::move(rq);
    if (rs) resp_cb = std::move(rs);
  }
  void SetVerifyRun(uint16_t v) { verify_run = v > 0; }
  void exit_client() { exit_flag = true; }
  bool is_client_listening() const { return !exit_flag; }
  virtual std::string getName() { return "BaseClient"; }

  virtual void* CreateRequest(void* request_params) = 0;
  virtual void SchedRequest(void* req_tag) = 0;
  virtual void CompleteReqListener() = 0;
  virtual void PreProcessRequests() {}
  virtual void PostProcessResponses() {}
};

class TransportAppClient : public BaseClient {
  Transport* port_;
  std::string uri_;
  std::unique_ptr<P2pRpcAppClient> eng_;

 public:
  TransportAppClient(StatsManager* stats, Transport* port, std::string client_uri)
      : BaseClient(stats), port_(port), uri_(std::move(client_uri)) {
    req_cb = echo_fill;
  }
  std::string getName() override { return "TransportAppClient"; }
  P2pRpcAppClient* engine() { return eng_.get(); }

  // Builds the engine from the settings made so far, then the request payloads.
  void PreProcessRequests() override {
    ClientConfig c;
    if (!uri_.empty()) c.client_uri = uri_;
    c.req_size = max_req_size;
    c.resp_size = max_resp_size;
    c.total_requests = maxRequests;
    c.num_warmup = n_r_warmup;
    c.verify = verify_run;
    eng_.reset(new P2pRpcAppClient(port_, c, req_cb, resp_cb));
    eng_->PreProcessRequests();
  }
  // The next call number as a tag, nullptr after maxRequests.  (The payloads are pre-built, as in the original.)
  void* CreateRequest(void* /*request_params*/) override {
    const uint32_t n = n_r_create.fetch_add(1) + 1;
    if (n > maxRequests) {
      n_r_create.fetch_sub(1);
      return nullptr;
    }
    return (void*)(uintptr_t)n;
  }
  // Sends the call; retries while the receiver's arena is full, gives up when the client is told to exit.
  void SchedRequest(void* req_tag) override {
    if (!eng_ || !isValidToken(req_tag)) return;
    if (n_r_sent.load() == 0) startTimeNs = getCurNs();
    while (!eng_->SchedRequest((uint64_t)(uintptr_t)req_tag - 1)) {
      if (exit_flag) return;
      std::this_thread::yield();
    }
    n_r_sent++;
  }
  // Runs on the caller's thread until exit_client(): receives, reassembles, stamps completions.
  void CompleteReqListener() override {
    if (!eng_) return;
    std::thread watch([this] {
      while (!exit_flag) std::this_thread::sleep_for(std::chrono::microseconds(200));
      eng_->request_exit();
    });
    eng_->CompleteReqListener();
    watch.join();
    endTimeNs = getCurNs();
  }
  void PostProcessResponses() override {
    if (!eng_) return;
    n_r_recv.store((uint32_t)eng_->received());
    auto st = eng_->PostProcessResponses();
    if (StatsCollector) {
      for (uint64_t v : eng_->stats().samples("sojournTime")) StatsCollector->recordEvent("sojournTime", v);
      for (auto& kv : st) StatsCollector->trackStatInfo(kv.first, kv.second);
    }
  }
  uint64_t received() const { return eng_ ? eng_->received() : 0; }
};

using UdpAppClient = TransportAppClient;     // over a UdpPort
using DpdkZcUdpClient = TransportAppClient;  // over a DpdkPort (builds with SPLITRPC_WITH_DPDK=1)
