// Load generator: arrival processes, request clients, statistics.
//
// Measurement protocol of reference src/lib_loadgen (dist_rpc_bench.cc:76-292,
// base_client.h:19-178, stats_factory.h:29-153): open loop = arrival instants
// precomputed from a deterministic / exponential / hyper-exponential
// inter-arrival distribution and issued by generator threads; closed loop = N
// requests outstanding, each completion re-issues; warm-up requests excluded;
// per-request sojourn time = completion - dispatch; summary written as
// agg_<exp>_stat.json with the same keys and the same percentile rule.
// The client is transport agnostic (loopback or UDP), reassembles fragmented
// replies by token and can verify every reply against an app callback.
#pragma once

#include <cmath>
#include <iomanip>
#include <map>
#include <thread>
#include <unordered_map>

#include "p2p_rpc_app.h"
#include "p2p_rpc_rr.h"
#include "transport.h"

// ------------------------------------------------------------------ distributions
class Distribution {
 protected:
  SrpcRng rng_;

 public:
  explicit Distribution(uint64_t seed) : rng_(seed) {}
  virtual ~Distribution() = default;
  virtual double nextRand() = 0;
  virtual void setMeanValue(double mean) = 0;
  double uniform01() {
    double u;
    do u = rng_.uniform();
    while (u <= 0.0);
    return u;
  }
};

class DistributionDet : public Distribution {
  double val_;

 public:
  explicit DistributionDet(double mean, uint64_t seed = 12345) : Distribution(seed), val_(mean) {}
  double nextRand() override { return val_; }
  void setMeanValue(double mean) override { val_ = mean; }
};

// Exponential with arrival rate `rate` (mean 1/rate).
class DistributionExp : public Distribution {
  double rate_;

 public:
  explicit DistributionExp(double rate, uint64_t seed = 12345) : Distribution(seed), rate_(rate) {}
  double nextRand() override { return -std::log(uniform01()) / rate_; }
  void setMeanValue(double rate) override { rate_ = rate; }
};

// Two-branch hyper-exponential with the given mean and squared coefficient of
// variation (Morse's balanced-means construction).
class DistributionHyp : public Distribution {
  double mean_, cov2_;

 public:
  DistributionHyp(double mean, double cov2, uint64_t seed = 12345) : Distribution(seed), mean_(mean), cov2_(cov2) {}
  double nextRand() override {
    double z1 = uniform01(), z2 = uniform01();
    double p = 0.5 * (1.0 - std::sqrt((cov2_ - 1.0) / (cov2_ + 1.0)));
    double branch_mean = (z1 > p) ? mean_ / (1.0 - p) : mean_ / p;
    return -0.5 * branch_mean * std::log(z2);
  }
  void setMeanValue(double mean) override { mean_ = mean; }
  void setCoVValue(double c) { cov2_ = c; }
};

// lambda = mean inter-arrival time in seconds.  cov: 0 deterministic, 1 Poisson,
// >1 hyper-exponential with that squared CoV (P2P_RPC_ARR_RATE_COV).
class LoadGenerator {
  std::unique_ptr<Distribution> dist_;

 public:
  explicit LoadGenerator(double lambda, int cov = -1, uint64_t seed = 12345) {
    if (cov < 0) cov = readEnvInfo<int>("P2P_RPC_ARR_RATE_COV", 0);
    if (cov == 0)
      dist_.reset(new DistributionDet(lambda, seed));
    else if (cov == 1)
      dist_.reset(new DistributionExp(1.0 / lambda, seed));
    else
      dist_.reset(new DistributionHyp(lambda, (double)cov, seed));
  }
  uint64_t nextReqArr(uint64_t prev_ns, bool blocking = true) {
    uint64_t next = prev_ns + (uint64_t)(dist_->nextRand() * 1e9);
    if (blocking) sleepUntil(next);
    return next;
  }
};

// ------------------------------------------------------------------ stats
static const char* const LAT_UNIT = "us";
static constexpr double LAT_UNIT_MULTIPLIER = 1000.0;  // samples are in ns

class StatsManager {
  std::string exp_name_, out_dir_;
  std::map<std::string, Measure<uint64_t>*> metrics_;
  std::map<std::string, std::string> info_str_;
  std::map<std::string, double> info_num_;

  static std::string json_escape(const std::string& s) {
    std::string o;
    for (char c : s) {
      if (c == '"' || c == '\\') o.push_back('\\');
      o.push_back(c);
    }
    return o;
  }

 public:
  explicit StatsManager(std::string exp_name, std::string out_dir = ".")
      : exp_name_(std::move(exp_name)), out_dir_(std::move(out_dir)) {}
  ~StatsManager() {
    for (auto& kv : metrics_) delete kv.second;
  }
  void recordEvent(const std::string& metric, uint64_t value) {
    auto it = metrics_.find(metric);
    if (it == metrics_.end()) it = metrics_.emplace(metric, new Measure<uint64_t>(metric)).first;
    it->second->add(value);
  }
  // The experiment clock and the explicit spellings of the original (reference src/lib_loadgen/stats_factory.h:57-85,
  // 118-123): a measurement may be declared before its first sample, raw samples can be fetched or dumped by name.
  uint64_t expStartTimeNs = getCurNs(), expEndTimeNs = 0;
  void startExp(uint64_t set_start = 0) {
    expStartTimeNs = set_start ? set_start : getCurNs();
    resetStats();
  }
  void endExp() {
    expEndTimeNs = getCurNs();
    trackStatInfo("exec_time_ns", (double)(expEndTimeNs - expStartTimeNs));
  }
  void addMeasurementType(const std::string& metric) {
    if (metrics_.find(metric) == metrics_.end()) metrics_.emplace(metric, new Measure<uint64_t>(metric));
  }
  std::vector<uint64_t>& getRawMeasure(const std::string& metric) { return samples(metric); }
  void dumpRawStats() {
    for (auto& kv : metrics_) kv.second->dumpStatsToFile(exp_name_, out_dir_);
  }
  void trackStatInfo(const std::string& k, const std::string& v) { info_str_[k] = v; }
  void trackStatInfo(const std::string& k, double v) { info_num_[k] = v; }
  void resetStats() {
    for (auto& kv : metrics_) kv.second->clear();
  }
  std::vector<uint64_t>& samples(const std::string& metric) {
    auto it = metrics_.find(metric);
    if (it == metrics_.end()) it = metrics_.emplace(metric, new Measure<uint64_t>(metric)).first;
    return it->second->getRawMeasurements();
  }

  // Key/value view of the summary (what saveStats writes).
  std::map<std::string, double> aggregate(const std::vector<std::string>& measures = {"sojournTime"}) {
    std::map<std::string, double> out = info_num_;
    const std::string u = std::string("_") + LAT_UNIT;
    for (const std::string& m : measures) {
      std::vector<uint64_t>& v = samples(m);
      uint64_t mn = 0, mx = 0;
      if (!v.empty()) {
        mn = *std::min_element(v.begin(), v.end());
        mx = *std::max_element(v.begin(), v.end());
      }
      out["n_" + m] = (double)v.size();
      out["min_" + m + u] = (double)mn / LAT_UNIT_MULTIPLIER;
      out["max_" + m + u] = (double)mx / LAT_UNIT_MULTIPLIER;
      out["mean_" + m + u] = getMean(v) / LAT_UNIT_MULTIPLIER;
      out["p50_" + m + u] = getPercentile(v, 0.50) / LAT_UNIT_MULTIPLIER;
      out["p90_" + m + u] = getPercentile(v, 0.90) / LAT_UNIT_MULTIPLIER;
      out["p95_" + m + u] = getPercentile(v, 0.95) / LAT_UNIT_MULTIPLIER;
      out["p99_" + m + u] = getPercentile(v, 0.99) / LAT_UNIT_MULTIPLIER;
      out["p999_" + m + u] = getPercentile(v, 0.999) / LAT_UNIT_MULTIPLIER;
    }
    return out;
  }

  std::string to_json(const std::vector<std::string>& measures = {"sojournTime"}) {
    std::ostringstream os;
    os << "{\n";
    bool first = true;
    for (auto& kv : info_str_) {
      os << (first ? "" : ",\n") << "    \"" << json_escape(kv.first) << "\": \"" << json_escape(kv.second) << "\"";
      first = false;
    }
    for (auto& kv : aggregate(measures)) {
      os << (first ? "" : ",\n") << "    \"" << json_escape(kv.first) << "\": " << std::setprecision(15) << kv.second;
      first = false;
    }
    os << "\n}\n";
    return os.str();
  }

  std::string saveStats(const std::vector<std::string>& measures = {"sojournTime"}, bool dump_raw = false) {
    if (dump_raw)
      for (auto& kv : metrics_) kv.second->dumpStatsToFile(exp_name_, out_dir_);
    std::string fn = out_dir_ + "/agg_" + exp_name_ + "_stat.json";
    std::ofstream out(fn);
    out << to_json(measures);
    return fn;
  }
};

// ------------------------------------------------------------------ payload callbacks
// app_req_cb fills one request payload; app_resp_cb checks one reply and returns 0
// when it is correct.
using app_req_cb = std::function<int(uint8_t* req, size_t len, uint64_t seq)>;
using app_resp_cb = std::function<int(const uint8_t* req, const uint8_t* resp, size_t resp_len)>;

// Echo payload: 0xDE,0xAD,0xBE,0xEF cycling at every 8192-byte boundary, 2
// elsewhere; the reply must be identical (reference src/lib_loadgen/echo_client.cc:11-70).
static inline int echo_fill(uint8_t* p, size_t n, uint64_t) {
  static const uint8_t magic[4] = {0xDE, 0xAD, 0xBE, 0xEF};
  std::memset(p, 2, n);
  for (size_t i = 0, c = 0; i < n; i += 8192, c++) p[i] = magic[c & 3];
  return 0;
}
static inline int echo_check(const uint8_t* req, const uint8_t* resp, size_t n) {
  return std::memcmp(req, resp, n) == 0 ? 0 : 1;
}
// vec_add payload: a repeating byte ramp; the reply must be every byte + 1.
static inline int vec_add_fill(uint8_t* p, size_t n, uint64_t seq) {
  for (size_t i = 0; i < n; i++) p[i] = (uint8_t)((i * 7 + seq) & 0xFF);
  return 0;
}
static inline int vec_add_check(const uint8_t* req, const uint8_t* resp, size_t n) {
  for (size_t i = 0; i < n; i++)
    if (resp[i] != (uint8_t)(req[i] + 1)) return 1;
  return 0;
}
// Model requests: every float 5.0 (reference src/lib_loadgen/ort_client.cc:10-22).
static inline int const_float_fill(uint8_t* p, size_t n, uint64_t) {
  float* f = reinterpret_cast<float*>(p);
  for (size_t i = 0; i < n / 4; i++) f[i] = 5.0f;
  return 0;
}
// Seeded uniform [0,1) floats, one stream per request index.
static inline int uniform_float_fill(uint8_t* p, size_t n, uint64_t seq) {
  SrpcRng r(0x51ED2701ull * (seq + 1) + 12345);
  float* f = reinterpret_cast<float*>(p);
  for (size_t i = 0; i < n / 4; i++) f[i] = (float)r.uniform();
  return 0;
}

// Seeded token ids: int32 uniform over a 30522-word vocabulary.
static inline int token_ids_fill(uint8_t* p, size_t n, uint64_t seq) {
  SrpcRng r(0xB5297A4Dull * (seq + 1) + 777);
  int32_t* ids = reinterpret_cast<int32_t*>(p);
  for (size_t i = 0; i < n / 4; i++) ids[i] = (int32_t)(r.next() % 30522u);
  return 0;
}
// Seeded standard-normal floats (Box-Muller), one stream per request index.
static inline int normal_float_fill(uint8_t* p, size_t n, uint64_t seq) {
  SrpcRng r(0x2545F491ull * (seq + 1) + 4242);
  float* f = reinterpret_cast<float*>(p);
  size_t m = n / 4;
  for (size_t i = 0; i < m; i += 2) {
    double u1 = r.uniform(), u2 = r.uniform();
    if (u1 < 1e-300) u1 = 1e-300;
    double rad = std::sqrt(-2.0 * std::log(u1));
    f[i] = (float)(rad * std::cos(6.283185307179586 * u2));
    if (i + 1 < m) f[i + 1] = (float)(rad * std::sin(6.283185307179586 * u2));
  }
  return 0;
}

// ------------------------------------------------------------------ client
enum R_STATES : uint32_t { R_CREATE = 0, R_SENT, R_RECV, R_ERROR };

struct CallToken {
  std::atomic<uint32_t> call_state{R_CREATE};
  bool warmup = false;
  uint32_t payload_idx = 0;
  uint64_t dispatchNs = 0, completionNs = 0;
  uint32_t resp_bytes = 0;
  uint32_t verify_rc = 0;
};

struct ClientConfig {
  std::string client_uri = "b8:ce:f6:cc:6a:53,192.168.25.2,50052,b8:ce:f6:cc:6a:52,192.168.25.1,50051";
  size_t req_size = 1024, resp_size = 1024;
  uint64_t total_requests = 100;
  uint64_t num_warmup = 10;
  int n_payloads = 16;       // distinct pre-built request payloads
  bool verify = false;
  std::string exp_name = "splitrpc";
  std::string out_dir = ".";
  uint64_t seed = 12345;
  uint64_t drain_timeout_ns = 10000000000ull;  // give up waiting for replies after this long
  bool send_by_reference = false;  // payload pool in pinned memory, handed to the transport without a host copy
};

class P2pRpcAppClient {
  Transport* port_;
  ClientConfig cfg_;
  p2p_rpc_conn_info* conn_;
  std::vector<CallToken> tokens_;
  std::vector<std::vector<uint8_t>> payloads_;
  std::vector<uint8_t*> payload_ptrs_;   // where each payload lives (own vector, or the pinned pool)
  uint8_t* pinned_pool_ = nullptr;
  std::vector<std::vector<uint8_t>> resp_bufs_;      // reassembly buffer per token
  std::atomic<uint64_t> n_sent_{0}, n_recv_{0}, n_bad_token_{0}, n_verify_fail_{0}, next_idx_{0};
  std::atomic<bool> exit_flag_{false};
  std::atomic<int> issuing_{0};  // send_next() calls between taking a call number and having sent it
  std::thread listener_;
  app_req_cb req_cb_;
  app_resp_cb resp_cb_;
  int closed_outstanding_ = 0;
  size_t n_frags_, mtu_;
  StatsManager stats_;

  bool token_ok(uint64_t tok, size_t* idx) const {
    uintptr_t base = (uintptr_t)tokens_.data();
    if (tok < base || tok >= base + tokens_.size() * sizeof(CallToken)) return false;
    if ((tok - base) % sizeof(CallToken)) return false;
    *idx = (tok - base) / sizeof(CallToken);
    return true;
  }

 public:
  P2pRpcAppClient(Transport* port, const ClientConfig& cfg, app_req_cb req_cb = echo_fill, app_resp_cb resp_cb = nullptr)
      : port_(port),
        cfg_(cfg),
        conn_(initialize_client_conn_info(cfg.client_uri)),
        tokens_(cfg.total_requests + 1),
        req_cb_(std::move(req_cb)),
        resp_cb_(std::move(resp_cb)),
        n_frags_(num_fragments(cfg.req_size, rpc_mtu())),
        mtu_(rpc_mtu()),
        stats_(cfg.exp_name, cfg.out_dir) {}
  ~P2pRpcAppClient() {
    stop_listener();
    if (pinned_pool_)
      if (const SrpcDeviceOps* ops = srpc_cuda_ops()) ops->host_free(pinned_pool_);
    release_conn_info(conn_);
  }
  std::string getName() const { return "P2pRpcAppClient"; }
  StatsManager& stats() { return stats_; }
  uint64_t sent() const { return n_sent_.load(); }
  uint64_t received() const { return n_recv_.load(); }
  uint64_t verify_failures() const { return n_verify_fail_.load(); }
  uint64_t bad_tokens() const { return n_bad_token_.load(); }
  const std::vector<uint8_t>& payload(int i) const { return payloads_[i]; }
  const std::vector<uint8_t>& response(uint64_t call) const { return resp_bufs_[call]; }

  // Builds the request payloads and marks the warm-up calls.
  void PreProcessRequests() {
    payloads_.resize((size_t)cfg_.n_payloads);
    payload_ptrs_.resize((size_t)cfg_.n_payloads);
    DmaRegion region;
    if (cfg_.send_by_reference && port_->alloc_dma_region(((cfg_.req_size + 255) / 256 * 256) * (size_t)cfg_.n_payloads, &region)) {
      // memory of the receiving port: it can share it with the processes that serve its requests
      size_t stride = (cfg_.req_size + 255) / 256 * 256;
      for (int i = 0; i < cfg_.n_payloads; i++) payload_ptrs_[i] = region.host_base + (size_t)i * stride;
    } else if (cfg_.send_by_reference) {
      const SrpcDeviceOps* ops = srpc_cuda_ops();
      void *h = nullptr, *d = nullptr;
      size_t stride = (cfg_.req_size + 255) / 256 * 256;
      if (!ops || ops->host_alloc_mapped(stride * (size_t)cfg_.n_payloads, &h, &d) != 0 || h != d) {
        srpc_log(SRPC_LOG_WARN, "send_by_reference needs pinned memory with unified addressing; copying instead");
        if (h) ops->host_free(h);
        cfg_.send_by_reference = false;
      } else {
        pinned_pool_ = (uint8_t*)h;
        for (int i = 0; i < cfg_.n_payloads; i++) payload_ptrs_[i] = pinned_pool_ + (size_t)i * stride;
      }
    }
    for (int i = 0; i < cfg_.n_payloads; i++) {
      payloads_[i].resize(cfg_.req_size);
      req_cb_(payloads_[i].data(), cfg_.req_size, (uint64_t)i);
      if (cfg_.send_by_reference) std::memcpy(payload_ptrs_[i], payloads_[i].data(), cfg_.req_size);
      else payload_ptrs_[i] = payloads_[i].data();
    }
    resp_bufs_.resize(tokens_.size());
    for (size_t i = 0; i < tokens_.size(); i++) {
      tokens_[i].warmup = i < cfg_.num_warmup;
      tokens_[i].payload_idx = (uint32_t)(i % (size_t)cfg_.n_payloads);
      if (cfg_.verify) resp_bufs_[i].resize(cfg_.resp_size);
    }
  }

  // Sends request number `idx` (all fragments in one burst).  Returns false when
  // the transport refused it (receiver arena full); the caller may retry.
  bool SchedRequest(uint64_t idx) {
    CallToken& t = tokens_[idx];
    const uint8_t* pl = payload_ptrs_[t.payload_idx];
    std::vector<p2p_rpc_hdr> hdrs(n_frags_);
    std::vector<const uint8_t*> ptrs(n_frags_);
    std::vector<uint32_t> lens(n_frags_);
    size_t left = cfg_.req_size;
    for (size_t i = 0; i < n_frags_; i++) {
      size_t len = left < mtu_ ? left : mtu_;
      fill_frag_hdr(&hdrs[i], conn_, (uint64_t)(uintptr_t)&t, (uint16_t)i, (uint16_t)len, false);
      ptrs[i] = pl + i * mtu_;
      lens[i] = (uint32_t)len;
      left -= len;
    }
    t.dispatchNs = getCurNs();
    t.call_state.store(R_SENT, std::memory_order_release);
    int rc = cfg_.send_by_reference ? port_->tx_ref(hdrs.data(), ptrs.data(), lens.data(), (int)n_frags_)
                                    : port_->tx_copy(hdrs.data(), ptrs.data(), lens.data(), (int)n_frags_);
    if (rc <= 0) {
      t.call_state.store(R_CREATE, std::memory_order_release);
      return false;
    }
    n_sent_++;
    return true;
  }

  // Takes the next call number and sends it.  `issuing_` covers the gap between taking the last number and counting
  // the call as sent: without it drain() could see "all numbers taken, as many replies as sends" in that gap and end the
  // run one reply short.
  bool send_next() {
    issuing_.fetch_add(1);
    uint64_t idx = next_idx_.fetch_add(1);
    bool sent = false;
    if (idx < cfg_.total_requests) {
      uint64_t t0 = getCurNs();
      sent = true;
      while (!SchedRequest(idx)) {
        if (exit_flag_.load() || getCurNs() - t0 > cfg_.drain_timeout_ns) {
          sent = false;
          break;
        }
        std::this_thread::yield();
      }
    }
    issuing_.fetch_sub(1);
    return sent;
  }

  // Receives reply fragments, reassembles by token, stamps completion; in closed
  // loop mode every completion issues the next request.
  void CompleteReqListener() {
    std::vector<SrpcPkt> pkts(256);
    std::unordered_map<uint64_t, uint32_t> got;  // token -> bytes so far
    IdleBackoff backoff;
    while (!exit_flag_.load(std::memory_order_acquire)) {
      int n = port_->rx_burst(pkts.data(), (int)pkts.size());
      if (n > 0) backoff.busy();
      else backoff.empty();
      for (int i = 0; i < n; i++) {
        SrpcPkt& p = pkts[i];
        size_t idx = 0;
        uint64_t tok = p.hdr->req_token;
        if (!token_ok(tok, &idx) || tokens_[idx].call_state.load(std::memory_order_acquire) != R_SENT) {
          n_bad_token_++;
          continue;
        }
        CallToken& t = tokens_[idx];
        if (cfg_.verify) {
          size_t off = (size_t)p.hdr->seq_num * mtu_;
          if (off + p.len <= cfg_.resp_size) std::memcpy(resp_bufs_[idx].data() + off, p.payload, p.len);
        }
        uint32_t total = (got[tok] += p.len);
        if (total >= cfg_.resp_size) {
          got.erase(tok);
          t.completionNs = getCurNs();
          t.resp_bytes = total;
          if (cfg_.verify && resp_cb_) {
            t.verify_rc = (uint32_t)resp_cb_(payloads_[t.payload_idx].data(), resp_bufs_[idx].data(), cfg_.resp_size);
            if (t.verify_rc) n_verify_fail_++;
          }
          t.call_state.store(R_RECV, std::memory_order_release);
          n_recv_++;
          if (closed_outstanding_ > 0) send_next();
        }
      }
      if (n > 0) port_->release_rx(pkts.data(), n);
    }
  }

  void start_listener() {
    exit_flag_.store(false);
    listener_ = std::thread([this] { CompleteReqListener(); });
  }
  void stop_listener() {
    exit_flag_.store(true, std::memory_order_release);
    if (listener_.joinable()) listener_.join();
  }
  // Makes a CompleteReqListener() that runs on a thread of the caller's return.
  void request_exit() { exit_flag_.store(true, std::memory_order_release); }

  // Waits (bounded) until every issued request was answered.
  bool drain() {
    uint64_t t0 = getCurNs();
    while (!(next_idx_.load() >= cfg_.total_requests && issuing_.load() == 0 && n_recv_.load() >= n_sent_.load())) {
      if (getCurNs() - t0 > cfg_.drain_timeout_ns) return false;
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    return true;
  }

  // Closed loop: `outstanding` requests in flight until total_requests were sent.
  bool run_closed_loop(int outstanding) {
    closed_outstanding_ = outstanding;
    start_listener();
    for (int i = 0; i < outstanding; i++) send_next();
    bool ok = drain();
    stop_listener();
    return ok;
  }

  // Open loop: arrival schedule at `rate` requests/s with the given CoV, issued
  // by `n_threads` generator threads.
  bool run_open_loop(double rate, int cov, int n_threads = 1) {
    closed_outstanding_ = 0;
    std::vector<uint64_t> sched(cfg_.total_requests);
    LoadGenerator lg(1.0 / rate, cov, cfg_.seed);
    uint64_t t = getCurNs() + 2000000;
    for (auto& s : sched) s = t = lg.nextReqArr(t, false);
    start_listener();
    std::vector<std::thread> gens;
    for (int g = 0; g < n_threads; g++)
      gens.emplace_back([this, &sched, g, n_threads] {
        for (uint64_t i = (uint64_t)g; i < cfg_.total_requests; i += (uint64_t)n_threads) {
          sleepUntil(sched[i]);
          uint64_t t0 = getCurNs();
          while (!SchedRequest(i)) {
            if (getCurNs() - t0 > 100000000ull) break;  // receiver stuck: skip this arrival
          }
        }
      });
    for (auto& th : gens) th.join();
    next_idx_.store(cfg_.total_requests);
    bool ok = drain();
    stop_listener();
    return ok;
  }

  // Computes sojourn times and throughput over the non-warm-up calls.
  std::map<std::string, double> PostProcessResponses() {
    uint64_t recorded = 0, warm = 0, bad = 0, first = UINT64_MAX, last = 0;
    stats_.resetStats();
    for (size_t i = 0; i < cfg_.total_requests; i++) {
      CallToken& t = tokens_[i];
      if (t.call_state.load() != R_RECV) {
        bad++;
        continue;
      }
      if (t.warmup) {
        warm++;
        continue;
      }
      first = std::min(first, t.dispatchNs);
      last = std::max(last, t.completionNs);
      stats_.recordEvent("sojournTime", t.completionNs - t.dispatchNs);
      recorded++;
    }
    double thr = (recorded && last > first) ? (double)recorded / ((double)(last - first) / 1e9) : 0.0;
    stats_.trackStatInfo("firstReqDispatchNs", (double)first);
    stats_.trackStatInfo("lastReqComplNs", (double)last);
    stats_.trackStatInfo("throughput_est", thr);
    stats_.trackStatInfo("n_r_sent", (double)n_sent_.load());
    stats_.trackStatInfo("n_r_recv", (double)n_recv_.load());
    stats_.trackStatInfo("recorded", (double)recorded);
    stats_.trackStatInfo("warmup_calls", (double)warm);
    stats_.trackStatInfo("incorrect_state_calls", (double)bad);
    stats_.trackStatInfo("verify_failures", (double)n_verify_fail_.load());
    stats_.trackStatInfo("exp_name", cfg_.exp_name);
    return stats_.aggregate();
  }
};
