// Environment-variable configuration, logging and small timing/statistics helpers.
//
// Every tunable of the stack is an environment variable with the same name and
// default as the original system (reference src/utils/config_utils.h:15-100), so
// existing launch scripts keep working.  Values are read through readEnvInfo<T>,
// which logs each read once at INFO level.  Unlike the original, RPC_MTU is not
// frozen in a static initialiser: rpc_mtu() reads P2P_RPC_MTU on first use and
// set_rpc_mtu() lets tests and embedding code change it.
#pragma once

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#define ACCESS_ONCE(x) (*(volatile decltype(x)*)&(x))

// ------------------------------------------------------------------ logging
enum SrpcLogLevel { SRPC_LOG_TRACE = 0, SRPC_LOG_DEBUG, SRPC_LOG_INFO, SRPC_LOG_WARN, SRPC_LOG_ERROR, SRPC_LOG_OFF };

inline std::atomic<int>& srpc_log_level_ref() {
  static std::atomic<int> lvl{[] {
    const char* e = std::getenv("P2P_RPC_LOG_LEVEL");
    if (!e) return (int)SRPC_LOG_WARN;
    std::string s(e);
    if (s == "trace") return (int)SRPC_LOG_TRACE;
    if (s == "debug") return (int)SRPC_LOG_DEBUG;
    if (s == "info") return (int)SRPC_LOG_INFO;
    if (s == "warn") return (int)SRPC_LOG_WARN;
    if (s == "error") return (int)SRPC_LOG_ERROR;
    if (s == "off") return (int)SRPC_LOG_OFF;
    return (int)SRPC_LOG_WARN;
  }()};
  return lvl;
}
inline void srpc_set_log_level(int lvl) { srpc_log_level_ref().store(lvl); }

inline void srpc_log(int lvl, const char* fmt, ...) {
  if (lvl < srpc_log_level_ref().load(std::memory_order_relaxed)) return;
  static const char* names[] = {"trace", "debug", "info", "warn", "error"};
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  std::fprintf(stderr, "[splitrpc %s] %s\n", names[lvl < 5 ? lvl : 4], buf);
}

#ifdef TRACE_MODE
#define TRACE_PRINTF(...) std::fprintf(stderr, __VA_ARGS__)
#else
#define TRACE_PRINTF(...) ((void)0)
#endif

// ------------------------------------------------------------------ env
template <typename T>
inline T srpc_parse(const std::string& s) {
  std::istringstream is(s);
  T v{};
  is >> v;
  return v;
}
template <>
inline std::string srpc_parse<std::string>(const std::string& s) { return s; }

template <typename T>
inline T readEnvInfo(const char* name, T def) {
  const char* e = std::getenv(name);
  T v = e ? srpc_parse<T>(std::string(e)) : def;
  if (srpc_log_level_ref().load() <= SRPC_LOG_INFO) {
    std::ostringstream os;
    os << name << " = " << v << (e ? "" : " (default)");
    srpc_log(SRPC_LOG_INFO, "%s", os.str().c_str());
  }
  return v;
}

static inline std::string get_p2p_path() { return readEnvInfo<std::string>("P2P_PATH", "./"); }
static inline std::string get_dataset_path() { return readEnvInfo<std::string>("P2P_DATA_SET_PATH", "../test_files/"); }
static inline int get_cuda_device_id() { return readEnvInfo<int>("P2P_RPC_CUDA_DEVICE_ID", 0); }
static inline size_t get_req_size() { return readEnvInfo<size_t>("P2P_RPC_REQ_SIZE", 1024); }
static inline size_t get_resp_size() { return readEnvInfo<size_t>("P2P_RPC_RESP_SIZE", 1024); }
static inline std::string get_server_mac() { return readEnvInfo<std::string>("P2P_RPC_SERVER_MAC", "b8:ce:f6:cc:6a:52"); }
static inline std::string get_server_ip() { return readEnvInfo<std::string>("P2P_RPC_SERVER_IP", "192.168.25.1"); }
static inline std::string get_server_port() { return readEnvInfo<std::string>("P2P_RPC_SERVER_PORT", "50051"); }
static inline std::string get_client_ip() { return readEnvInfo<std::string>("P2P_RPC_CLIENT_IP", "192.168.25.2"); }
static inline std::string get_client_port() { return readEnvInfo<std::string>("P2P_RPC_CLIENT_PORT", "50052"); }
static inline std::string get_ort_model_name() { return readEnvInfo<std::string>("P2P_RPC_ORT_MODEL_NAME", "resnet50v2batched.onnx"); }
static inline int get_ort_batch_size() { return readEnvInfo<int>("P2P_RPC_ORT_BATCH_SIZE", 1); }
// 0 = copy-engine DMA per run, 1 = persistent gather kernel, 2 = one kernel per list, 3 = device memcpy
static inline int get_gpu_copy_type() { return readEnvInfo<int>("P2P_RPC_GPU_COPY_TYPE", 1); }
static inline int get_zerocopy_mode() { return readEnvInfo<int>("P2P_RPC_ZEROCOPY_MODE", 0); }
// 0 = fixed-batch sync, 1 = async (GPU-armed), 2 = dynamic batching
static inline int get_server_mode() { return readEnvInfo<int>("P2P_RPC_SERVER_MODE", 0); }
// 0 none, 1 kernel launches, 2 device-side launch (not available on sm_100), 3 persistent kernel, 4 CUDA graph
static inline int get_work_launch_type() { return readEnvInfo<int>("P2P_RPC_WORK_LAUNCH_TYPE", 1); }
static inline int get_dpdk_port() { return readEnvInfo<int>("P2P_RPC_DPDK_PORT", 0); }
static inline int get_dpdk_mem_alloc_type() { return readEnvInfo<int>("P2P_RPC_DPDK_MEM_ALLOC_TYPE", 0); }
static inline int get_g_pp_launch_type() { return readEnvInfo<int>("P2P_RPC_G_PP_LAUNCH_TYPE", 2); }

inline std::atomic<size_t>& srpc_mtu_ref() {
  static std::atomic<size_t> mtu{readEnvInfo<size_t>("P2P_RPC_MTU", 1024)};
  return mtu;
}
// Payload bytes carried by one packet; the frame on the wire is rpc_mtu() + 64.
static inline size_t rpc_mtu() { return srpc_mtu_ref().load(std::memory_order_relaxed); }
static inline void set_rpc_mtu(size_t v) { srpc_mtu_ref().store(v); }
#define RPC_MTU (rpc_mtu())

// ------------------------------------------------------------------ time
static inline uint64_t getCurNs() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

// Sleeps most of the way, then spins the last 50 us, so open-loop arrivals are
// issued close to their scheduled instant without burning a core the whole time.
static inline void sleepUntil(uint64_t target_ns) {
  for (;;) {
    uint64_t now = getCurNs();
    if (now >= target_ns) return;
    uint64_t left = target_ns - now;
    if (left > 100000) std::this_thread::sleep_for(std::chrono::nanoseconds(left - 50000));
  }
}

// Polling loops spin while there is work and back off to short sleeps after a run of empty polls, so that an idle
// server (or several servers on one host) does not burn a core per thread.  P2P_RPC_IDLE_SPIN sets how many empty
// polls are tolerated before sleeping (0 = always spin).
struct IdleBackoff {
  int limit;
  int idle = 0;
  IdleBackoff() : limit(spin_limit()) {}
  static int spin_limit() {
    static int v = readEnvInfo<int>("P2P_RPC_IDLE_SPIN", 4000);
    return v;
  }
  void busy() { idle = 0; }
  void empty() {
    if (limit > 0 && ++idle > limit) {
      std::this_thread::sleep_for(std::chrono::microseconds(20));
    } else {
#if defined(__x86_64__)
      __builtin_ia32_pause();
#endif
    }
  }
};

// ------------------------------------------------------------------ stats
// Percentile rule of the measurement protocol: element at index round(p*(n-1))
// of the sorted sample (reference src/utils/stats_utils.h:10-21).
static inline size_t getTailPercentileIndex(double p, uint64_t n) {
  if (n == 0) return 0;
  return (size_t)std::llround(p * (double)(n - 1));
}

static inline double getPercentile(std::vector<uint64_t>& v, double p) {
  if (v.empty()) return 0.0;
  size_t idx = getTailPercentileIndex(p, v.size());
  if (idx >= v.size()) return 0.0;
  std::nth_element(v.begin(), v.begin() + idx, v.end());
  return (double)v[idx];
}

static inline double getMean(const std::vector<uint64_t>& v) {
  double mean = 0.0;
  uint64_t k = 0;
  for (uint64_t x : v) mean += ((double)x - mean) / (double)(++k);
  return mean;
}

template <typename T>
class Measure {
  std::string name_;
  std::vector<T> samples_;

 public:
  explicit Measure(std::string n) : name_(std::move(n)) {}
  void add(T v) { samples_.push_back(v); }
  std::vector<T>& getRawMeasurements() { return samples_; }
  void clear() { samples_.clear(); }
  size_t numMeasurements() const { return samples_.size(); }
  const std::string& name() const { return name_; }
  void dumpStatsToFile(const std::string& exp_name, const std::string& dir = ".") {
    std::ofstream out(dir + "/raw_" + name_ + "_" + exp_name + ".stat");
    for (const auto& s : samples_) out << s << "\n";
  }
};

static inline std::string format_stat(const std::string& key, std::vector<uint64_t> v) {
  uint64_t mn = 0, mx = 0;
  if (!v.empty()) {
    mn = *std::min_element(v.begin(), v.end());
    mx = *std::max_element(v.begin(), v.end());
  }
  char buf[512];
  std::snprintf(buf, sizeof(buf),
                "%s stats(ns) [N, Mean, p90, p95, p99, min, max]: %zu, %0.2f, %0.2f, %0.2f, %0.2f, %lu, %lu",
                key.c_str(), v.size(), getMean(v), getPercentile(v, 0.90), getPercentile(v, 0.95),
                getPercentile(v, 0.99), (unsigned long)mn, (unsigned long)mx);
  return std::string(buf);
}
static inline void print_stat(const std::string& key, const std::vector<uint64_t>& v) {
  std::printf("%s\n", format_stat(key, v).c_str());
}

// Per-stage wall-clock timers, compiled in only with -DPROFILE_MODE.
#ifdef PROFILE_MODE
#define PROF_DECL(name) uint64_t name##_t0 = 0; std::vector<uint64_t> name##_samples
#define PROF_START(name) name##_t0 = getCurNs()
#define PROF_STOP(name) name##_samples.push_back(getCurNs() - name##_t0)
#define PROF_PRINT(label, name) print_stat(label, name##_samples)
#else
#define PROF_DECL(name)
#define PROF_START(name) ((void)0)
#define PROF_STOP(name) ((void)0)
#define PROF_PRINT(label, name) ((void)0)
#endif

// NVTX ranges on the host threads (receive, shunter, worker), compiled in with -DPROFILE_MODE like the timers above
// (reference src/utils/time_utils.h:16-38).  NVTX 3 is header-only; without a profiler attached the calls are no-ops.
#if defined(PROFILE_MODE) && defined(__has_include)
#if __has_include(<nvtx3/nvToolsExt.h>)
#include <nvtx3/nvToolsExt.h>
#define SRPC_HAVE_NVTX 1
#endif
#endif
#ifdef SRPC_HAVE_NVTX
#define NVTX_R(name) nvtxRangePushA(name)
#define NVTX_P() nvtxRangePop()
#define NVTX_M(name) nvtxMarkA(name)
#else
#define NVTX_R(name) ((void)0)
#define NVTX_P() ((void)0)
#define NVTX_M(name) ((void)0)
#endif

// Seeded xorshift generator used by payload generators and arrival processes so
// that every run with the same P2P_RPC_RANDOM_SEED produces the same bytes.
struct SrpcRng {
  uint64_t s;
  explicit SrpcRng(uint64_t seed = 12345) : s(seed ? seed : 0x9E3779B97F4A7C15ull) {}
  uint64_t next() {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    return s;
  }
  double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }
};
