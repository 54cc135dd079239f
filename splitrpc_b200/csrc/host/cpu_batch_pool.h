// Fork-join helper threads for short host-side loops: the requests of a batch of a CPU app, the fragment copies of
// an emulated NIC DMA burst.
//
// run(n, fn) calls fn(i) for every i in [0, n): the index range is cut into equal shares, the caller takes the first
// and every helper one of the others, and run() returns when all shares are done.  The hand-over is a generation
// counter that the helpers poll for a short while after each job (jobs come in bursts, and waking a sleeping thread
// takes longer than a small job) before they go to sleep on a condition variable; no lock is taken on the polling
// path.  One caller at a time.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

class CpuBatchPool {
 public:
  explicit CpuBatchPool(int helpers) : parts_(helpers > 0 ? helpers + 1 : 1) {
    for (int h = 0; h < helpers; h++) threads_.emplace_back([this, h] { loop(h + 1); });
  }
  ~CpuBatchPool() {
    stop_.store(true);
    gen_.fetch_add(1);
    {
      std::lock_guard<std::mutex> g(mu_);
      cv_.notify_all();
    }
    for (auto& t : threads_) t.join();
  }
  CpuBatchPool(const CpuBatchPool&) = delete;
  int helpers() const { return parts_ - 1; }

  template <class F>
  void run(int n, F&& fn) {
    const int parts = parts_;
    if (n <= 1 || parts == 1) {
      for (int i = 0; i < n; i++) fn(i);
      return;
    }
    std::function<void(int)> f = std::ref(fn);
    fn_ = &f;
    n_ = n;
    done_.store(0, std::memory_order_relaxed);
    gen_.fetch_add(1);  // publishes fn_ / n_ (sequentially consistent, paired with the sleepers_ protocol below)
    if (sleepers_.load() > 0) {
      std::lock_guard<std::mutex> g(mu_);
      cv_.notify_all();
    }
    share(0, parts, n, f);
    const int helpers = parts - 1;
    for (uint32_t spins = 1; done_.load(std::memory_order_acquire) != helpers; spins++) {
      if ((spins & 1023) == 0) std::this_thread::yield();
      else relax();
    }
  }

 private:
  static void relax() {
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#endif
  }
  static void share(int part, int parts, int n, const std::function<void(int)>& f) {
    const int lo = (int)((int64_t)n * part / parts), hi = (int)((int64_t)n * (part + 1) / parts);
    for (int i = lo; i < hi; i++) f(i);
  }
  void loop(int part) {
    uint64_t seen = 0;
    for (;;) {
      const auto t0 = std::chrono::steady_clock::now();
      bool changed = false;
      for (uint32_t spins = 1;; spins++) {
        if (gen_.load(std::memory_order_acquire) != seen) {
          changed = true;
          break;
        }
        if ((spins & 63) == 0 && std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(kSpinUs)) break;
        relax();
      }
      if (!changed) {
        std::unique_lock<std::mutex> lk(mu_);
        sleepers_.fetch_add(1);
        cv_.wait(lk, [&] { return gen_.load() != seen; });
        sleepers_.fetch_sub(1);
      }
      seen = gen_.load(std::memory_order_acquire);
      if (stop_.load()) return;
      // every helper takes part in every job, so fn_ / n_ stay valid until this share has been counted
      share(part, parts_, n_, *fn_);
      done_.fetch_add(1, std::memory_order_release);
    }
  }

  const int parts_;  // the caller and the helpers
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable cv_;
  const std::function<void(int)>* fn_ = nullptr;
  int n_ = 0;
  std::atomic<int> done_{0}, sleepers_{0};
  std::atomic<uint64_t> gen_{0};
  std::atomic<bool> stop_{false};
  static constexpr int kSpinUs = 100;
};
