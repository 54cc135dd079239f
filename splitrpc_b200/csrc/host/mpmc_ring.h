// Bounded lock-free multi-producer/multi-consumer ring of trivially copyable items.
//
// Replaces the DPDK rte_ring / moodycamel queues the original pools are built on
// (reference src/p2p_rpc_rr_pool_ng.h:12-40, src/udp_rr.h:277-300) with a
// self-contained sequence-number ring: each cell carries a ticket that says
// whether it is ready for the producer or the consumer of a given lap.
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <new>

template <typename T>
class MpmcRing {
  struct Cell {
    std::atomic<size_t> seq;
    T value;
  };
  static constexpr size_t kLine = 64;
  std::unique_ptr<Cell[]> cells_;
  size_t mask_;
  alignas(kLine) std::atomic<size_t> head_{0};  // next ticket to enqueue
  alignas(kLine) std::atomic<size_t> tail_{0};  // next ticket to dequeue

  static size_t pow2_at_least(size_t n) {
    size_t p = 2;
    while (p < n) p <<= 1;
    return p;
  }

 public:
  explicit MpmcRing(size_t capacity) {
    size_t n = pow2_at_least(capacity);
    cells_.reset(new Cell[n]);
    mask_ = n - 1;
    for (size_t i = 0; i < n; i++) cells_[i].seq.store(i, std::memory_order_relaxed);
  }
  MpmcRing(const MpmcRing&) = delete;
  MpmcRing& operator=(const MpmcRing&) = delete;

  size_t capacity() const { return mask_ + 1; }

  bool push(const T& v) {
    size_t pos = head_.load(std::memory_order_relaxed);
    for (;;) {
      Cell& c = cells_[pos & mask_];
      size_t seq = c.seq.load(std::memory_order_acquire);
      intptr_t dif = (intptr_t)seq - (intptr_t)pos;
      if (dif == 0) {
        if (head_.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
          c.value = v;
          c.seq.store(pos + 1, std::memory_order_release);
          return true;
        }
      } else if (dif < 0) {
        return false;  // full
      } else {
        pos = head_.load(std::memory_order_relaxed);
      }
    }
  }

  bool pop(T& out) {
    size_t pos = tail_.load(std::memory_order_relaxed);
    for (;;) {
      Cell& c = cells_[pos & mask_];
      size_t seq = c.seq.load(std::memory_order_acquire);
      intptr_t dif = (intptr_t)seq - (intptr_t)(pos + 1);
      if (dif == 0) {
        if (tail_.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
          out = c.value;
          c.seq.store(pos + mask_ + 1, std::memory_order_release);
          return true;
        }
      } else if (dif < 0) {
        return false;  // empty
      } else {
        pos = tail_.load(std::memory_order_relaxed);
      }
    }
  }

  // Approximate under concurrency; exact when quiescent.
  size_t size() const {
    size_t h = head_.load(std::memory_order_acquire), t = tail_.load(std::memory_order_acquire);
    return h >= t ? h - t : 0;
  }
  bool empty() const { return size() == 0; }
};
