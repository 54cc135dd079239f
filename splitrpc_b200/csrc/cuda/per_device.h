// "Once per device" state for kernel attributes: the opt-in to large dynamic shared memory and the like belong to a
// (function, device) pair, and one process may drive several GPUs.  The set-ups guarded by it are idempotent, so two
// threads that both find the flag clear may both run them.
#pragma once
#include <cuda_runtime.h>

#include <atomic>

struct PerDeviceFlag {
  std::atomic<unsigned char> done[64];  // static storage: zero-initialised
  static int current() {
    int d = 0;
    cudaGetDevice(&d);
    return d & 63;
  }
  bool needed(int d) const { return !done[d].load(std::memory_order_acquire); }
  void set(int d) { done[d].store(1, std::memory_order_release); }
};
