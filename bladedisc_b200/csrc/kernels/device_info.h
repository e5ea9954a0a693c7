// Per-device facts the launch code asks for on every call.  A process may
// drive several GPUs (a context names its device), so nothing here is cached
// per process: the cache is indexed by the ordinal of the current device.
#pragma once
#include <cuda_runtime.h>

#include <atomic>

namespace disc_b200 {

constexpr int kMaxDeviceOrdinals = 64;

inline int current_device_ordinal() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDeviceOrdinals) return 0;
  return dev;
}

// Number of SMs of the current device (148 on a B200; that value also stands
// in when the query fails).
inline int device_sm_count() {
  static std::atomic<int> cache[kMaxDeviceOrdinals];
  const int dev = current_device_ordinal();
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace disc_b200
