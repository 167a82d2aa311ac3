// Host-side helpers shared by all launchers: error checks, device queries and
// the process-wide count of kernel launches issued by this library.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <stdexcept>
#include <string>

namespace b200 {

inline void check_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

inline int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

std::atomic<long long>& launch_counter();

inline void count_launch(int n = 1) { launch_counter().fetch_add(n, std::memory_order_relaxed); }

}  // namespace b200
