// Host-side helpers shared by the kernel launchers.
#pragma once
#include <cuda_runtime.h>

namespace mdt {
// Number of SMs of the current device (grids are sized in multiples of it); cached per device ordinal.
inline int sm_count_of_current_device() {
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
    cache[dev] = n;
  }
  return cache[dev];
}
}  // namespace mdt
