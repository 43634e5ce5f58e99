// Small host-side helpers shared by the kernel launchers.
#pragma once
#include <cuda_runtime.h>

namespace fa2 {

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel instantiation and device
// instead of on every launch (the call is idempotent, so a race between two host threads that
// both find the flag clear is harmless).
template <class Kernel>
static cudaError_t opt_in_dynamic_smem(Kernel kern, int bytes, bool (&done)[64]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev >= 0 && done[dev]) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && dev >= 0) done[dev] = true;
  return e;
}

// Streaming multiprocessors of the current device (cached per device; 148 if it cannot be read).
inline int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace fa2
