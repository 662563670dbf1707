// Host-side helpers of the launchers: per-device facts are looked up once, not on every call (a decode step launches these
// kernels every few tens of microseconds).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

namespace dsa {

// Ordinal and SM count of the current device (the count is cached per ordinal).
inline cudaError_t current_device_sms(int* dev, int* sms) {
  constexpr int kMax = 64;
  static int cached[kMax] = {0};
  static std::mutex mu;
  cudaError_t e = cudaGetDevice(dev);
  if (e != cudaSuccess) return e;
  if (*dev >= 0 && *dev < kMax) {
    std::lock_guard<std::mutex> lock(mu);
    if (cached[*dev] == 0) {
      int n = 0;
      if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, *dev)) != cudaSuccess) return e;
      cached[*dev] = n;
    }
    *sms = cached[*dev];
    return cudaSuccess;
  }
  return cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, *dev);
}

// Makes sure `kernel` may use `bytes` of dynamic shared memory on device `dev`: cudaFuncSetAttribute is called only when
// the value asked for exceeds what was set before for this (kernel, device).
template <typename Kernel>
cudaError_t ensure_dynamic_smem(Kernel kernel, int dev, int bytes) {
  static std::unordered_map<uint64_t, int> done;
  static std::mutex mu;
  const uint64_t key = (static_cast<uint64_t>(reinterpret_cast<uintptr_t>(kernel)) << 6) ^ static_cast<uint64_t>(dev & 63);
  std::lock_guard<std::mutex> lock(mu);
  auto it = done.find(key);
  if (it != done.end() && it->second >= bytes) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[key] = bytes;
  return e;
}

}  // namespace dsa
