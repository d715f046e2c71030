// Host-side launch helper shared by the exchange kernels: how many CTAs of a kernel the current device
// can hold at once. The exchange kernels walk task lists in which a wait may depend on work that sits in
// another CTA of the same launch, so a launch must never be larger than that number (and a cooperative
// launch is refused if it is). The answer is cached per (kernel, device).
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <utility>

namespace nangila {

// Also opts the kernel in to `smem` bytes of dynamic shared memory.
inline cudaError_t resident_ctas(const void* fn, int threads, size_t smem, int* out) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, int> cache;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find({fn, dev});
  if (it != cache.end()) {
    *out = it->second;
    return cudaSuccess;
  }
  if (smem > 0) {  // static shared memory counts towards the 48 KB default limit too: always opt in
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
  }
  int per_sm = 0, sms = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, smem);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  *out = std::max(1, per_sm * sms);
  cache[{fn, dev}] = *out;
  return cudaSuccess;
}

// CTAs per rank for a launch that emulates `nvr` ranks: `want` (<= 0: as many as fit) clamped to residency.
inline cudaError_t clamp_grid(const void* fn, int threads, size_t smem, int want, int nvr, int* grid_x) {
  int resident = 0;
  cudaError_t e = resident_ctas(fn, threads, smem, &resident);
  if (e != cudaSuccess) return e;
  const int cap = std::max(1, resident / std::max(1, nvr));
  *grid_x = want > 0 ? std::min(want, cap) : cap;
  return cudaSuccess;
}

}  // namespace nangila
