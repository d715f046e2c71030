// max |x|, an exact order statistic of |x| (by default the 99th percentile the host quantizer uses
// for its scale) and a 256-bin histogram of |x| / max, in one cooperative launch.
//
// Replaces find_max_abs_kernel + compute_gamma_simple_kernel (nangila-cuda/src/kernels/gamma.cu:18-36,
// :88-106: gamma = max/7), histogram_abs_kernel + host-side bin search (:42-82: p99 with 1/256
// resolution) and the host sort behind Quantizer::compute_gamma (nangila-core/src/quantizer.rs:81-96).
// Here the percentile is exact: the k-th largest |x| is found by a three-pass radix select.
// Output (float[4]): {max |x|, k-th largest |x|, gamma = max(kth / qmax, 1e-8), count of non-finite}.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nangila_kernels.h"
#include "quant.cuh"
#include "radix_select.cuh"

namespace cg = cooperative_groups;

namespace nangila {
namespace {

using namespace rsel;
constexpr int kThreads = 256;
constexpr int kH0 = 0, kH1 = kH0 + kBins0, kH2 = kH1 + kBins1, kLin = kH2 + kBins2, kMax = kLin + 256, kBad = kMax + 1;
constexpr int kWords = kBad + 7;

template <typename T>
__device__ __forceinline__ uint32_t abs_bits(const T* x, int64_t i, uint32_t& bad) {
  float f = dev::Vec16<T>::to_float(x[i]);
  uint32_t b = __float_as_uint(f) & 0x7fffffffu;
  if (b >= 0x7f800000u) {  // NaN / Inf count as zero, like the host quantizer
    ++bad;
    return 0u;
  }
  return b;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
absmax_hist_kernel(const T* __restrict__ x, int64_t n, uint32_t k, float qmax, uint32_t* scratch, float* out,
                   uint32_t* hist256) {
  cg::grid_group grid = cg::this_grid();
  __shared__ uint32_t sh[kBins0];
  __shared__ uint32_t sel[2];
  const int64_t t0 = int64_t(blockIdx.x) * kThreads + threadIdx.x, stride = int64_t(gridDim.x) * kThreads;
  for (int i = int(t0); i < kWords; i += int(stride)) scratch[i] = 0u;
  grid.sync();
  for (int i = threadIdx.x; i < kBins0; i += kThreads) sh[i] = 0u;
  __syncthreads();
  uint32_t mx = 0, bad = 0;
  for (int64_t i = t0; i < n; i += stride) {
    uint32_t b = abs_bits(x, i, bad);
    mx = max(mx, b);
    atomicAdd(&sh[b >> 20], 1u);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    bad += __shfl_xor_sync(0xffffffffu, bad, off);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMax(&scratch[kMax], mx);
    if (bad) atomicAdd(&scratch[kBad], bad);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kBins0; i += kThreads)
    if (sh[i]) atomicAdd(&scratch[kH0 + i], sh[i]);
  grid.sync();
  uint32_t want = k, b0, b1, b2, dummy = 0;
  select_bin(scratch + kH0, kBins0, want, b0, sel);
  for (int i = threadIdx.x; i < kBins1; i += kThreads) sh[i] = 0u;
  __syncthreads();
  for (int64_t i = t0; i < n; i += stride) {
    uint32_t b = abs_bits(x, i, dummy);
    if ((b >> 20) == b0) atomicAdd(&sh[(b >> 9) & 0x7ffu], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kBins1; i += kThreads)
    if (sh[i]) atomicAdd(&scratch[kH1 + i], sh[i]);
  grid.sync();
  select_bin(scratch + kH1, kBins1, want, b1, sel);
  const uint32_t prefix = (b0 << 11) | b1;
  const float vmax = __uint_as_float(scratch[kMax]);
  const float inv = vmax > 0.0f ? 255.999f / vmax : 0.0f;
  for (int i = threadIdx.x; i < kBins2 + 256; i += kThreads) sh[i] = 0u;
  __syncthreads();
  for (int64_t i = t0; i < n; i += stride) {
    uint32_t b = abs_bits(x, i, dummy);
    if ((b >> 9) == prefix) atomicAdd(&sh[b & 0x1ffu], 1u);
    atomicAdd(&sh[kBins2 + min(255, int(__uint_as_float(b) * inv))], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kBins2 + 256; i += kThreads)
    if (sh[i]) atomicAdd(&scratch[kH2 + i], sh[i]);  // kLin == kH2 + kBins2
  grid.sync();
  select_bin(scratch + kH2, kBins2, want, b2, sel);
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      const float kth = __uint_as_float((prefix << 9) | b2);
      out[0] = vmax;
      out[1] = kth;
      out[2] = fmaxf(kth / qmax, 1e-8f);
      out[3] = float(scratch[kBad]);
    }
    if (hist256 != nullptr)
      for (int i = threadIdx.x; i < 256; i += kThreads) hist256[i] = scratch[kLin + i];
  }
}

}  // namespace
}  // namespace nangila

extern "C" uint32_t nangila_absmax_scratch_words(void) { return nangila::kWords; }

// k: 1-based rank from the top of the order statistic wanted (k = n - floor(0.99 n) gives the host
// quantizer's p99). out: float[4]; hist256: 256 uint32 or NULL; scratch: nangila_absmax_scratch_words().
extern "C" int nangila_absmax_hist(const void* x, int32_t dtype, int64_t n, uint32_t k, float qmax, uint32_t* scratch,
                                   float* out, uint32_t* hist256, cudaStream_t stream) {
  using namespace nangila;
  if (x == nullptr || scratch == nullptr || out == nullptr || n <= 0 || n > 0x7fffffffll || k == 0 || k > n ||
      !(qmax > 0.0f))
    return int(cudaErrorInvalidValue);
  const void* fn;
  switch (dtype) {
    case NANGILA_F32: fn = reinterpret_cast<const void*>(&absmax_hist_kernel<float>); break;
    case NANGILA_BF16: fn = reinterpret_cast<const void*>(&absmax_hist_kernel<__nv_bfloat16>); break;
    case NANGILA_F16: fn = reinterpret_cast<const void*>(&absmax_hist_kernel<__half>); break;
    default: return int(cudaErrorInvalidValue);
  }
  int64_t blocks = (n + kThreads - 1) / kThreads;
  blocks = blocks > 148 * 2 ? 148 * 2 : blocks;
  dim3 grid{unsigned(blocks)}, block{unsigned(kThreads)};
  void* args[] = {&x, &n, &k, &qmax, &scratch, &out, &hist256};
  return int(cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream));
}
