// Sculptor calibration statistics on the device.
//  * layer_sumsq: sum of squares of every recorded layer in one launch (-> L2 norms for the Welford
//    norm statistics and the kNN pair schedule);
//  * pair_update: for every scheduled pair of equal-size layers, one Welford step of the element-wise
//    means, second moments and co-moment (five FP32 state vectors per pair, resident on the device);
//  * pair_finalize: reduces a pair's state to the scalars the mask builder needs — the element-
//    averaged Pearson correlation and the element-averaged regression (alpha, beta) in both
//    directions — with FP64 accumulation.
// All pairs of a step are processed by ONE launch each (grid.y = pair).
//
// Replaces the host loops of nangila-core/src/sculptor.rs: record (:238-255, sum of squares),
// StreamingCorrelation::update (:108-141), correlation (:144-170) and coupling (:428-474), keeping
// their validity thresholds (1e-10 on sqrt(var_i var_j) and on var_driver).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nangila_kernels.h"
#include "quant.cuh"

namespace nangila {
namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ float ld(const void* p, int64_t i) {
  return dev::Vec16<T>::to_float(static_cast<const T*>(p)[i]);
}
__device__ __forceinline__ float ld_any(const void* p, int dtype, int64_t i) {
  return dtype == NANGILA_F32 ? ld<float>(p, i) : dtype == NANGILA_BF16 ? ld<__nv_bfloat16>(p, i) : ld<__half>(p, i);
}

__device__ __forceinline__ double block_sum(double v, double* sh) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  double r = 0;
  if (threadIdx.x == 0)
    for (int i = 0; i < kThreads / 32; ++i) r += sh[i];
  __syncthreads();
  return r;  // valid in thread 0
}

__global__ void __launch_bounds__(kThreads) layer_sumsq_kernel(const NangilaLayerDesc* __restrict__ layers, double* out) {
  __shared__ double sh[kThreads / 32];
  const NangilaLayerDesc L = layers[blockIdx.y];
  double acc = 0;
  for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < L.numel; i += int64_t(gridDim.x) * kThreads) {
    const double v = ld_any(L.data, L.dtype, i);
    acc += v * v;
  }
  const double s = block_sum(acc, sh);
  if (threadIdx.x == 0 && s != 0.0) atomicAdd(&out[blockIdx.y], s);
}

// state layout per pair: mean_i[n], mean_j[n], m2_i[n], m2_j[n], co[n]
__global__ void __launch_bounds__(kThreads) pair_update_kernel(const NangilaPairDesc* __restrict__ pairs) {
  const NangilaPairDesc P = pairs[blockIdx.y];
  const float inv_n = 1.0f / float(P.count_after);
  float* mean_i = P.state;
  float* mean_j = P.state + P.numel;
  float* m2_i = P.state + 2 * P.numel;
  float* m2_j = P.state + 3 * P.numel;
  float* co = P.state + 4 * P.numel;
  for (int64_t k = int64_t(blockIdx.x) * kThreads + threadIdx.x; k < P.numel; k += int64_t(gridDim.x) * kThreads) {
    const float vi = ld_any(P.data_i, P.dtype, k), vj = ld_any(P.data_j, P.dtype, k);
    const float di = vi - mean_i[k], dj = vj - mean_j[k];
    const float mi = __fmaf_rn(di, inv_n, mean_i[k]), mj = __fmaf_rn(dj, inv_n, mean_j[k]);
    mean_i[k] = mi;
    mean_j[k] = mj;
    m2_i[k] = __fmaf_rn(di, vi - mi, m2_i[k]);
    m2_j[k] = __fmaf_rn(dj, vj - mj, m2_j[k]);
    co[k] = __fmaf_rn(di, vj - mj, co[k]);
  }
}

// out per pair (8 doubles): sum corr, valid corr, sum alpha(i->j), sum beta(i->j), valid(i->j),
//                           sum alpha(j->i), sum beta(j->i), valid(j->i)
__global__ void __launch_bounds__(kThreads) pair_finalize_kernel(const NangilaPairDesc* __restrict__ pairs, double* out) {
  __shared__ double sh[kThreads / 32];
  const NangilaPairDesc P = pairs[blockIdx.y];
  const float* mean_i = P.state;
  const float* mean_j = P.state + P.numel;
  const float* m2_i = P.state + 2 * P.numel;
  const float* m2_j = P.state + 3 * P.numel;
  const float* co = P.state + 4 * P.numel;
  const double denom = double(P.count_after > 1 ? P.count_after - 1 : 1);
  double a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int64_t k = int64_t(blockIdx.x) * kThreads + threadIdx.x; k < P.numel; k += int64_t(gridDim.x) * kThreads) {
    const double vi = m2_i[k] / denom, vj = m2_j[k] / denom, cov = co[k] / denom;
    const double d = sqrt(vi * vj);
    if (d > 1e-10) {
      a[0] += cov / d;
      a[1] += 1.0;
    }
    if (vi > 1e-10) {  // i drives j
      const double al = cov / vi;
      a[2] += al;
      a[3] += double(mean_j[k]) - al * double(mean_i[k]);
      a[4] += 1.0;
    }
    if (vj > 1e-10) {  // j drives i
      const double al = cov / vj;
      a[5] += al;
      a[6] += double(mean_i[k]) - al * double(mean_j[k]);
      a[7] += 1.0;
    }
  }
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const double s = block_sum(a[q], sh);
    if (threadIdx.x == 0 && s != 0.0) atomicAdd(&out[blockIdx.y * 8 + q], s);
  }
}

int grid_x_for(int64_t max_numel) {
  int64_t b = (max_numel + kThreads * 4 - 1) / (kThreads * 4);
  return int(b < 1 ? 1 : (b > 148 * 4 ? 148 * 4 : b));
}

}  // namespace
}  // namespace nangila

// `layers` / `pairs` are DEVICE arrays of descriptors; `out` must be zero-filled by the caller.
extern "C" int nangila_sculptor_layer_sumsq(const NangilaLayerDesc* layers, int32_t nlayers, int64_t max_numel,
                                            double* out, cudaStream_t stream) {
  if (layers == nullptr || out == nullptr || nlayers <= 0 || nlayers > 65535) return int(cudaErrorInvalidValue);
  dim3 grid(unsigned(nangila::grid_x_for(max_numel)), unsigned(nlayers));
  nangila::layer_sumsq_kernel<<<grid, nangila::kThreads, 0, stream>>>(layers, out);
  return int(cudaGetLastError());
}
extern "C" int nangila_sculptor_pair_update(const NangilaPairDesc* pairs, int32_t npairs, int64_t max_numel,
                                            cudaStream_t stream) {
  if (pairs == nullptr || npairs <= 0 || npairs > 65535) return int(cudaErrorInvalidValue);
  dim3 grid(unsigned(nangila::grid_x_for(max_numel)), unsigned(npairs));
  nangila::pair_update_kernel<<<grid, nangila::kThreads, 0, stream>>>(pairs);
  return int(cudaGetLastError());
}
extern "C" int nangila_sculptor_pair_finalize(const NangilaPairDesc* pairs, int32_t npairs, int64_t max_numel,
                                              double* out, cudaStream_t stream) {
  if (pairs == nullptr || out == nullptr || npairs <= 0 || npairs > 65535) return int(cudaErrorInvalidValue);
  dim3 grid(unsigned(nangila::grid_x_for(max_numel)), unsigned(npairs));
  nangila::pair_finalize_kernel<<<grid, nangila::kThreads, 0, stream>>>(pairs, out);
  return int(cudaGetLastError());
}
