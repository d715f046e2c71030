// Single-scale compatibility kernels with the argument lists of the reference's two CUDA entry
// points (nangila-cuda/src/kernels/predict.cu:252-364 launch_predict_subtract_quantize and
// reconstruct.cu:142-243 launch_dequantize_add_reconstruct): FP32 gradient and history in, one scalar
// gamma, two INT4 values per output byte (low nibble = even element).
//
// They exist for users of `nangila.experimental.cuda_predict_and_quantize` /
// `cuda_dequantize_and_reconstruct` and for the experimental FSDP1 hook; the DDP product path uses
// the fused bucket kernel instead. Rounding is unbiased stochastic rounding keyed by
// (step, layer_id, element index), identical on every rank.
#include <cuda_runtime.h>

#include "nangila_kernels.h"
#include "quant.cuh"

namespace nangila {
namespace {

using namespace dev;

// 8 elements per thread: 2 x float4 of each input, one 32-bit store.
__global__ void __launch_bounds__(256)
predict_quantize_gamma_kernel(const float* __restrict__ grad, const float* __restrict__ cur,
                              const float* __restrict__ prv, float mu, float inv_gamma, uint8_t* __restrict__ out,
                              int64_t n, uint32_t key, bool vec_ok) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x * 8;
  for (int64_t base = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8; base < n; base += stride) {
    float g[8], c[8], p[8];
    if (vec_ok && base + 8 <= n) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float4 a = reinterpret_cast<const float4*>(grad + base)[h];
        float4 b = reinterpret_cast<const float4*>(cur + base)[h];
        float4 d = reinterpret_cast<const float4*>(prv + base)[h];
        g[4 * h] = a.x; g[4 * h + 1] = a.y; g[4 * h + 2] = a.z; g[4 * h + 3] = a.w;
        c[4 * h] = b.x; c[4 * h + 1] = b.y; c[4 * h + 2] = b.z; c[4 * h + 3] = b.w;
        p[4 * h] = d.x; p[4 * h + 1] = d.y; p[4 * h + 2] = d.z; p[4 * h + 3] = d.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool in = base + i < n;
        g[i] = in ? grad[base + i] : 0.0f;
        c[i] = in ? cur[base + i] : 0.0f;
        p[i] = in ? prv[base + i] : 0.0f;
      }
    }
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const uint32_t h = mix32(key + uint32_t((base + i) >> 1) * 0x9E3779B9u);
      const float u0 = float(h & 0xffffu) * (1.0f / 65536.0f), u1 = float(h >> 16) * (1.0f / 65536.0f);
      const float r0 = sanitize(g[i]) - __fmaf_rn(mu, c[i] - p[i], c[i]);
      const float r1 = sanitize(g[i + 1]) - __fmaf_rn(mu, c[i + 1] - p[i + 1], c[i + 1]);
      const int q0 = int(fminf(fmaxf(floorf(__fmaf_rn(r0, inv_gamma, u0)), -8.0f), 7.0f));
      const int q1 = int(fminf(fmaxf(floorf(__fmaf_rn(r1, inv_gamma, u1)), -8.0f), 7.0f));
      w |= (uint32_t(q0) & 0xfu) << (4 * i) | (uint32_t(q1) & 0xfu) << (4 * (i + 1));
    }
    const int64_t byte0 = base >> 1;
    const int64_t nbytes = (n + 1) >> 1;
    if (vec_ok && base + 8 <= n) {
      *reinterpret_cast<uint32_t*>(out + byte0) = w;
    } else {
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (byte0 + b < nbytes) out[byte0 + b] = uint8_t(w >> (8 * b));
    }
  }
}

__global__ void __launch_bounds__(256)
dequant_reconstruct_gamma_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ cur,
                                 const float* __restrict__ prv, float mu, float gamma, float* __restrict__ out,
                                 int64_t n, bool vec_ok) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x * 8;
  for (int64_t base = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8; base < n; base += stride) {
    const int64_t byte0 = base >> 1;
    const int64_t nbytes = (n + 1) >> 1;
    uint32_t w = 0;
    const bool full = vec_ok && base + 8 <= n;
    if (full) {
      w = *reinterpret_cast<const uint32_t*>(packed + byte0);
    } else {
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (byte0 + b < nbytes) w |= uint32_t(packed[byte0 + b]) << (8 * b);
    }
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool in = base + i < n;
      const float c = in ? cur[base + i] : 0.0f, p = in ? prv[base + i] : 0.0f;
      const int q = int(w << (28 - 4 * i)) >> 28;
      o[i] = __fmaf_rn(float(q), gamma, __fmaf_rn(mu, c - p, c));
    }
    if (full) {
      reinterpret_cast<float4*>(out + base)[0] = make_float4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<float4*>(out + base)[1] = make_float4(o[4], o[5], o[6], o[7]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (base + i < n) out[base + i] = o[i];
    }
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int grid_for(int64_t n) {
  int64_t blocks = (n + 2047) / 2048;
  return int(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}
bool bad_common(const void* a, const void* b, const void* c, const void* d, int64_t n, float mu, float gamma) {
  return !a || !b || !c || !d || n <= 0 || n > 1000000000ll || !(mu >= 0.0f && mu <= 1.0f) ||
         !(gamma >= 1e-8f && gamma <= 1e6f);
}

}  // namespace
}  // namespace nangila

extern "C" int nangila_predict_quantize_gamma(const float* grad, const float* g_curr, const float* g_prev, float mu,
                                              float gamma, uint8_t* out, int64_t n, uint32_t step, uint32_t layer_id,
                                              cudaStream_t stream) {
  using namespace nangila;
  if (bad_common(grad, g_curr, g_prev, out, n, mu, gamma)) return int(cudaErrorInvalidValue);
  const bool vec = aligned16(grad) && aligned16(g_curr) && aligned16(g_prev) && (reinterpret_cast<uintptr_t>(out) & 3u) == 0;
  const uint32_t key = dev::make_key(42u, step, layer_id, 0u, 0u);
  predict_quantize_gamma_kernel<<<grid_for(n), 256, 0, stream>>>(grad, g_curr, g_prev, mu, 1.0f / gamma, out, n, key, vec);
  return int(cudaGetLastError());
}

extern "C" int nangila_dequant_reconstruct_gamma(const uint8_t* packed, const float* g_curr, const float* g_prev,
                                                 float mu, float gamma, float* out, int64_t n, cudaStream_t stream) {
  using namespace nangila;
  if (bad_common(packed, g_curr, g_prev, out, n, mu, gamma)) return int(cudaErrorInvalidValue);
  const bool vec = aligned16(out) && (reinterpret_cast<uintptr_t>(packed) & 3u) == 0;
  dequant_reconstruct_gamma_kernel<<<grid_for(n), 256, 0, stream>>>(packed, g_curr, g_prev, mu, gamma, out, n, vec);
  return int(cudaGetLastError());
}
