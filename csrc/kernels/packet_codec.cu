// Device-side packet codec: the prediction-residual compressor of the host core
// (csrc/core/compressor.hpp, PredictionResidualCompressor) for a tensor that lives on the GPU, writing
// and reading the host's own wire format, so a packet made on the device decodes on the host and the
// other way round:
//
//   payload = f32 -64 (block size, negated) | u32 numel | u32 ndim = 1 | u32 numel | f32 kappa |
//             f32 scale[ceil(numel / 64)] | u8 packed[ceil(numel / 2)]   (low nibble = even element)
//
// Three kernels: the two inner products that give the least-squares prediction gain
// kappa = clip(<g + ef, g_hat> / <g_hat, g_hat>, 0, 1); the encoder (x = g + ef - kappa g_hat, one FP32
// scale per 64 elements = amax / 7, round to nearest, error memory, nibble packing); the decoder
// (out = q * scale + kappa g_hat). kappa stays on the device between the first two, so nothing
// synchronises. This is what NangilaHook.compress_gpu / decompress_gpu and the C entry points
// nangila_compress_gpu / nangila_decompress_gpu run (reference: nangila-hook/src/python.rs:315-460 and
// ffi.rs:526-840, whose versions launched predict.cu / reconstruct.cu with one scale per tensor).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nangila_kernels.h"
#include "quant.cuh"

namespace nangila {
namespace {

using namespace dev;

constexpr int kThreads = 256;
constexpr int kMaxBlocks = 1184;  // grid-stride loops: enough blocks to fill any current device
constexpr int kPer = 8;  // elements per thread and iteration: one packed word, one eighth of a scale block

template <typename T>
__device__ __forceinline__ void load8_any(const T* p, int64_t base, int64_t n, float (&v)[8]) {
  // the tensor may start at any element-aligned address: vector loads only when 16-byte aligned
  if (base + 8 <= n && ((reinterpret_cast<uintptr_t>(p + base) & 15u) == 0)) {
    Vec8<T>::load(p + base, v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (base + i < n) ? Vec16<T>::to_float(p[base + i]) : 0.0f;
  }
}
__device__ __forceinline__ void load8_f32(const float* p, int64_t base, int64_t n, float (&v)[8]) {
  if (p == nullptr) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    return;
  }
  load8_any<float>(p, base, n, v);
}

// sums[0] += <g + ef, g_hat>, sums[1] += <g_hat, g_hat>
template <typename T>
__global__ void __launch_bounds__(kThreads) packet_gain_kernel(const T* __restrict__ grad, const float* __restrict__ curr,
                                                               const float* __restrict__ prev, const float* __restrict__ ef,
                                                               float mu, int64_t n, float* __restrict__ sums) {
  float xp = 0.0f, pp = 0.0f;
  const int64_t stride = int64_t(gridDim.x) * kThreads * kPer;
  for (int64_t base = (int64_t(blockIdx.x) * kThreads + threadIdx.x) * kPer; base < n; base += stride) {
    float g[8], c[8], p[8], e[8];
    load8_any<T>(grad, base, n, g);
    load8_f32(curr, base, n, c);
    load8_f32(prev, base, n, p);
    load8_f32(ef, base, n, e);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float pred = __fmaf_rn(mu, c[i] - p[i], c[i]);
      xp = __fmaf_rn(sanitize(g[i]) + e[i], pred, xp);
      pp = __fmaf_rn(pred, pred, pp);
    }
  }
  __shared__ float red[2][kThreads / 32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    xp += __shfl_xor_sync(0xffffffffu, xp, off);
    pp += __shfl_xor_sync(0xffffffffu, pp, off);
  }
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = xp;
    red[1][threadIdx.x >> 5] = pp;
  }
  __syncthreads();
  if (threadIdx.x < 2) {
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) a += red[threadIdx.x][i];
    atomicAdd(&sums[threadIdx.x], a);
  }
}

// kappa: fixed (>= 0) or taken from the inner products in `sums` (fixed < 0). Thread 0 of block 0 writes the value
// it used into the payload's gain field.
__device__ __forceinline__ float resolve_gain(float fixed, const float* sums) {
  if (fixed >= 0.0f) return fixed;
  const float xp = sums[0], pp = sums[1];
  return pp > 0.0f ? fminf(fmaxf(xp / pp, 0.0f), 1.0f) : 0.0f;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) packet_encode_kernel(const T* __restrict__ grad, const float* __restrict__ curr,
                                                                 const float* __restrict__ prev, float* __restrict__ ef,
                                                                 float mu, float fixed_gain, const float* __restrict__ sums,
                                                                 int64_t n, float* __restrict__ gain_out,
                                                                 float* __restrict__ scales, uint8_t* __restrict__ packed) {
  const float kappa = resolve_gain(fixed_gain, sums);
  if (blockIdx.x == 0 && threadIdx.x == 0) *gain_out = kappa;
  const int64_t padded = (n + 255) / 256 * 256;  // whole warps: every lane of a warp runs the same number of iterations (shuffles below)
  const int64_t stride = int64_t(gridDim.x) * kThreads * kPer;
  for (int64_t base = (int64_t(blockIdx.x) * kThreads + threadIdx.x) * kPer; base < padded; base += stride) {
    float g[8], c[8], p[8], e[8];
    load8_any<T>(grad, base, n, g);
    load8_f32(curr, base, n, c);
    load8_f32(prev, base, n, p);
    load8_f32(ef, base, n, e);
    float x[8], amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float pred = __fmaf_rn(mu, c[i] - p[i], c[i]);
      x[i] = sanitize(g[i]) + e[i] - kappa * pred;
      amax = fmaxf(amax, fabsf(x[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float s = __fdiv_rn(amax, 7.0f);  // the host quantizer's scale, bit for bit
    uint32_t word = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float q = 0.0f;
      if (s > 0.0f) {
        const float scaled = __fdiv_rn(x[i], s);
        const float fl = floorf(scaled);
        q = (scaled - fl >= 0.5f) ? fl + 1.0f : fl;
        q = fminf(fmaxf(q, -8.0f), 7.0f);
      }
      x[i] -= q * s;  // what was not sent
      word |= (uint32_t(int(q)) & 0xFu) << (4 * i);
    }
    if (base < n) {
      if ((threadIdx.x & 7) == 0) scales[base / 64] = s;
      const int64_t byte0 = base / 2;
      const int64_t nbytes = (n + 1) / 2;
      if (byte0 + 4 <= nbytes && ((reinterpret_cast<uintptr_t>(packed + byte0) & 3u) == 0)) {
        *reinterpret_cast<uint32_t*>(packed + byte0) = word;
      } else {
        for (int k = 0; k < 4 && byte0 + k < nbytes; ++k) packed[byte0 + k] = uint8_t(word >> (8 * k));
      }
      if (ef != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (base + i < n) ef[base + i] = x[i];
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads) packet_decode_kernel(const float* __restrict__ scales, const uint8_t* __restrict__ packed,
                                                                 const float* __restrict__ curr, const float* __restrict__ prev,
                                                                 float mu, float fixed_gain, const float* __restrict__ gain_in,
                                                                 int64_t n, float* __restrict__ out) {
  const float kappa = fixed_gain >= 0.0f ? fixed_gain : *gain_in;
  const int64_t nbytes = (n + 1) / 2;
  const int64_t stride = int64_t(gridDim.x) * kThreads * kPer;
  for (int64_t base = (int64_t(blockIdx.x) * kThreads + threadIdx.x) * kPer; base < n; base += stride) {
    const int64_t byte0 = base / 2;
    uint32_t word = 0u;
    if (byte0 + 4 <= nbytes && ((reinterpret_cast<uintptr_t>(packed + byte0) & 3u) == 0)) {
      word = *reinterpret_cast<const uint32_t*>(packed + byte0);
    } else {
      for (int k = 0; k < 4 && byte0 + k < nbytes; ++k) word |= uint32_t(packed[byte0 + k]) << (8 * k);
    }
    const float s = scales[base / 64];
    float c[8], p[8];
    load8_f32(kappa != 0.0f ? curr : nullptr, base, n, c);
    load8_f32(kappa != 0.0f ? prev : nullptr, base, n, p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (base + i < n) {
        const int q = int(word << (28 - 4 * i)) >> 28;
        out[base + i] = __fmaf_rn(kappa, __fmaf_rn(mu, c[i] - p[i], c[i]), float(q) * s);
      }
    }
  }
}

int grid_for(int64_t n) {
  const int64_t blocks = (n + int64_t(kThreads) * kPer - 1) / (int64_t(kThreads) * kPer);
  return int(blocks < 1 ? 1 : blocks > kMaxBlocks ? kMaxBlocks : blocks);
}

}  // namespace
}  // namespace nangila

extern "C" int64_t nangila_packet_payload_bytes(int64_t n) { return 20 + 4 * ((n + 63) / 64) + (n + 1) / 2; }

extern "C" int nangila_packet_encode(const void* grad, int32_t dtype, const float* curr, const float* prev, float* ef, float mu,
                                     float gain, int64_t n, uint8_t* payload, cudaStream_t stream) {
  using namespace nangila;
  if (grad == nullptr || payload == nullptr || n <= 0 || n > 0x7fffffffll || (reinterpret_cast<uintptr_t>(payload) & 3u) != 0 ||
      (curr == nullptr) != (prev == nullptr) || !(mu >= 0.0f && mu <= 1.0f))
    return int(cudaErrorInvalidValue);
  float* gain_out = reinterpret_cast<float*>(payload + 16);
  float* scales = reinterpret_cast<float*>(payload + 20);
  uint8_t* packed = payload + 20 + 4 * ((n + 63) / 64);
  // The two inner products live in the first 8 bytes of the payload until the encoder has read them; the
  // fixed words that belong there are copied in afterwards (the encoder never writes the first 16 bytes).
  float* sums = reinterpret_cast<float*>(payload);
  const int grid = grid_for(n);
  if (curr == nullptr) gain = 0.0f;
  cudaError_t e;
  if (gain < 0.0f) {
    e = cudaMemsetAsync(sums, 0, 2 * sizeof(float), stream);
    if (e != cudaSuccess) return int(e);
  }
#define NANGILA_PACKET_LAUNCH(TYPE)                                                                                  \
  do {                                                                                                               \
    if (gain < 0.0f)                                                                                                 \
      packet_gain_kernel<TYPE><<<grid, kThreads, 0, stream>>>(static_cast<const TYPE*>(grad), curr, prev, ef, mu, n, sums); \
    packet_encode_kernel<TYPE><<<grid, kThreads, 0, stream>>>(static_cast<const TYPE*>(grad), curr, prev, ef, mu, gain, \
                                                              sums, n, gain_out, scales, packed);                    \
  } while (0)
  switch (dtype) {
    case NANGILA_F32: NANGILA_PACKET_LAUNCH(float); break;
    case NANGILA_BF16: NANGILA_PACKET_LAUNCH(__nv_bfloat16); break;
    case NANGILA_F16: NANGILA_PACKET_LAUNCH(__half); break;
    default: return int(cudaErrorInvalidValue);
  }
#undef NANGILA_PACKET_LAUNCH
  e = cudaGetLastError();
  if (e != cudaSuccess) return int(e);
  // fixed words of the payload: block size (negated), numel, ndim, dim
  const float neg_block = -64.0f;
  uint32_t head[4];
  memcpy(&head[0], &neg_block, 4);
  head[1] = head[3] = uint32_t(n);
  head[2] = 1u;
  // pageable source: the runtime stages it before the call returns, so the stack buffer may go away
  return int(cudaMemcpyAsync(payload, head, 16, cudaMemcpyHostToDevice, stream));
}

extern "C" int nangila_packet_decode(const uint8_t* payload, int64_t payload_bytes, int32_t ndim, const float* curr,
                                     const float* prev, float mu, float gain, int64_t n, float* out, cudaStream_t stream) {
  using namespace nangila;
  if (payload == nullptr || out == nullptr || n <= 0 || ndim < 0 || ndim > 8 || (reinterpret_cast<uintptr_t>(payload) & 3u) != 0 ||
      (curr == nullptr) != (prev == nullptr))
    return int(cudaErrorInvalidValue);
  const int64_t off_gain = 12 + 4 * int64_t(ndim);
  const int64_t need = off_gain + 4 + 4 * ((n + 63) / 64) + (n + 1) / 2;
  if (payload_bytes < need) return int(cudaErrorInvalidValue);
  const float* gain_in = reinterpret_cast<const float*>(payload + off_gain);
  const float* scales = gain_in + 1;
  const uint8_t* packed = reinterpret_cast<const uint8_t*>(scales + (n + 63) / 64);
  if (curr == nullptr) gain = 0.0f;
  packet_decode_kernel<<<grid_for(n), kThreads, 0, stream>>>(scales, packed, curr, prev, mu, gain, gain_in, n, out);
  return int(cudaGetLastError());
}

// Small runtime helpers for callers that bind this library without linking the CUDA runtime themselves
// (the host core's C entry points).
extern "C" int nangila_copy_to_host(void* dst, const void* src, int64_t nbytes, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyAsync(dst, src, size_t(nbytes), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return int(e);
  return int(cudaStreamSynchronize(stream));
}
extern "C" int nangila_copy_to_device(void* dst, const void* src, int64_t nbytes, cudaStream_t stream) {
  return int(cudaMemcpyAsync(dst, src, size_t(nbytes), cudaMemcpyHostToDevice, stream));
}
extern "C" int nangila_stream_sync(cudaStream_t stream) { return int(cudaStreamSynchronize(stream)); }
