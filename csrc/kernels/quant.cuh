// Device helpers shared by the fused kernels: 16-element vector loads/stores for fp32 / bf16 / fp16
// tensors, the counter-based random generator, and the block-scaled INT4 quantizer (64 elements per
// scale, scale stored as bf16 rounded up so that |x / scale| <= 7 always holds).
//
// The rounding replaces the reference's host quantizer (nangila-core/src/quantizer.rs:106-214, one
// scale per tensor, biased rounding of negative values) and its device twin
// (nangila-cuda/src/kernels/predict.cu:30-112): here q = floor(x / scale + u) with u uniform in
// [0, 1), which is unbiased for either sign, and u = 0.5 gives round-to-nearest for tests.
// Nibble order is the reference's: byte k holds element 2k in its low and 2k+1 in its high nibble,
// two's complement.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace nangila {
namespace dev {

constexpr int kQuantBlock = 64;      // elements per scale

__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
// One key per (seed, step, bucket, rank, phase); elements are then addressed by their pair index.
__host__ __device__ __forceinline__ uint32_t make_key(uint32_t seed, uint32_t step, uint32_t bucket, uint32_t rank,
                                             uint32_t phase) {
  uint32_t k = mix32(seed ^ 0x9E3779B9u);
  k = mix32(k + step * 0x85ebca6bu);
  k = mix32(k + bucket * 0xc2b2ae35u);
  k = mix32(k + rank * 0x27d4eb2fu + phase * 0x165667b1u);
  return k;
}

// ---- 16-element loads / stores --------------------------------------------------------------------
template <typename T>
struct Vec16;

template <>
struct Vec16<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[16]) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 a = q[i];
      v[4 * i] = a.x; v[4 * i + 1] = a.y; v[4 * i + 2] = a.z; v[4 * i + 3] = a.w;
    }
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[16]) {
    float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  }
  static __device__ __forceinline__ float to_float(float x) { return x; }
  static __device__ __forceinline__ float from_float(float x) { return x; }
};

template <>
struct Vec16<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 a = q[i];
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
        v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[16]) {
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      q[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

template <>
struct Vec16<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 a = q[i];
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        v[8 * i + 2 * j] = f.x;
        v[8 * i + 2 * j + 1] = f.y;
      }
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[16]) {
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2 h = __floats2half2_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      q[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
};

// Load 16 elements starting at element `base` of a tensor of `n` elements; elements at or beyond n
// read as 0. `p` must be 16-byte aligned and `base` a multiple of 16.
__device__ __forceinline__ float sanitize(float x) { return (fabsf(x) <= 3.0e38f) ? x : 0.0f; }  // NaN/Inf -> 0

// bf16 bit pattern of the smallest bf16 >= s (s >= 0, finite).
__device__ __forceinline__ uint32_t bf16_ceil_bits(float s) {
  uint32_t b = __float_as_uint(s);
  b = (b + 0xffffu) >> 16;
  return b >= 0x7f80u ? 0x7f7fu : b;
}
__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

constexpr int kElems8 = 8;
constexpr int kLanes8 = kQuantBlock / kElems8;  // 8

template <typename T>
struct Vec8;
template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = __uint_as_float(w[j] << 16);
      v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <typename T>
__device__ __forceinline__ void load8_guarded(const T* p, int64_t base, int64_t n, float (&v)[8]) {
  if (base + 8 <= n) {
    Vec8<T>::load(p + base, v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (base + i < n) ? Vec16<T>::to_float(p[base + i]) : 0.0f;
  }
}
template <typename T, bool GUARD>
__device__ __forceinline__ void load8(const T* p, int64_t base, int64_t n, float (&v)[8]) {
  if constexpr (GUARD) load8_guarded<T>(p, base, n, v);
  else Vec8<T>::load(p + base, v);
}
template <typename T>
__device__ __forceinline__ void store8_guarded(T* p, int64_t base, int64_t n, const float (&v)[8]) {
  if (base + 8 <= n) {
    Vec8<T>::store(p + base, v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (base + i < n) p[base + i] = Vec16<T>::from_float(v[i]);
  }
}

// Quantize the 8 values of this lane; the eight lanes (lane & ~7 .. lane | 7) holding one 64-element
// block call it together. On return `e` holds the error e - q * scale. `pair0` = index of e[0] / 2.
//
// Instruction diet (this routine bounds the kernel's issue rate):
//  * uniforms: one hash per FOUR elements; byte k becomes the float 2^23 + byte with one byte-permute,
//    and one FMA maps it to u = (byte + 0.5) / 256 (centred, so E[u] = 0.5 exactly);
//  * q = min(floor(e / s + u), 7): no lower clamp is needed because |e| <= 7 s by construction, and a
//    dead block (s == 0) has inv = 0, hence q = 0 and the error stays e;
//  * packing: q + 8 of four elements is accumulated in ONE float by Horner steps of 16 (exact below
//    2^16), converted once, and the two halves are merged; xor 0x88888888 turns the offset nibbles into
//    two's complement.
__device__ __forceinline__ void quantize8(float (&e)[8], uint32_t key, uint32_t pair0, bool stochastic,
                                          uint32_t& packed, uint32_t& scale_bits) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(e[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  scale_bits = bf16_ceil_bits(__fmul_rn(amax, 0.14285715f));  // amax * fl(1/7), rounded up to bf16
  float s = bf16_bits_to_float(scale_bits);
  const bool live = s > 1e-30f;
  const float inv = live ? __frcp_rn(s) : 0.0f;
  if (!live) {
    scale_bits = 0;
    s = 0.0f;
  }
  float half[2];
#pragma unroll
  for (int hlf = 0; hlf < 2; ++hlf) {
    float u[4] = {0.5f, 0.5f, 0.5f, 0.5f};
    if (stochastic) {
      const uint32_t h = mix32(key + (pair0 + uint32_t(hlf)) * 0x9E3779B9u);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // bytes {h.byte[k], 0x00, 0x00, 0x4B}: the float 2^23 + byte
        const float m = __uint_as_float(__byte_perm(h, 0x4B000000u, 0x7540u + uint32_t(k)));
        u[k] = __fmaf_rn(m, 0.00390625f, -32767.998046875f);  // (byte + 0.5) / 256
      }
    }
    float q[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = 4 * hlf + k;
      q[k] = fminf(floorf(__fmaf_rn(e[i], inv, u[k])), 7.0f);
      e[i] = __fmaf_rn(-q[k], s, e[i]);
    }
    half[hlf] = __fmaf_rn(__fmaf_rn(__fmaf_rn(q[3], 16.0f, q[2]), 16.0f, q[1]), 16.0f, q[0]) + 34952.0f;  // + 0x8888
  }
  packed = (__float2uint_rn(half[0]) | (__float2uint_rn(half[1]) << 16)) ^ 0x88888888u;
}
__device__ __forceinline__ void dequant8_add(uint32_t packed, float scale, float (&acc)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int q = int(packed << (28 - 4 * i)) >> 28;
    acc[i] = __fmaf_rn(float(q), scale, acc[i]);
  }
}

template <typename T, bool GUARD>
__device__ __forceinline__ void store8(T* p, int64_t base, int64_t n, const float (&v)[8]) {
  if constexpr (GUARD) store8_guarded<T>(p, base, n, v);
  else Vec8<T>::store(p + base, v);
}

}  // namespace dev
}  // namespace nangila
