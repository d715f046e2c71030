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


// ---- packed bf16x2 variants (gradient and state both bf16) ----------------------------------------------------
// The quantizer bounds the exchange kernels' instruction issue rate, and FP32 arithmetic on values that
// arrive as bf16 and leave as 4-bit codes or bf16 spends most of it on conversions. These variants stay
// in packed bf16: one instruction handles two elements. What that costs in accuracy: g + ef and the
// error e - q s are rounded to 8 significant bits (they are stored as bf16 anyway), which is ~1.4 % of a
// quantization step at the block's largest element; a code may land on the other side of a tie. Every
// rank executes the same instructions on the same bytes, so replicas stay bit-identical.
//
// Tricks: (1) rounding to the nearest integer is one fused multiply-add, t = x * (1/s) + 192: in
// [128, 256) a bf16 has unit spacing, so t is the integer 192 + q (round-to-nearest-even); 1/s is
// truncated to bf16 so that |x / s| cannot exceed 7.03; (2) the two's complement nibble of q is the
// low nibble of t's bit pattern (0x4300 | (64 + q)); (3) the reverse: the bit pattern 0x4300 | n is the
// bf16 number 128 + n.
using bf162 = __nv_bfloat162;
__device__ __forceinline__ bf162 as_bf162(uint32_t w) { return *reinterpret_cast<bf162*>(&w); }
__device__ __forceinline__ uint32_t as_u32(bf162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// True if any of the eight bf16 values in w[0..3] may be Inf or NaN (exponent all ones). May also fire when
// values of magnitude >= 2 with different exponents share the words; the caller then takes the FP32 path.
__device__ __forceinline__ bool maybe_nonfinite8(const uint32_t (&w)[4]) {
  const uint32_t t = (w[0] | w[1] | w[2] | w[3]) & 0x7F807F80u;
  return ((t + 0x00800080u) & 0x80008000u) != 0u;
}

// x[0..3]: eight values as bf16x2 words (element 2j in the low half of word j). On return x holds the error
// x - q * scale, `qs` the dequantized values q * scale, `packed` the eight codes, `scale_bits` the block's
// bf16 scale. The eight lanes holding one 64-element block call it together; all values must be finite.
__device__ __forceinline__ void quantize8_bf16(uint32_t (&x)[4], uint32_t& packed, uint32_t& scale_bits, uint32_t (&qs)[4]) {
  const uint32_t m01 = as_u32(__hmax2(__habs2(as_bf162(x[0])), __habs2(as_bf162(x[1]))));
  const uint32_t m23 = as_u32(__hmax2(__habs2(as_bf162(x[2])), __habs2(as_bf162(x[3]))));
  const uint32_t m = as_u32(__hmax2(as_bf162(m01), as_bf162(m23)));
  float amax = fmaxf(__uint_as_float(m << 16), __uint_as_float(m & 0xffff0000u));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  scale_bits = bf16_ceil_bits(__fmul_rn(amax, 0.14285715f));
  const float s = bf16_bits_to_float(scale_bits);
  const bool live = s > 1e-30f;
  if (!live) scale_bits = 0u;
  const uint32_t inv_bits = live ? (__float_as_uint(__frcp_rn(s)) >> 16) : 0u;  // truncated: never above 1 / s
  const bf162 inv2 = as_bf162(inv_bits | (inv_bits << 16));
  const uint32_t s2_bits = scale_bits | (scale_bits << 16);
  const bf162 s2 = as_bf162(s2_bits), neg_s2 = as_bf162(s2_bits ^ 0x80008000u);
  const bf162 magic = as_bf162(0x43404340u);   // 192, 192
  uint32_t t[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const bf162 xj = as_bf162(x[j]);
    const bf162 tj = __hfma2(xj, inv2, magic);             // 192 + q
    const bf162 qj = __hsub2(tj, magic);                   // q, exact
    t[j] = as_u32(tj);
    qs[j] = as_u32(__hmul2(qj, s2));                       // q * s
    x[j] = as_u32(__hfma2(qj, neg_s2, xj));                // x - q * s
  }
  // nibbles: byte 0 of each half of t holds the code in its low four bits
  const uint32_t a = __byte_perm(t[0], t[1], 0x6420) & 0x0F0F0F0Fu;   // codes of elements 0, 1, 2, 3 (one per byte)
  const uint32_t b = __byte_perm(t[2], t[3], 0x6420) & 0x0F0F0F0Fu;   // elements 4, 5, 6, 7
  const uint32_t a2 = (a | (a >> 4)) & 0x00FF00FFu;                   // bytes 0 and 2: two codes each
  const uint32_t b2 = (b | (b >> 4)) & 0x00FF00FFu;
  packed = __byte_perm(a2, b2, 0x6420);
}

// Unpack eight bf16 values held in four words into floats (element 2j in the low half of word j).
__device__ __forceinline__ void words_to_float8(const uint32_t (&w)[4], float (&v)[8]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}
// bf16 bit pattern (round to nearest even) of a finite float.
__device__ __forceinline__ uint32_t bf16_rn_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}

// acc[j] += q * scale for the eight codes in `packed` (two's complement nibbles), as bf16x2 words.
__device__ __forceinline__ void dequant8_bf16_fma(uint32_t packed, uint32_t scale_bits, uint32_t (&acc)[4]) {
  const uint32_t w = packed ^ 0x88888888u;                 // offset codes n = q + 8 in [0, 15]
  const uint32_t lo = w & 0x0F0F0F0Fu;                     // elements 0, 2, 4, 6
  const uint32_t hi = (w >> 4) & 0x0F0F0F0Fu;              // elements 1, 3, 5, 7
  const bf162 s2 = as_bf162(scale_bits | (scale_bits << 16));
  const bf162 off = as_bf162(0x43084308u);                 // 136 = 128 + 8
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // bytes {lo.byte j, 0, hi.byte j, 0} (selector nibbles 8..15 replicate the byte's sign bit, which is 0 here)
    const uint32_t sel = uint32_t(j) | (uint32_t(8 + j) << 4) | (uint32_t(4 + j) << 8) | (uint32_t(12 + j) << 12);
    uint32_t v;  // prmt in PTX: the CUDA intrinsic ignores bit 3 of a selector nibble (the sign-replicate flag)
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(lo), "r"(hi), "r"(sel));
    v |= 0x43004300u;                                       // 128 + n in both halves
    const bf162 q = __hsub2(as_bf162(v), off);              // exact
    acc[j] = as_u32(__hfma2(q, s2, as_bf162(acc[j])));
  }
}

template <typename T, bool GUARD>
__device__ __forceinline__ void store8(T* p, int64_t base, int64_t n, const float (&v)[8]) {
  if constexpr (GUARD) store8_guarded<T>(p, base, n, v);
  else Vec8<T>::store(p + base, v);
}

}  // namespace dev
}  // namespace nangila
