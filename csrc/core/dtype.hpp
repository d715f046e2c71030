// Conversions between raw little-endian FP16 / BF16 byte strings and FP32 vectors.
//
// Parity: nangila-core/src/dtype.rs:8-42. FP32->half conversions round to nearest even, like the
// `half` crate the reference relies on.
#pragma once
#include <cstdint>
#include <cstring>
#include <vector>

#include "types.hpp"

namespace nangila {

inline float bf16_bits_to_f32(uint16_t b) {
  uint32_t u = uint32_t(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x0040u);  // quiet NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return uint16_t(u >> 16);
}
inline float f16_bits_to_f32(uint16_t h) {
  uint32_t sign = uint32_t(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {  // subnormal: renormalise
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      u = sign | uint32_t(127 - 15 - e) << 23 | (man & 0x3ffu) << 13;
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | man << 13;
  } else {
    u = sign | (exp + 127 - 15) << 23 | man << 13;
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_f16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000u;
  uint32_t absu = u & 0x7fffffffu;
  if (absu > 0x7f800000u) return uint16_t(sign | 0x7e00u);             // NaN
  if (absu >= 0x47800000u) return uint16_t(sign | 0x7c00u);            // overflow -> inf
  if (absu < 0x33000000u) return uint16_t(sign);                       // underflow -> 0
  int32_t exp = int32_t(absu >> 23) - 127 + 15;
  uint32_t man = absu & 0x7fffffu;
  if (exp <= 0) {  // subnormal result
    man |= 0x800000u;
    uint32_t shift = uint32_t(14 - exp);
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1u))) ++half_man;
    return uint16_t(sign | half_man);
  }
  uint32_t half = (uint32_t(exp) << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;  // may carry into exponent: ok
  return uint16_t(sign | half);
}

inline std::vector<float> f16_bytes_to_f32(const uint8_t* bytes, size_t nbytes) {
  std::vector<float> out(nbytes / 2);
  for (size_t i = 0; i < out.size(); ++i)
    out[i] = f16_bits_to_f32(uint16_t(bytes[2 * i] | (bytes[2 * i + 1] << 8)));
  return out;
}
inline std::vector<float> bf16_bytes_to_f32(const uint8_t* bytes, size_t nbytes) {
  std::vector<float> out(nbytes / 2);
  for (size_t i = 0; i < out.size(); ++i)
    out[i] = bf16_bits_to_f32(uint16_t(bytes[2 * i] | (bytes[2 * i + 1] << 8)));
  return out;
}
inline std::vector<uint8_t> f32_to_f16_bytes(const float* p, size_t n) {
  std::vector<uint8_t> out(n * 2);
  for (size_t i = 0; i < n; ++i) {
    uint16_t h = f32_to_f16_bits(p[i]);
    out[2 * i] = uint8_t(h & 0xff);
    out[2 * i + 1] = uint8_t(h >> 8);
  }
  return out;
}
inline std::vector<uint8_t> f32_to_bf16_bytes(const float* p, size_t n) {
  std::vector<uint8_t> out(n * 2);
  for (size_t i = 0; i < n; ++i) {
    uint16_t h = f32_to_bf16_bits(p[i]);
    out[2 * i] = uint8_t(h & 0xff);
    out[2 * i + 1] = uint8_t(h >> 8);
  }
  return out;
}

// Raw bytes of `dtype` -> FP32 tensor (1-D), used by the `_ex` C entry points.
inline Tensor tensor_from_bytes(const uint8_t* bytes, size_t count, DataType dtype) {
  std::vector<float> v;
  if (dtype == DataType::F32) {
    v.resize(count);
    std::memcpy(v.data(), bytes, count * 4);
  } else if (dtype == DataType::F16) {
    v = f16_bytes_to_f32(bytes, count * 2);
  } else {
    v = bf16_bytes_to_f32(bytes, count * 2);
  }
  return Tensor(std::move(v), {count}, dtype);
}
inline void tensor_to_bytes(const Tensor& t, DataType dtype, uint8_t* out) {
  if (dtype == DataType::F32) {
    std::memcpy(out, t.data.data(), t.data.size() * 4);
  } else if (dtype == DataType::F16) {
    auto b = f32_to_f16_bytes(t.data.data(), t.data.size());
    std::memcpy(out, b.data(), b.size());
  } else {
    auto b = f32_to_bf16_bytes(t.data.data(), t.data.size());
    std::memcpy(out, b.data(), b.size());
  }
}

}  // namespace nangila
