// Q8.23 signed fixed point (1 sign, 8 integer, 23 fraction bits in an int32) and a buffer of such
// values. Used for the bit-exact, platform-independent predictor state of the host path and for
// the checkpoint format.
//
// Parity: nangila-core/src/fixed_point.rs:57-84 (from_f32: clamp to [-256, 256), round half away
// from zero, saturating cast), :104-112 (saturating add/sub), :118-123 (mul through int64 and an
// arithmetic shift by 23), :137-141 (fma), :185-320 (buffer operations and hash).
#pragma once
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

#include "siphash.hpp"

namespace nangila {

constexpr float kQ823Scale = 8388608.0f;  // 2^23

// Number of inputs that had to be clamped since process start (diagnostics only).
inline std::atomic<uint64_t>& q823_saturation_counter() {
  static std::atomic<uint64_t> c{0};
  return c;
}

struct Q8_23 {
  int32_t bits = 0;

  static Q8_23 from_bits(int32_t b) { return Q8_23{b}; }

  static Q8_23 from_f32(float f) {
    if (std::isnan(f)) return Q8_23{0};
    // The upper bound 255.99999988 is not representable in FP32 and reads as 256.0f; the
    // saturating cast below then yields INT32_MAX for every input >= 256.
    float clamped = std::min(std::max(f, -256.0f), 256.0f);
    if (clamped != f || f >= 256.0f) q823_saturation_counter().fetch_add(1, std::memory_order_relaxed);
    float scaled = std::round(clamped * kQ823Scale);
    if (scaled >= 2147483648.0f) return Q8_23{std::numeric_limits<int32_t>::max()};
    if (scaled <= -2147483648.0f) return Q8_23{std::numeric_limits<int32_t>::min()};
    return Q8_23{static_cast<int32_t>(scaled)};
  }
  static Q8_23 from_f32_clipped(float f, float clip) {
    return from_f32(std::min(std::max(f, -clip), clip));
  }
  float to_f32() const { return static_cast<float>(bits) / kQ823Scale; }

  static int32_t sat(int64_t v) {
    return static_cast<int32_t>(std::min<int64_t>(std::max<int64_t>(v, INT32_MIN), INT32_MAX));
  }
  Q8_23 operator+(Q8_23 o) const { return Q8_23{sat(int64_t(bits) + int64_t(o.bits))}; }
  Q8_23 operator-(Q8_23 o) const { return Q8_23{sat(int64_t(bits) - int64_t(o.bits))}; }
  Q8_23 operator*(Q8_23 o) const { return Q8_23{sat((int64_t(bits) * int64_t(o.bits)) >> 23)}; }
  Q8_23 mul_scalar(float s) const { return *this * from_f32(s); }
  // this + a * b
  Q8_23 fma(Q8_23 a, Q8_23 b) const {
    return Q8_23{sat(int64_t(bits) + ((int64_t(a.bits) * int64_t(b.bits)) >> 23))};
  }
  Q8_23 abs() const {
    return Q8_23{bits == INT32_MIN ? INT32_MAX : (bits < 0 ? -bits : bits)};
  }
  bool is_negative() const { return bits < 0; }
  bool operator==(Q8_23 o) const { return bits == o.bits; }
};

class FixedPointBuffer {
 public:
  FixedPointBuffer() = default;
  explicit FixedPointBuffer(std::vector<Q8_23> d) : data_(std::move(d)) {}

  static FixedPointBuffer from_f32(const float* p, size_t n) {
    FixedPointBuffer b;
    b.data_.resize(n);
    for (size_t i = 0; i < n; ++i) b.data_[i] = Q8_23::from_f32(p[i]);
    return b;
  }
  static FixedPointBuffer from_f32(const std::vector<float>& v) { return from_f32(v.data(), v.size()); }
  static FixedPointBuffer from_f32_clipped(const std::vector<float>& v, float clip) {
    FixedPointBuffer b;
    b.data_.resize(v.size());
    for (size_t i = 0; i < v.size(); ++i) b.data_[i] = Q8_23::from_f32_clipped(v[i], clip);
    return b;
  }
  // Clip at the 99.9th percentile of |x| (at most 256) before conversion.
  static FixedPointBuffer from_f32_auto_clip(const std::vector<float>& v) {
    std::vector<float> a(v.size());
    for (size_t i = 0; i < v.size(); ++i) a[i] = std::fabs(v[i]);
    std::sort(a.begin(), a.end());
    size_t idx = static_cast<size_t>(static_cast<float>(a.size()) * 0.999f);
    float clip = idx < a.size() ? a[idx] : 256.0f;
    return from_f32_clipped(v, std::min(clip, 256.0f));
  }
  static FixedPointBuffer from_bits(const std::vector<int32_t>& bits) {
    FixedPointBuffer b;
    b.data_.resize(bits.size());
    for (size_t i = 0; i < bits.size(); ++i) b.data_[i] = Q8_23{bits[i]};
    return b;
  }

  std::vector<float> to_f32() const {
    std::vector<float> out(data_.size());
    for (size_t i = 0; i < data_.size(); ++i) out[i] = data_[i].to_f32();
    return out;
  }
  std::vector<int32_t> to_bits() const {
    std::vector<int32_t> out(data_.size());
    for (size_t i = 0; i < data_.size(); ++i) out[i] = data_[i].bits;
    return out;
  }
  size_t size() const { return data_.size(); }
  bool empty() const { return data_.empty(); }
  const Q8_23& operator[](size_t i) const { return data_[i]; }
  const std::vector<Q8_23>& values() const { return data_; }

  FixedPointBuffer add(const FixedPointBuffer& o) const { return zip(o, [](Q8_23 a, Q8_23 b) { return a + b; }); }
  FixedPointBuffer sub(const FixedPointBuffer& o) const { return zip(o, [](Q8_23 a, Q8_23 b) { return a - b; }); }
  FixedPointBuffer scale(float f) const {
    Q8_23 q = Q8_23::from_f32(f);
    FixedPointBuffer r;
    r.data_.resize(data_.size());
    for (size_t i = 0; i < data_.size(); ++i) r.data_[i] = data_[i] * q;
    return r;
  }
  // this + other * scale
  FixedPointBuffer fma(const FixedPointBuffer& o, float s) const {
    Q8_23 q = Q8_23::from_f32(s);
    return zip(o, [q](Q8_23 a, Q8_23 b) { return a.fma(b, q); });
  }
  // SipHash-1-3 (zero key) over the raw int32 values in order.
  uint64_t hash() const {
    SipHasher13 h;
    for (const Q8_23& q : data_) h.write_i32(q.bits);
    return h.finish();
  }

 private:
  template <class F>
  FixedPointBuffer zip(const FixedPointBuffer& o, F f) const {
    if (o.data_.size() != data_.size())
      throw std::invalid_argument("FixedPointBuffer length mismatch");
    FixedPointBuffer r;
    r.data_.resize(data_.size());
    for (size_t i = 0; i < data_.size(); ++i) r.data_[i] = f(data_[i], o.data_[i]);
    return r;
  }
  std::vector<Q8_23> data_;
};

}  // namespace nangila
