// Host-side INT4 (or narrower/wider, up to 8 bit) stochastic quantizer. This is the quantizer of
// the CPU/gloo transport and the oracle for the device kernels.
//
// Two behaviours:
//  * default: one scale per block of 64 elements (scale = absmax / qmax, nothing is clipped), like
//    the fused device kernels; unbiased stochastic rounding q = floor(x/scale + u), u in [0,1) from
//    a counter-based generator keyed by (seed, layer, step, global element index). With
//    block_size = 0 it falls back to one scale per tensor, gamma = p99(|x|) / qmax (no lag);
//  * reference_exact: reproduces nangila-core/src/quantizer.rs as written — gamma is an EMA
//    (0.99) shared by all layers starting at 1.0 (:64-73, :123-131), and negative values are
//    rounded away from zero with probability frac (:178-190).
// Parity: quantizer.rs:10-33 (CompressedTensor), :81-96 (gamma), :106-214 (quantize),
// :217-232 (dequantize), :235-272 (nibble packing, low nibble = even index, two's complement),
// :275-330 (dequantize_partial).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

#include "types.hpp"

namespace nangila {

struct CompressedTensor {
  std::vector<uint8_t> data;
  float gamma = 0.0f;          // per-tensor scale; with block scales: their mean (informational)
  std::vector<size_t> shape;
  size_t numel = 0;
  size_t block = 0;            // 0 = one scale (gamma); else elements per entry of `scales`
  std::vector<float> scales;
  float pred_gain = 1.0f;      // kappa the sender applied to its prediction (block format only)

  float scale_at(size_t i) const { return block ? scales[i / block] : gamma; }
  size_t size_bytes() const { return data.size() + scales.size() * 4 + 4 + shape.size() * 8 + 8; }
  float compression_ratio(size_t original_numel) const {
    size_t b = size_bytes();
    return b == 0 ? 1.0f : float(original_numel * 4) / float(b);
  }
};

inline uint64_t splitmix64_finalize(uint64_t z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  return z;
}

inline std::vector<uint8_t> pack_int4(const std::vector<int8_t>& v) {
  std::vector<uint8_t> out((v.size() + 1) / 2);
  for (size_t i = 0; i < v.size(); i += 2) {
    uint8_t lo = uint8_t(v[i]) & 0x0F;
    uint8_t hi = i + 1 < v.size() ? uint8_t((uint8_t(v[i + 1]) & 0x0F) << 4) : 0;
    out[i / 2] = lo | hi;
  }
  return out;
}
inline int8_t sign_extend4(uint8_t nib) { return int8_t((nib & 0x08) ? (nib | 0xF0) : nib); }
inline std::vector<int8_t> unpack_int4(const std::vector<uint8_t>& p, size_t numel) {
  std::vector<int8_t> out;
  out.reserve(numel);
  for (uint8_t b : p) {
    if (out.size() < numel) out.push_back(sign_extend4(b & 0x0F));
    if (out.size() < numel) out.push_back(sign_extend4((b >> 4) & 0x0F));
  }
  return out;
}

class Quantizer {
 public:
  Quantizer(uint8_t bits = 4, bool dynamic_gamma = true, bool reference_exact = false)
      : bits_(bits), dynamic_gamma_(dynamic_gamma), reference_exact_(reference_exact),
        block_(reference_exact ? 0 : 64) {
    if (bits == 0 || bits > 8) throw NangilaError(ErrorKind::Config, "Maximum 8 bits supported");
  }
  static Quantizer int4() { return Quantizer(4, true); }

  int qmax() const { return (1 << (bits_ - 1)) - 1; }
  int qmin() const { return -(1 << (bits_ - 1)); }

  // p99(|x|) / qmax, floored at 1e-8.
  float compute_gamma(const Tensor& t) const {
    std::vector<float> a(t.data.size());
    for (size_t i = 0; i < a.size(); ++i) {
      float v = std::fabs(t.data[i]);
      a[i] = std::isfinite(v) ? v : 0.0f;
    }
    size_t idx = static_cast<size_t>(static_cast<float>(a.size()) * 0.99f);
    float p99 = 1.0f;
    if (idx < a.size()) {
      std::nth_element(a.begin(), a.begin() + idx, a.end());
      p99 = a[idx];
    }
    return std::max(p99 / float(qmax()), 1e-8f);
  }

  CompressedTensor quantize(const Tensor& t, uint32_t layer_id, uint64_t step) {
    return quantize_with_offset(t, layer_id, step, 0);
  }
  // `global_offset` = index of element 0 inside the full (unsharded) parameter, so that a sharded
  // caller draws the same random number for an element as an unsharded one would.
  CompressedTensor quantize_with_offset(const Tensor& t, uint32_t layer_id, uint64_t step, size_t global_offset) {
    CompressedTensor out;
    if (t.numel() == 0) return out;
    const bool blocked = block_ > 0 && dynamic_gamma_;
    if (blocked) {
      const size_t nb = (t.numel() + block_ - 1) / block_;
      out.block = block_;
      out.scales.resize(nb);
      double mean = 0;
      for (size_t b = 0; b < nb; ++b) {
        float amax = 0.0f;
        for (size_t i = b * block_, e = std::min(t.numel(), (b + 1) * block_); i < e; ++i) {
          float v = std::fabs(t.data[i]);
          if (std::isfinite(v)) amax = std::max(amax, v);
        }
        out.scales[b] = amax / float(qmax());
        mean += out.scales[b];
      }
      gamma_ema_ = float(mean / double(nb));
    }
    float gamma;
    if (blocked) {
      gamma = gamma_ema_;
    } else if (dynamic_gamma_) {
      float g = compute_gamma(t);
      gamma_ema_ = reference_exact_ ? gamma_momentum_ * gamma_ema_ + (1.0f - gamma_momentum_) * g : g;
      gamma = std::max(gamma_ema_, 1e-8f);
    } else {
      gamma = std::max(gamma_ema_, 1e-8f);
    }
    const uint64_t base = uint64_t(layer_id) * 0x9E3779B97F4A7C15ull + step * 0xBF58476D1CE4E5B9ull;
    const uint64_t seeded = seed_ * 0x9E3779B97F4A7C15ull + base;
    const int hi = qmax(), lo = qmin();
    std::vector<int8_t> q(t.numel());
    for (size_t i = 0; i < t.numel(); ++i) {
      float x = t.data[i];
      if (!std::isfinite(x)) x = 0.0f;
      const float sc = blocked ? out.scales[i / block_] : gamma;
      float scaled = sc > 0.0f ? x / sc : 0.0f;
      float fl = std::floor(scaled);
      float frac = scaled - fl;
      float r;
      if (!stochastic_) {
        r = frac >= 0.5f ? fl + 1.0f : fl;
      } else {
        uint64_t h = splitmix64_finalize(seeded + uint64_t(global_offset + i));
        if (reference_exact_) {
          float u = float(h) / float(UINT64_MAX);
          bool up = frac >= u;
          r = scaled >= 0.0f ? (up ? fl + 1.0f : fl) : (up ? fl : fl + 1.0f);
        } else {
          float u = float(h >> 40) * (1.0f / 16777216.0f);  // 24 random bits in [0,1)
          r = std::floor(scaled + u);
        }
      }
      r = std::min(std::max(r, float(lo)), float(hi));
      q[i] = int8_t(r);
    }
    if (bits_ <= 4) {
      out.data = pack_int4(q);
    } else {
      out.data.resize(q.size());
      for (size_t i = 0; i < q.size(); ++i) out.data[i] = uint8_t(q[i]);
    }
    out.gamma = gamma;
    out.shape = t.shape;
    out.numel = t.numel();
    return out;
  }

  std::vector<int8_t> unpack(const CompressedTensor& c) const {
    if (bits_ <= 4) return unpack_int4(c.data, c.numel);
    std::vector<int8_t> q(std::min(c.numel, c.data.size()));
    for (size_t i = 0; i < q.size(); ++i) q[i] = int8_t(c.data[i]);
    return q;
  }
  Tensor dequantize(const CompressedTensor& c) const {
    if (c.numel == 0) return Tensor::zeros(c.shape);
    std::vector<int8_t> q = unpack(c);
    std::vector<float> d(c.numel, 0.0f);
    for (size_t i = 0; i < q.size() && i < d.size(); ++i) d[i] = float(q[i]) * c.scale_at(i);
    return Tensor(std::move(d), c.shape.empty() ? std::vector<size_t>{c.numel} : c.shape);
  }
  Tensor dequantize_partial(const CompressedTensor& c, size_t start, size_t end) const {
    start = std::min(start, c.numel);
    end = std::min(end, c.numel);
    if (c.numel == 0 || start >= end) return Tensor::zeros({0});
    std::vector<float> d;
    d.reserve(end - start);
    for (size_t i = start; i < end; ++i) {
      int8_t q;
      if (bits_ <= 4) {
        size_t byte = i / 2;
        if (byte >= c.data.size()) break;
        uint8_t b = c.data[byte];
        q = sign_extend4((i & 1) ? ((b >> 4) & 0x0F) : (b & 0x0F));
      } else {
        if (i >= c.data.size()) break;
        q = int8_t(c.data[i]);
      }
      d.push_back(float(q) * c.scale_at(i));
    }
    size_t n = d.size();
    return Tensor(std::move(d), {n});
  }

  float gamma() const { return gamma_ema_; }
  void set_gamma(float g) { gamma_ema_ = g; }
  void set_dynamic_gamma(bool d) { dynamic_gamma_ = d; }
  void set_stochastic(bool s) { stochastic_ = s; }
  void set_seed(uint64_t s) { seed_ = s; }
  void set_block_size(size_t b) { block_ = b; }
  size_t block_size() const { return block_; }
  uint8_t bits() const { return bits_; }
  bool reference_exact() const { return reference_exact_; }

 private:
  uint8_t bits_;
  bool dynamic_gamma_;
  bool reference_exact_;
  size_t block_;
  bool stochastic_ = true;
  float gamma_ema_ = 1.0f;
  float gamma_momentum_ = 0.99f;
  uint64_t seed_ = 42;
};

}  // namespace nangila
