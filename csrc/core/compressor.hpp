// Compressor interface and the three host-side compressors (prediction-residual INT4, DGC top-k,
// PowerSGD low rank). These run the CPU/gloo transport and are the oracles the device kernels are
// tested against.
//
// Parity: nangila-core/src/compressor.rs:12-52 (trait), :91-131 (prediction-residual compress /
// decompress), :158-211 (single-stage pipeline wrapper); dgc.rs:64-186; power_sgd.rs:46-193;
// reconstructor.rs:40-60 (driver = prediction + dequantized residual).
// Deliberate differences from the reference, all opt-out:
//  * the prediction-residual path keeps an error-feedback memory (the reference drops the
//    quantization error); with no history yet the prediction is zero instead of an error;
//  * DGC optionally applies momentum correction and momentum-factor masking;
//  * payloads are plain little-endian structs (documented per compressor), not bincode.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <numeric>

#include "config.hpp"
#include "packet.hpp"
#include "predictor.hpp"
#include "quantizer.hpp"
#include "types.hpp"

namespace nangila {

namespace wire {
inline void put_u32(std::vector<uint8_t>& o, uint32_t v) {
  uint8_t b[4];
  detail::put_le<uint32_t>(b, v);
  o.insert(o.end(), b, b + 4);
}
inline void put_f32(std::vector<uint8_t>& o, float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  put_u32(o, u);
}
struct Reader {
  const uint8_t* p;
  size_t len;
  size_t off = 0;
  bool ok = true;
  uint32_t u32() {
    if (off + 4 > len) { ok = false; return 0; }
    uint32_t v = detail::get_le<uint32_t>(p + off);
    off += 4;
    return v;
  }
  float f32() {
    uint32_t u = u32();
    float f;
    std::memcpy(&f, &u, 4);
    return f;
  }
};

// Driver payload: f32 gamma, u32 numel, u32 ndim, u32 dims[ndim], u8 packed[...]
// (nangila-hook/src/hook.rs:697-742). Block-scaled extension: the gamma field holds -block_size
// (a negative number no real scale can be) and, after the dims, f32 prediction_gain and
// f32 scales[ceil(numel / block_size)] precede the packed bytes.
inline std::vector<uint8_t> serialize_compressed(const CompressedTensor& c) {
  std::vector<uint8_t> o;
  o.reserve(12 + 4 * c.shape.size() + 4 * c.scales.size() + c.data.size());
  put_f32(o, c.block ? -float(c.block) : c.gamma);
  put_u32(o, uint32_t(c.numel));
  put_u32(o, uint32_t(c.shape.size()));
  for (size_t d : c.shape) put_u32(o, uint32_t(d));
  if (c.block) put_f32(o, c.pred_gain);
  for (float sc : c.scales) put_f32(o, sc);
  o.insert(o.end(), c.data.begin(), c.data.end());
  return o;
}
inline CompressedTensor deserialize_compressed(const uint8_t* p, size_t len) {
  CompressedTensor c;
  if (len < 12) return c;
  Reader r{p, len};
  c.gamma = r.f32();
  c.numel = r.u32();
  uint32_t nd = r.u32();
  for (uint32_t i = 0; i < nd && r.off + 4 <= len; ++i) c.shape.push_back(r.u32());
  if (c.gamma < 0.0f) {
    c.block = size_t(-c.gamma);
    size_t nb = c.block ? (c.numel + c.block - 1) / c.block : 0;
    if (c.block == 0 || r.off + 4 + nb * 4 > len) return CompressedTensor{};
    c.pred_gain = r.f32();
    c.scales.resize(nb);
    double mean = 0;
    for (size_t b = 0; b < nb; ++b) mean += (c.scales[b] = r.f32());
    c.gamma = nb ? float(mean / double(nb)) : 0.0f;
  }
  c.data.assign(p + r.off, p + len);
  return c;
}
// Raw tensor payload: u32 numel, u32 ndim, u32 dims[ndim], f32 data[numel] (hook.rs:744-794).
inline std::vector<uint8_t> serialize_tensor(const Tensor& t) {
  std::vector<uint8_t> o;
  o.reserve(8 + 4 * t.shape.size() + 4 * t.data.size());
  put_u32(o, uint32_t(t.numel()));
  put_u32(o, uint32_t(t.shape.size()));
  for (size_t d : t.shape) put_u32(o, uint32_t(d));
  size_t off = o.size();
  o.resize(off + 4 * t.data.size());
  if (!t.data.empty()) std::memcpy(o.data() + off, t.data.data(), 4 * t.data.size());
  return o;
}
inline Tensor deserialize_tensor(const uint8_t* p, size_t len) {
  if (len < 8) return Tensor::zeros({1});
  Reader r{p, len};
  size_t numel = r.u32();
  uint32_t nd = r.u32();
  std::vector<size_t> shape;
  for (uint32_t i = 0; i < nd && r.off + 4 <= len; ++i) shape.push_back(r.u32());
  size_t avail = (len - r.off) / 4;
  size_t n = std::min(numel, avail);
  std::vector<float> d(n);
  if (n) std::memcpy(d.data(), p + r.off, 4 * n);
  return Tensor(std::move(d), std::move(shape));
}
}  // namespace wire

class Compressor {
 public:
  virtual ~Compressor() = default;
  virtual Packet compress(const Tensor& gradient, LayerId layer) = 0;
  virtual Tensor decompress(const Packet& packet, LayerId layer) = 0;
  // Feed the averaged, reconstructed gradient back (predictor-based compressors need it).
  virtual void update(LayerId layer, const Tensor& gradient) = 0;
  virtual void step() = 0;
  virtual uint64_t state_hash() const { return 0; }
  virtual void force_sync_layer(LayerId, const Tensor&) {}
  virtual float last_compression_ratio() const { return 1.0f; }
  virtual float last_prediction_error() const { return 0.0f; }
  virtual float quantizer_gamma() const { return 0.0f; }
  virtual const char* name() const = 0;
};

// ---------------------------------------------------------------------------------------------
class PredictionResidualCompressor : public Compressor {
 public:
  explicit PredictionResidualCompressor(const NangilaConfig& cfg, bool error_feedback = true,
                                        bool reference_exact = false)
      : predictor_(cfg.momentum, cfg.warmup_steps),
        quantizer_(cfg.quantize_bits, cfg.dynamic_gamma, reference_exact),
        error_feedback_(error_feedback && !reference_exact),
        adaptive_gain_(!reference_exact) {}

  Tensor prediction_or_zero(LayerId layer, size_t n) const {
    if (predictor_.can_predict(layer)) {
      Tensor p = predictor_.predict(layer);
      if (p.numel() == n) return p;
    }
    return Tensor::zeros({n});
  }

  // Prediction gain. The compressor subtracts kappa * g_hat, with kappa the least-squares shrinkage
  // <g + ef, g_hat> / <g_hat, g_hat> clipped to [0, 1]: 1 when the momentum predictor tracks the
  // gradient, near 0 when consecutive gradients are dominated by mini-batch noise (a full-size
  // prediction would then make the residual larger than the gradient and, through error feedback,
  // amplify the predictor's own quantization noise). kappa travels in the block-scaled payload;
  // single-scale payloads carry it as the NO_PREDICTION flag (kappa = 0) or its absence (kappa = 1).
  void set_adaptive_gain(bool on) { adaptive_gain_ = on; }
  float last_gain() const { return last_gain_; }

  Packet compress(const Tensor& g, LayerId layer) override {
    const bool can = predictor_.can_predict(layer);
    Tensor pred = prediction_or_zero(layer, g.numel());
    Tensor x = g;  // g + ef
    auto ef_it = ef_.find(layer);
    if (error_feedback_ && ef_it != ef_.end() && ef_it->second.size() == x.data.size())
      for (size_t i = 0; i < x.data.size(); ++i) x.data[i] += ef_it->second[i];
    float kappa = can ? 1.0f : 0.0f;
    if (can && adaptive_gain_) {
      double xp = 0, pp = 0;
      for (size_t i = 0; i < x.data.size(); ++i) {
        xp += double(x.data[i]) * double(pred.data[i]);
        pp += double(pred.data[i]) * double(pred.data[i]);
      }
      kappa = pp > 0 ? float(std::min(std::max(xp / pp, 0.0), 1.0)) : 0.0f;
      if (quantizer_.block_size() == 0) kappa = kappa >= 0.5f ? 1.0f : 0.0f;  // only the flag can travel
    }
    last_gain_ = kappa;
    Tensor resid = x;
    if (kappa != 0.0f)
      for (size_t i = 0; i < resid.data.size(); ++i) resid.data[i] -= kappa * pred.data[i];
    const float gn = g.norm();
    last_pred_error_ = gn > 0 ? resid.norm() / gn : 0.0f;
    CompressedTensor c = quantizer_.quantize(resid, layer, step_);
    c.shape = g.shape;
    c.pred_gain = kappa;
    if (error_feedback_) {
      Tensor deq = quantizer_.dequantize(c);
      std::vector<float>& ef = ef_[layer];
      ef.resize(resid.data.size());
      for (size_t i = 0; i < ef.size(); ++i) ef[i] = resid.data[i] - deq.data[i];
    }
    std::vector<uint8_t> payload = wire::serialize_compressed(c);
    last_ratio_ = float(g.numel() * 4) / float(std::max<size_t>(payload.size(), 1));
    PacketHeader h = PacketHeader::new_driver(uint32_t(step_), layer);
    if (kappa == 0.0f && can) h.flags |= flags::NO_PREDICTION;
    return Packet(h, std::move(payload));
  }
  static float packet_gain(const Packet& p, const CompressedTensor& c) {
    if (p.header.flags & flags::NO_PREDICTION) return 0.0f;
    return c.block ? c.pred_gain : 1.0f;
  }
  Tensor decompress(const Packet& p, LayerId layer) override {
    CompressedTensor c = wire::deserialize_compressed(p.payload.data(), p.payload.size());
    Tensor out = quantizer_.dequantize(c);
    const float kappa = packet_gain(p, c);
    if (kappa != 0.0f && predictor_.can_predict(layer)) {
      Tensor pred = predictor_.predict(layer);
      if (pred.numel() == out.numel())
        for (size_t i = 0; i < out.data.size(); ++i) out.data[i] += kappa * pred.data[i];
    }
    out.shape = c.shape.empty() ? std::vector<size_t>{out.numel()} : c.shape;
    return out;
  }
  Tensor decompress_partial(const Packet& p, LayerId layer, size_t start, size_t end) {
    CompressedTensor c = wire::deserialize_compressed(p.payload.data(), p.payload.size());
    Tensor resid = quantizer_.dequantize_partial(c, start, end);
    const float kappa = packet_gain(p, c);
    if (kappa != 0.0f && predictor_.can_predict(layer)) {
      Tensor pred = predictor_.predict_partial(layer, start, end);
      if (pred.numel() == resid.numel()) return pred.scale(kappa).add(resid);
    }
    return resid;
  }
  void update(LayerId layer, const Tensor& g) override { predictor_.update(layer, g); }
  void step() override {
    ++step_;
    predictor_.step();
  }
  uint64_t state_hash() const override { return predictor_.state_hash(); }
  void force_sync_layer(LayerId layer, const Tensor& g) override {
    predictor_.force_sync_layer(layer, g);
    ef_.erase(layer);
  }
  float last_compression_ratio() const override { return last_ratio_; }
  float last_prediction_error() const override { return last_pred_error_; }
  float quantizer_gamma() const override { return quantizer_.gamma(); }
  const char* name() const override { return "prediction_residual"; }

  Predictor& predictor() { return predictor_; }
  const Predictor& predictor() const { return predictor_; }
  Quantizer& quantizer() { return quantizer_; }
  std::map<LayerId, std::vector<float>>& error_feedback() { return ef_; }
  uint64_t current_step() const { return step_; }
  void set_step(uint64_t s) { step_ = s; }

 private:
  Predictor predictor_;
  Quantizer quantizer_;
  bool error_feedback_;
  std::map<LayerId, std::vector<float>> ef_;
  bool adaptive_gain_ = true;
  float last_gain_ = 1.0f;
  uint64_t step_ = 0;
  float last_ratio_ = 1.0f;
  float last_pred_error_ = 0.0f;
};

// ---------------------------------------------------------------------------------------------
// DGC payload: u32 numel, u32 k, u32 ndim, u32 dims[ndim], u32 index[k], f32 value[k].
struct SparseTensor {
  std::vector<uint32_t> indices;
  std::vector<float> values;
  std::vector<size_t> shape;
  size_t numel = 0;
  float compression_ratio() const {
    size_t b = indices.size() * 8;
    return b == 0 ? 1.0f : float(numel * 4) / float(b);
  }
};

class DGCCompressor : public Compressor {
 public:
  // momentum_correction = 0 reproduces the reference (plain residual accumulation).
  explicit DGCCompressor(const NangilaConfig& cfg, float momentum_correction = 0.0f)
      : sparsity_(cfg.dgc_sparsity), mc_(momentum_correction) {}

  static size_t keep_count(size_t numel, float sparsity) {
    return size_t(std::ceil(float(numel) * (1.0f - sparsity)));
  }
  // Indices of the k largest |v| (ties broken towards the lower index), in descending magnitude.
  static std::vector<uint32_t> top_k(const std::vector<float>& v, size_t k) {
    std::vector<uint32_t> idx(v.size());
    std::iota(idx.begin(), idx.end(), 0u);
    if (k >= v.size()) return idx;
    auto cmp = [&v](uint32_t a, uint32_t b) {
      float fa = std::fabs(v[a]), fb = std::fabs(v[b]);
      return fa > fb || (fa == fb && a < b);
    };
    std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), cmp);
    idx.resize(k);
    return idx;
  }

  Packet compress(const Tensor& g, LayerId layer) override {
    std::vector<float>& v = residual_[layer];
    if (v.size() != g.numel()) v.assign(g.numel(), 0.0f);
    if (mc_ > 0.0f) {
      std::vector<float>& u = velocity_[layer];
      if (u.size() != g.numel()) u.assign(g.numel(), 0.0f);
      for (size_t i = 0; i < v.size(); ++i) {
        u[i] = mc_ * u[i] + g.data[i];
        v[i] += u[i];
      }
    } else {
      for (size_t i = 0; i < v.size(); ++i) v[i] += g.data[i];
    }
    size_t k = keep_count(v.size(), sparsity_);
    SparseTensor s;
    s.indices = top_k(v, k);
    s.values.reserve(s.indices.size());
    for (uint32_t i : s.indices) s.values.push_back(v[i]);
    for (uint32_t i : s.indices) v[i] = 0.0f;
    if (mc_ > 0.0f) {
      std::vector<float>& u = velocity_[layer];
      for (uint32_t i : s.indices) u[i] = 0.0f;  // momentum-factor masking
    }
    s.shape = g.shape;
    s.numel = g.numel();
    last_ratio_ = s.compression_ratio();
    return Packet(PacketHeader::new_driver(uint32_t(step_), layer), serialize(s));
  }
  Tensor decompress(const Packet& p, LayerId) override {
    SparseTensor s = deserialize(p.payload.data(), p.payload.size());
    std::vector<float> d(s.numel, 0.0f);
    for (size_t i = 0; i < s.indices.size(); ++i) {
      if (s.indices[i] >= d.size())
        throw NangilaError::invalid_format("Index " + std::to_string(s.indices[i]) +
                                           " out of bounds for size " + std::to_string(d.size()));
      d[s.indices[i]] = s.values[i];
    }
    return Tensor(std::move(d), s.shape.empty() ? std::vector<size_t>{s.numel} : s.shape);
  }
  void update(LayerId, const Tensor&) override {}
  void step() override { ++step_; }
  float last_compression_ratio() const override { return last_ratio_; }
  const char* name() const override { return "dgc"; }
  std::map<LayerId, std::vector<float>>& residuals() { return residual_; }

  static std::vector<uint8_t> serialize(const SparseTensor& s) {
    std::vector<uint8_t> o;
    wire::put_u32(o, uint32_t(s.numel));
    wire::put_u32(o, uint32_t(s.indices.size()));
    wire::put_u32(o, uint32_t(s.shape.size()));
    for (size_t d : s.shape) wire::put_u32(o, uint32_t(d));
    for (uint32_t i : s.indices) wire::put_u32(o, i);
    for (float f : s.values) wire::put_f32(o, f);
    return o;
  }
  static SparseTensor deserialize(const uint8_t* p, size_t len) {
    wire::Reader r{p, len};
    SparseTensor s;
    s.numel = r.u32();
    uint32_t k = r.u32();
    uint32_t nd = r.u32();
    for (uint32_t i = 0; i < nd; ++i) s.shape.push_back(r.u32());
    if (!r.ok || r.off + size_t(k) * 8 > len) throw NangilaError::invalid_format("truncated sparse payload");
    s.indices.resize(k);
    s.values.resize(k);
    for (uint32_t i = 0; i < k; ++i) s.indices[i] = r.u32();
    for (uint32_t i = 0; i < k; ++i) s.values[i] = r.f32();
    return s;
  }

 private:
  float sparsity_;
  float mc_;
  std::map<LayerId, std::vector<float>> residual_;
  std::map<LayerId, std::vector<float>> velocity_;
  uint64_t step_ = 0;
  float last_ratio_ = 1.0f;
};

// ---------------------------------------------------------------------------------------------
// Row-major dense helpers for PowerSGD.
struct Mat {
  size_t rows = 0, cols = 0;
  std::vector<float> a;
  Mat() = default;
  Mat(size_t r, size_t c) : rows(r), cols(c), a(r * c, 0.0f) {}
  float& at(size_t i, size_t j) { return a[i * cols + j]; }
  float at(size_t i, size_t j) const { return a[i * cols + j]; }
};
// Classical Gram-Schmidt on the columns, in column order; a column of norm <= 1e-10 is left as is.
inline void orthogonalize_columns(Mat& m) {
  for (size_t i = 0; i < m.cols; ++i) {
    for (size_t j = 0; j < i; ++j) {
      double dot = 0;
      for (size_t r = 0; r < m.rows; ++r) dot += double(m.at(r, i)) * double(m.at(r, j));
      for (size_t r = 0; r < m.rows; ++r) m.at(r, i) -= float(dot) * m.at(r, j);
    }
    double nn = 0;
    for (size_t r = 0; r < m.rows; ++r) nn += double(m.at(r, i)) * double(m.at(r, i));
    float norm = float(std::sqrt(nn));
    if (norm > 1e-10f)
      for (size_t r = 0; r < m.rows; ++r) m.at(r, i) /= norm;
  }
}
inline Mat matmul(const Mat& x, const Mat& y) {  // (r x k)(k x c)
  Mat o(x.rows, y.cols);
  for (size_t i = 0; i < x.rows; ++i)
    for (size_t k = 0; k < x.cols; ++k) {
      float v = x.at(i, k);
      if (v == 0.0f) continue;
      for (size_t j = 0; j < y.cols; ++j) o.at(i, j) += v * y.at(k, j);
    }
  return o;
}
inline Mat matmul_tn(const Mat& x, const Mat& y) {  // x^T y : (k x r)^T (k x c)
  Mat o(x.cols, y.cols);
  for (size_t k = 0; k < x.rows; ++k)
    for (size_t i = 0; i < x.cols; ++i) {
      float v = x.at(k, i);
      if (v == 0.0f) continue;
      for (size_t j = 0; j < y.cols; ++j) o.at(i, j) += v * y.at(k, j);
    }
  return o;
}
inline Mat matmul_nt(const Mat& x, const Mat& y) {  // x y^T : (r x k)(c x k)^T
  Mat o(x.rows, y.rows);
  for (size_t i = 0; i < x.rows; ++i)
    for (size_t j = 0; j < y.rows; ++j) {
      float s = 0;
      for (size_t k = 0; k < x.cols; ++k) s += x.at(i, k) * y.at(j, k);
      o.at(i, j) = s;
    }
  return o;
}

// PowerSGD payload: u32 m, u32 n, u32 r, u32 ndim, u32 dims[ndim], f32 P[m*r], f32 Q[n*r].
class PowerSGDCompressor : public Compressor {
 public:
  explicit PowerSGDCompressor(const NangilaConfig& cfg) : rank_(cfg.power_sgd_rank) {}

  // Deterministic warm start: Q[i][j] = ((i + j) mod 100) / 100, then orthonormalised.
  static Mat initial_q(size_t n, size_t r) {
    Mat q(n, r);
    for (size_t i = 0; i < n; ++i)
      for (size_t j = 0; j < r; ++j) q.at(i, j) = float((i + j) % 100) / 100.0f;
    orthogonalize_columns(q);
    return q;
  }

  Packet compress(const Tensor& g, LayerId layer) override {
    PacketHeader hdr = PacketHeader::new_driver(uint32_t(step_), layer);
    if (g.numel() == 0 || g.shape.empty()) return Packet(hdr, {});
    size_t m = g.shape[0];
    size_t n = 1;
    for (size_t i = 1; i < g.shape.size(); ++i) n *= g.shape[i];
    if (m == 0 || n == 0) return Packet(hdr, {});
    std::vector<float>& mem = residual_[layer];
    if (mem.size() != g.numel()) mem.assign(g.numel(), 0.0f);
    for (size_t i = 0; i < mem.size(); ++i) mem[i] += g.data[i];
    Mat M(m, n);
    M.a = mem;
    size_t r = std::min(rank_, std::min(m, n));
    auto it = q_memory_.find(layer);
    if (it == q_memory_.end() || it->second.rows != n || it->second.cols != r)
      it = q_memory_.insert_or_assign(layer, initial_q(n, r)).first;
    Mat P = matmul(M, it->second);
    orthogonalize_columns(P);
    Mat Q = matmul_tn(M, P);  // n x r, not normalised: P Q^T approximates M
    Mat next = Q;
    orthogonalize_columns(next);
    it->second = std::move(next);
    Mat approx = matmul_nt(P, Q);
    for (size_t i = 0; i < mem.size(); ++i) mem[i] -= approx.a[i];
    std::vector<uint8_t> o;
    wire::put_u32(o, uint32_t(m));
    wire::put_u32(o, uint32_t(n));
    wire::put_u32(o, uint32_t(r));
    wire::put_u32(o, uint32_t(g.shape.size()));
    for (size_t d : g.shape) wire::put_u32(o, uint32_t(d));
    for (float f : P.a) wire::put_f32(o, f);
    for (float f : Q.a) wire::put_f32(o, f);
    last_ratio_ = float(g.numel()) / float(std::max<size_t>((m + n) * r, 1));
    return Packet(hdr, std::move(o));
  }
  Tensor decompress(const Packet& p, LayerId) override {
    if (p.payload.empty()) return Tensor::zeros({0});
    wire::Reader rd{p.payload.data(), p.payload.size()};
    size_t m = rd.u32(), n = rd.u32(), r = rd.u32();
    uint32_t nd = rd.u32();
    std::vector<size_t> shape;
    for (uint32_t i = 0; i < nd; ++i) shape.push_back(rd.u32());
    if (!rd.ok || rd.off + (m + n) * r * 4 > p.payload.size())
      throw NangilaError::invalid_format("truncated PowerSGD payload");
    Mat P(m, r), Q(n, r);
    for (float& f : P.a) f = rd.f32();
    for (float& f : Q.a) f = rd.f32();
    Mat rec = matmul_nt(P, Q);
    return Tensor(std::move(rec.a), std::move(shape));
  }
  void update(LayerId, const Tensor&) override {}
  void step() override { ++step_; }
  float last_compression_ratio() const override { return last_ratio_; }
  const char* name() const override { return "power_sgd"; }
  std::map<LayerId, std::vector<float>>& residuals() { return residual_; }
  std::map<LayerId, Mat>& q_memory() { return q_memory_; }

 private:
  size_t rank_;
  std::map<LayerId, std::vector<float>> residual_;
  std::map<LayerId, Mat> q_memory_;
  uint64_t step_ = 0;
  float last_ratio_ = 1.0f;
};

// Single-stage pipeline wrapper (chaining several stages is not defined by the reference either).
class PipelineCompressor : public Compressor {
 public:
  explicit PipelineCompressor(std::unique_ptr<Compressor> stage) : stage_(std::move(stage)) {}
  Packet compress(const Tensor& g, LayerId l) override { return stage_->compress(g, l); }
  Tensor decompress(const Packet& p, LayerId l) override { return stage_->decompress(p, l); }
  void update(LayerId l, const Tensor& g) override { stage_->update(l, g); }
  void step() override { stage_->step(); }
  uint64_t state_hash() const override { return stage_->state_hash(); }
  void force_sync_layer(LayerId l, const Tensor& g) override { stage_->force_sync_layer(l, g); }
  float last_compression_ratio() const override { return stage_->last_compression_ratio(); }
  float last_prediction_error() const override { return stage_->last_prediction_error(); }
  float quantizer_gamma() const override { return stage_->quantizer_gamma(); }
  const char* name() const override { return stage_->name(); }
  Compressor* stage() { return stage_.get(); }

 private:
  std::unique_ptr<Compressor> stage_;
};

inline std::unique_ptr<Compressor> make_compressor(const NangilaConfig& cfg) {
  switch (cfg.compressor_type) {
    case CompressorType::DGC: return std::make_unique<DGCCompressor>(cfg);
    case CompressorType::PowerSGD: return std::make_unique<PowerSGDCompressor>(cfg);
    default: return std::make_unique<PredictionResidualCompressor>(cfg);
  }
}

}  // namespace nangila
