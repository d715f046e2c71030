// Basic value types shared by the host-side core: a flat FP32 tensor with a shape, the wire
// data-type enum, layer ids and the error type.
//
// Parity: nangila-core/src/lib.rs:83-112 (DataType), :114-224 (Tensor), :226-253 (errors).
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace nangila {

using LayerId = uint32_t;

enum class DataType : int32_t { F32 = 0, F16 = 1, BF16 = 2 };

inline size_t element_size(DataType t) { return t == DataType::F32 ? 4 : 2; }

inline bool data_type_from_i32(int32_t v, DataType* out) {
  if (v < 0 || v > 2) return false;
  *out = static_cast<DataType>(v);
  return true;
}

enum class ErrorKind {
  ShapeMismatch,
  LayerNotFound,
  InsufficientHistory,
  InsufficientSamples,
  InvalidFormat,
  Io,
  Config,
};

class NangilaError : public std::runtime_error {
 public:
  NangilaError(ErrorKind kind, const std::string& msg) : std::runtime_error(msg), kind_(kind) {}
  ErrorKind kind() const { return kind_; }

  static NangilaError layer_not_found(LayerId id) {
    return NangilaError(ErrorKind::LayerNotFound, "Layer not found: " + std::to_string(id));
  }
  static NangilaError insufficient_history(LayerId id) {
    return NangilaError(ErrorKind::InsufficientHistory,
                        "Insufficient history for layer " + std::to_string(id));
  }
  static NangilaError insufficient_samples() {
    return NangilaError(ErrorKind::InsufficientSamples,
                        "Insufficient calibration samples: need at least 2 layers");
  }
  static NangilaError invalid_format(const std::string& m) {
    return NangilaError(ErrorKind::InvalidFormat, "Invalid format: " + m);
  }
  static NangilaError io(const std::string& m) { return NangilaError(ErrorKind::Io, "IO error: " + m); }

 private:
  ErrorKind kind_;
};

// Flat FP32 tensor. All host-side math is done in FP32 whatever the original dtype was; `dtype`
// only records what the caller handed in so that it can be converted back on the way out.
struct Tensor {
  std::vector<float> data;
  std::vector<size_t> shape;
  DataType dtype = DataType::F32;

  Tensor() = default;
  Tensor(std::vector<float> d, std::vector<size_t> s, DataType t = DataType::F32)
      : data(std::move(d)), shape(std::move(s)), dtype(t) {}

  static Tensor zeros(std::vector<size_t> s) {
    size_t n = 1;
    for (size_t d : s) n *= d;
    return Tensor(std::vector<float>(n, 0.0f), std::move(s));
  }
  static Tensor from_slice(const float* p, size_t n) {
    return Tensor(std::vector<float>(p, p + n), {n});
  }

  size_t numel() const { return data.size(); }

  void check_same(const Tensor& o) const {
    if (o.data.size() != data.size())
      throw NangilaError(ErrorKind::ShapeMismatch,
                         "Shape mismatch: " + std::to_string(data.size()) + " vs " +
                             std::to_string(o.data.size()));
  }
  Tensor sub(const Tensor& o) const {
    check_same(o);
    Tensor r(std::vector<float>(data.size()), shape, dtype);
    for (size_t i = 0; i < data.size(); ++i) r.data[i] = data[i] - o.data[i];
    return r;
  }
  Tensor add(const Tensor& o) const {
    check_same(o);
    Tensor r(std::vector<float>(data.size()), shape, dtype);
    for (size_t i = 0; i < data.size(); ++i) r.data[i] = data[i] + o.data[i];
    return r;
  }
  Tensor scale(float f) const {
    Tensor r(std::vector<float>(data.size()), shape, dtype);
    for (size_t i = 0; i < data.size(); ++i) r.data[i] = data[i] * f;
    return r;
  }
  float norm() const {
    double s = 0;
    for (float v : data) s += double(v) * double(v);
    return static_cast<float>(std::sqrt(s));
  }
};

}  // namespace nangila
