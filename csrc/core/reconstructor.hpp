// Receiver-side reconstruction helpers: cache of the step's reconstructed Driver gradients and
// synthesis of Passenger gradients from them (g_passenger = alpha * g_driver + beta).
//
// Parity: nangila-core/src/reconstructor.rs:40-60 (driver reconstruction + cache), :69-91 and
// :196-237 (partial variants for sharded consumers), :96-152 (passenger synthesis with missing /
// empty driver checks), :155-182 (reconstruct_all: drivers first, then passengers), :185-188.
#pragma once
#include <map>

#include "mask.hpp"
#include "predictor.hpp"
#include "quantizer.hpp"

namespace nangila {

class Reconstructor {
 public:
  Tensor reconstruct_driver(LayerId id, const CompressedTensor& c, const Predictor& pred, const Quantizer& q) {
    Tensor out = pred.predict(id).add(q.dequantize(c));
    cache_driver_gradient(id, out);
    return out;
  }
  Tensor reconstruct_driver_partial(LayerId id, const CompressedTensor& c, const Predictor& pred,
                                    const Quantizer& q, size_t start, size_t end) const {
    return pred.predict_partial(id, start, end).add(q.dequantize_partial(c, start, end));
  }
  void cache_driver_gradient(LayerId id, Tensor g) {
    driver_cache_[id] = std::move(g);
    last_reconstruction_step_ = current_step_;
    have_reconstruction_ = true;
  }
  bool has_driver(LayerId id) const { return driver_cache_.count(id) != 0; }

  Tensor synthesize_passenger(LayerId id, const TopologyMask& mask) const {
    const LayerRole& role = mask.get_role(id);
    if (!role.is_passenger()) throw NangilaError::layer_not_found(id);
    auto it = driver_cache_.find(role.source_id);
    if (it == driver_cache_.end()) throw NangilaError::layer_not_found(role.source_id);
    if (it->second.numel() == 0)
      throw NangilaError::invalid_format("Driver " + std::to_string(role.source_id) +
                                         " has zero elements, cannot synthesize passenger " + std::to_string(id));
    Tensor out = it->second.scale(role.alpha);
    if (std::fabs(role.beta) > 1e-8f)
      for (float& v : out.data) v += role.beta;
    return out;
  }
  Tensor synthesize_passenger_partial(LayerId id, const TopologyMask& mask, size_t start, size_t end) const {
    Tensor full = synthesize_passenger(id, mask);
    start = std::min(start, full.numel());
    end = std::min(end, full.numel());
    if (start >= end) return Tensor::zeros({0});
    std::vector<float> d(full.data.begin() + start, full.data.begin() + end);
    size_t n = d.size();
    return Tensor(std::move(d), {n});
  }
  // True when the cached drivers were produced in an earlier step than the current one.
  bool cache_is_stale() const { return have_reconstruction_ && last_reconstruction_step_ != current_step_; }

  std::map<LayerId, Tensor> reconstruct_all(const std::map<LayerId, CompressedTensor>& drivers,
                                            const TopologyMask& mask, const Predictor& pred, const Quantizer& q) {
    std::map<LayerId, Tensor> out;
    for (auto& kv : drivers) out[kv.first] = reconstruct_driver(kv.first, kv.second, pred, q);
    for (auto& p : mask.passengers()) out[p.id] = synthesize_passenger(p.id, mask);
    return out;
  }
  void clear_cache() {
    driver_cache_.clear();
    ++current_step_;
  }

 private:
  std::map<LayerId, Tensor> driver_cache_;
  size_t current_step_ = 0;
  size_t last_reconstruction_step_ = 0;
  bool have_reconstruction_ = false;
};

}  // namespace nangila
