// Momentum predictor ("slow head"): g_hat(t+1) = g(t) + mu * (g(t) - g(t-1)), with the two-step
// history held per layer in Q8.23 so every rank computes bit-identical predictions on any host.
//
// Parity: nangila-core/src/predictor.rs:16-74 (history window), :77-91 and :181-254 (memory
// modes with the 10-billion-parameter auto threshold), :157-179 and :256-305 (adaptive momentum:
// window 10, mu in [0.5, 0.95], rate 0.1), :307-384 (predict / predict_partial), :390-417
// (update, step, warm-up), :455-477 (state hash), :480-507 (snapshots, reset, force sync).
#pragma once
#include <algorithm>
#include <map>
#include <numeric>
#include <optional>
#include <set>
#include <vector>

#include "q8_23.hpp"
#include "siphash.hpp"
#include "types.hpp"

namespace nangila {

struct LayerHistorySnapshot {
  std::optional<std::vector<int32_t>> prev;
  std::optional<std::vector<int32_t>> current;
};

enum class MemoryMode { Full, DriversOnly, Auto };

class Predictor {
 public:
  Predictor(float momentum, size_t warmup_steps) : momentum_(momentum), warmup_steps_(warmup_steps) {}

  // --- configuration ---------------------------------------------------------------------
  void set_adaptive_config(float min_mu, float max_mu, float rate, size_t window) {
    min_momentum_ = min_mu;
    max_momentum_ = max_mu;
    adaptation_rate_ = rate;
    error_window_ = window;
  }
  void disable_adaptive_momentum() {
    adaptive_momentum_.clear();
    error_history_.clear();
  }
  void set_memory_mode(MemoryMode m) {
    memory_mode_ = m;
    if (m != MemoryMode::Auto) effective_mode_ = m;
  }
  void set_large_model_threshold(size_t params) { large_model_threshold_ = params; }
  void set_memory_budget_mb(size_t mb) { large_model_threshold_ = mb * 1024 * 1024 / 8; }
  void set_driver_layers(const std::vector<LayerId>& d) { driver_layers_ = std::set<LayerId>(d.begin(), d.end()); }
  bool should_track_layer(LayerId id) const {
    return effective_mode_ == MemoryMode::DriversOnly ? driver_layers_.count(id) != 0 : true;
  }
  struct MemoryStats { MemoryMode mode; size_t total_params, num_layers, estimated_mb; };
  MemoryStats memory_stats() const {
    return {effective_mode_, total_tracked_params_, history_.size(), total_tracked_params_ * 8 / (1024 * 1024)};
  }

  // --- adaptive momentum -------------------------------------------------------------------
  float get_momentum(LayerId id) const {
    auto it = adaptive_momentum_.find(id);
    return it == adaptive_momentum_.end() ? momentum_ : it->second;
  }
  void record_error(LayerId id, float err) {
    auto& h = error_history_[id];
    h.push_back(err);
    if (h.size() > error_window_) h.erase(h.begin());
    if (h.size() >= 3) adapt_momentum(id);
  }

  // --- prediction --------------------------------------------------------------------------
  Tensor predict(LayerId id) const {
    const LayerHistory& h = find(id);
    if (!h.can_predict()) throw NangilaError::insufficient_history(id);
    FixedPointBuffer delta = h.current->sub(*h.prev);
    FixedPointBuffer pred = h.current->add(delta.scale(get_momentum(id)));
    std::vector<float> d = pred.to_f32();
    size_t n = d.size();
    return Tensor(std::move(d), {n});
  }
  Tensor predict_partial(LayerId id, size_t start, size_t end) const {
    const LayerHistory& h = find(id);
    if (!h.can_predict()) throw NangilaError::insufficient_history(id);
    Q8_23 mu = Q8_23::from_f32(get_momentum(id));
    size_t n = std::min(h.current->size(), h.prev->size());
    end = std::min(end, n);
    std::vector<float> out;
    for (size_t i = start; i < end; ++i) {
      Q8_23 now = (*h.current)[i], prev = (*h.prev)[i];
      out.push_back((now + (now - prev) * mu).to_f32());
    }
    size_t len = out.size();
    return Tensor(std::move(out), {len});
  }

  // Always feed the *reconstructed, averaged* gradient so all ranks stay in consensus.
  void update(LayerId id, const Tensor& g) {
    if (!history_.count(id)) total_tracked_params_ += g.numel();
    LayerHistory& h = history_[id];
    h.prev = std::move(h.current);
    h.current = FixedPointBuffer::from_f32(g.data);
  }
  void step() {
    ++step_;
    check_memory_threshold();
    if (step_ >= warmup_steps_) warmed_up_ = true;
  }
  bool is_ready() const { return warmed_up_; }
  bool can_predict(LayerId id) const {
    auto it = history_.find(id);
    return it != history_.end() && it->second.can_predict();
  }
  size_t current_step() const { return step_; }
  void set_step(size_t s) { step_ = s; warmed_up_ = step_ >= warmup_steps_; }
  float momentum() const { return momentum_; }
  void reset() {
    history_.clear();
    step_ = 0;
    warmed_up_ = false;
  }
  size_t num_tracked_layers() const { return history_.size(); }

  // SipHash-1-3 over: step (8 bytes), then per layer in ascending id: id (4 bytes) and the 8-byte
  // buffer hash of prev and of current when present.
  uint64_t state_hash() const {
    SipHasher13 h;
    h.write_usize(step_);
    for (auto& kv : history_) {
      h.write_u32(kv.first);
      if (kv.second.prev) h.write_u64(kv.second.prev->hash());
      if (kv.second.current) h.write_u64(kv.second.current->hash());
    }
    return h.finish();
  }

  std::map<LayerId, LayerHistorySnapshot> export_snapshots() const {
    std::map<LayerId, LayerHistorySnapshot> out;
    for (auto& kv : history_) {
      LayerHistorySnapshot s;
      if (kv.second.prev) s.prev = kv.second.prev->to_bits();
      if (kv.second.current) s.current = kv.second.current->to_bits();
      out[kv.first] = std::move(s);
    }
    return out;
  }
  void restore_snapshots(const std::map<LayerId, LayerHistorySnapshot>& snaps) {
    history_.clear();
    total_tracked_params_ = 0;
    for (auto& kv : snaps) {
      LayerHistory h;
      if (kv.second.prev) h.prev = FixedPointBuffer::from_bits(*kv.second.prev);
      if (kv.second.current) {
        h.current = FixedPointBuffer::from_bits(*kv.second.current);
        total_tracked_params_ += kv.second.current->size();
      }
      history_[kv.first] = std::move(h);
    }
  }
  void reset_layer(LayerId id) { history_.erase(id); }
  // prev = current = g, so the next prediction equals g.
  void force_sync_layer(LayerId id, const Tensor& g) {
    LayerHistory h;
    h.current = FixedPointBuffer::from_f32(g.data);
    h.prev = h.current;
    if (!history_.count(id)) total_tracked_params_ += g.numel();
    history_[id] = std::move(h);
  }

 private:
  struct LayerHistory {
    std::optional<FixedPointBuffer> prev, current;
    bool can_predict() const { return prev.has_value() && current.has_value(); }
  };
  const LayerHistory& find(LayerId id) const {
    auto it = history_.find(id);
    if (it == history_.end()) throw NangilaError::layer_not_found(id);
    return it->second;
  }
  void check_memory_threshold() {
    if (memory_mode_ != MemoryMode::Auto) return;
    size_t est_mb = total_tracked_params_ * 8 / (1024 * 1024);
    size_t thr_mb = large_model_threshold_ * 8 / (1024 * 1024);
    effective_mode_ = est_mb > thr_mb ? MemoryMode::DriversOnly : MemoryMode::Full;
  }
  void adapt_momentum(LayerId id) {
    const auto& h = error_history_[id];
    if (h.size() < 3) return;
    float cur = get_momentum(id);
    float recent = (h[h.size() - 1] + h[h.size() - 2] + h[h.size() - 3]) / 3.0f;
    float older = (h[0] + h[1] + h[2]) / 3.0f;
    float next;
    if (recent > older * 1.1f) next = std::max(cur - adaptation_rate_, min_momentum_);
    else if (recent < older * 0.9f) next = std::min(cur + adaptation_rate_ * 0.5f, max_momentum_);
    else next = cur + (momentum_ - cur) * 0.05f;
    adaptive_momentum_[id] = next;
  }

  float momentum_;
  std::map<LayerId, LayerHistory> history_;
  size_t step_ = 0;
  bool warmed_up_ = false;
  size_t warmup_steps_;
  std::map<LayerId, float> adaptive_momentum_;
  std::map<LayerId, std::vector<float>> error_history_;
  size_t error_window_ = 10;
  float min_momentum_ = 0.5f, max_momentum_ = 0.95f, adaptation_rate_ = 0.1f;
  MemoryMode memory_mode_ = MemoryMode::Auto;
  MemoryMode effective_mode_ = MemoryMode::Full;
  size_t large_model_threshold_ = 10000000000ull;
  size_t total_tracked_params_ = 0;
  std::set<LayerId> driver_layers_;
};

}  // namespace nangila
