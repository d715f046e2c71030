// Sculptor: calibration pass that discovers which layers can be Passengers of which Drivers.
// Per layer it keeps Welford statistics of the gradient L2 norm; per scheduled pair of equal-size
// layers it keeps element-wise streaming means, variances and the co-moment, from which the
// element-averaged Pearson correlation and the regression (alpha, beta) follow.
//
// Parity: nangila-core/src/sculptor.rs:33-72 (norm statistics), :76-170 (pair statistics and
// correlation), :238-255 (record), :259-383 (end_step with the Full / kNN-by-norm / random /
// hierarchical-by-size pair strategies), :396-399 (equal sizes only), :428-474 (coupling),
// :477-550 (greedy mask: layers by descending std-dev of norm; a layer becomes the Passenger of
// the already-assigned Driver with the largest |corr| > threshold, else a Driver), :206-224
// (large-model preset), :553-604 (matrix, counters, reset).
// Additions: a layer id seen twice closes the open step automatically, and pair results computed
// elsewhere (the device statistics kernel) can be injected with set_pair_result().
#pragma once
#include <algorithm>
#include <cmath>
#include <map>
#include <optional>
#include <utility>
#include <vector>

#include "mask.hpp"
#include "siphash.hpp"
#include "types.hpp"

namespace nangila {

struct SamplingStrategy {
  enum Kind { Full, KNearestNeighbors, RandomSampling, Hierarchical } kind = Full;
  size_t param = 0;  // k / pairs_per_layer / max_cluster_size
};

class Sculptor {
 public:
  explicit Sculptor(float threshold = 0.95f) : threshold_(threshold) {}
  static Sculptor new_large_model(float threshold, size_t num_layers) {
    Sculptor s(threshold);
    if (num_layers < 100) s.strategy_ = {SamplingStrategy::Full, 0};
    else if (num_layers < 500) s.strategy_ = {SamplingStrategy::KNearestNeighbors, 20};
    else s.strategy_ = {SamplingStrategy::KNearestNeighbors, 10};
    return s;
  }
  void set_sampling_strategy(SamplingStrategy s) { strategy_ = s; }
  SamplingStrategy sampling_strategy() const { return strategy_; }

  void record(LayerId id, const float* g, size_t n) {
    if (auto_end_step_ && current_.count(id)) end_step();
    layer_sizes_[id] = n;
    double ss = 0;
    for (size_t i = 0; i < n; ++i) ss += double(g[i]) * double(g[i]);
    stats_[id].update(std::sqrt(ss));
    current_[id].assign(g, g + n);
  }
  void record(LayerId id, const Tensor& t) { record(id, t.data.data(), t.data.size()); }
  // Norm-only record: for callers that compute pair statistics elsewhere.
  void record_norm(LayerId id, double l2_norm, size_t numel) {
    layer_sizes_[id] = numel;
    stats_[id].update(l2_norm);
  }

  void end_step() {
    std::vector<LayerId> ids;
    for (auto& kv : current_) ids.push_back(kv.first);  // map order = ascending id
    for (auto& pr : scheduled_pairs(ids)) update_pair(pr.first, pr.second);
    current_.clear();
    ++step_count_;
  }
  // The pairs `end_step` would update for this set of layers (exposed so a device implementation
  // follows the same schedule).
  std::vector<std::pair<LayerId, LayerId>> scheduled_pairs(const std::vector<LayerId>& ids) const {
    std::vector<std::pair<LayerId, LayerId>> out;
    auto same_size = [this](LayerId a, LayerId b) {
      auto ia = layer_sizes_.find(a), ib = layer_sizes_.find(b);
      return ia != layer_sizes_.end() && ib != layer_sizes_.end() && ia->second == ib->second;
    };
    auto push = [&](LayerId a, LayerId b) {
      if (a != b && same_size(a, b)) out.emplace_back(a, b);
    };
    switch (strategy_.kind) {
      case SamplingStrategy::Full:
        for (size_t i = 0; i < ids.size(); ++i)
          for (size_t j = i + 1; j < ids.size(); ++j) push(ids[i], ids[j]);
        break;
      case SamplingStrategy::KNearestNeighbors: {
        std::vector<std::pair<LayerId, double>> norms;
        for (LayerId id : ids) {
          auto it = current_.find(id);
          double ss = 0;
          if (it != current_.end())
            for (float v : it->second) ss += double(v) * double(v);
          else if (stats_.count(id)) ss = stats_.at(id).last * stats_.at(id).last;
          norms.emplace_back(id, std::sqrt(ss));
        }
        std::stable_sort(norms.begin(), norms.end(), [](auto& a, auto& b) { return a.second < b.second; });
        size_t k = strategy_.param;
        for (size_t i = 0; i < norms.size(); ++i) {
          size_t s = i >= k / 2 ? i - k / 2 : 0;
          size_t e = std::min(i + k / 2 + 1, norms.size());
          for (size_t j = s; j < e; ++j) push(norms[i].first, norms[j].first);
        }
        break;
      }
      case SamplingStrategy::RandomSampling:
        for (LayerId a : ids) {
          SipHasher13 h;
          h.write_u32(a);
          h.write_usize(step_count_);
          uint64_t seed = h.finish();
          for (size_t j = 0; j < strategy_.param; ++j) push(a, ids[size_t((seed + j) % ids.size())]);
        }
        break;
      case SamplingStrategy::Hierarchical: {
        std::map<size_t, std::vector<LayerId>> groups;
        for (LayerId id : ids)
          if (layer_sizes_.count(id)) groups[layer_sizes_.at(id)].push_back(id);
        size_t k = strategy_.param;
        for (auto& kv : groups) {
          auto& g = kv.second;
          if (g.size() <= k) {
            for (size_t i = 0; i < g.size(); ++i)
              for (size_t j = i + 1; j < g.size(); ++j) push(g[i], g[j]);
          } else {
            for (size_t i = 0; i < g.size(); ++i) {
              size_t s = i >= k / 2 ? i - k / 2 : 0;
              size_t e = std::min(i + k / 2 + 1, g.size());
              for (size_t j = s; j < e; ++j) push(g[i], g[j]);
            }
          }
        }
        break;
      }
    }
    return out;
  }

  // Inject a finished pair result: correlation and regression "hi ≈ alpha_lo_to_hi * lo + beta"
  // in both directions, as a device implementation produces them.
  void set_pair_result(LayerId a, LayerId b, size_t count, float corr, float alpha_ab, float beta_ab,
                       float alpha_ba, float beta_ba) {
    Injected r{count, corr, alpha_ab, beta_ab, alpha_ba, beta_ba};
    if (a > b) {
      std::swap(a, b);
      std::swap(r.alpha_ab, r.alpha_ba);
      std::swap(r.beta_ab, r.beta_ba);
    }
    injected_[{a, b}] = r;
  }
  void note_step() { ++step_count_; }

  std::optional<float> correlation(LayerId a, LayerId b) const {
    auto key = std::minmax(a, b);
    auto inj = injected_.find({key.first, key.second});
    if (inj != injected_.end()) {
      if (inj->second.count < 2) return std::nullopt;
      return inj->second.corr;
    }
    auto it = pairs_.find({key.first, key.second});
    if (it == pairs_.end()) return std::nullopt;
    return it->second.correlation();
  }
  // passenger ≈ alpha * driver + beta (element-wise regression, averaged over elements).
  std::optional<std::pair<float, float>> coupling(LayerId driver, LayerId passenger) const {
    auto key = std::minmax(driver, passenger);
    auto inj = injected_.find({key.first, key.second});
    if (inj != injected_.end()) {
      if (inj->second.count < 2) return std::nullopt;
      return driver < passenger ? std::make_pair(inj->second.alpha_ab, inj->second.beta_ab)
                                : std::make_pair(inj->second.alpha_ba, inj->second.beta_ba);
    }
    auto it = pairs_.find({key.first, key.second});
    if (it == pairs_.end() || it->second.count < 2) return std::nullopt;
    const Pair& c = it->second;
    bool driver_is_i = driver < passenger;
    const auto& mean_d = driver_is_i ? c.mean_i : c.mean_j;
    const auto& mean_p = driver_is_i ? c.mean_j : c.mean_i;
    const auto& m2_d = driver_is_i ? c.m2_i : c.m2_j;
    double sa = 0, sb = 0;
    size_t valid = 0;
    for (size_t k = 0; k < c.size; ++k) {
      double var_d = m2_d[k] / double(c.count - 1);
      double cov = c.co[k] / double(c.count - 1);
      if (var_d > 1e-10) {
        double alpha = cov / var_d;
        sa += alpha;
        sb += mean_p[k] - alpha * mean_d[k];
        ++valid;
      }
    }
    if (!valid) return std::nullopt;
    return std::make_pair(float(sa / double(valid)), float(sb / double(valid)));
  }

  TopologyMask generate_mask() const {
    if (stats_.size() < 2) throw NangilaError::insufficient_samples();
    std::vector<std::pair<LayerId, double>> order;
    for (auto& kv : stats_) order.emplace_back(kv.first, kv.second.std_dev());
    std::stable_sort(order.begin(), order.end(), [](auto& a, auto& b) { return a.second > b.second; });
    TopologyMask mask;
    std::vector<LayerId> drivers;
    for (auto& ov : order) {
      LayerId id = ov.first;
      bool found = false;
      LayerId best = 0;
      float best_corr = 0, best_a = 0, best_b = 0;
      for (LayerId d : drivers) {
        auto c = correlation(id, d);
        if (!c || !(std::fabs(*c) > threshold_)) continue;
        auto ab = coupling(d, id);
        if (!ab) continue;
        if (!found || std::fabs(*c) > std::fabs(best_corr)) {
          found = true;
          best = d;
          best_corr = *c;
          best_a = ab->first;
          best_b = ab->second;
        }
      }
      if (found) {
        mask.add_passenger(id, best, best_a, best_b);
      } else {
        mask.add_driver(id);
        drivers.push_back(id);
      }
    }
    return mask;
  }

  size_t num_samples() const {
    size_t m = 0;
    bool first = true;
    for (auto& kv : stats_) {
      m = first ? kv.second.count : std::min(m, kv.second.count);
      first = false;
    }
    return m;
  }
  size_t num_layers() const { return stats_.size(); }
  size_t num_steps() const { return step_count_; }
  size_t num_pairs() const { return pairs_.size() + injected_.size(); }
  float threshold() const { return threshold_; }
  void set_auto_end_step(bool b) { auto_end_step_ = b; }
  bool has_open_step() const { return !current_.empty(); }
  std::vector<LayerId> layer_ids() const {
    std::vector<LayerId> v;
    for (auto& kv : stats_) v.push_back(kv.first);
    return v;
  }
  double norm_std_dev(LayerId id) const {
    auto it = stats_.find(id);
    return it == stats_.end() ? 0.0 : it->second.std_dev();
  }

  std::optional<std::vector<std::vector<float>>> correlation_matrix() const {
    std::vector<LayerId> ids = layer_ids();
    if (ids.size() < 2) return std::nullopt;
    size_t n = ids.size();
    std::vector<std::vector<float>> m(n, std::vector<float>(n, 0.0f));
    for (size_t i = 0; i < n; ++i) {
      m[i][i] = 1.0f;
      for (size_t j = i + 1; j < n; ++j) {
        float c = correlation(ids[i], ids[j]).value_or(0.0f);
        m[i][j] = m[j][i] = c;
      }
    }
    return m;
  }
  void reset() {
    stats_.clear();
    pairs_.clear();
    injected_.clear();
    current_.clear();
    layer_sizes_.clear();
    step_count_ = 0;
  }

 private:
  struct NormStats {
    size_t count = 0;
    double mean = 0, m2 = 0, last = 0;
    void update(double x) {
      ++count;
      double d = x - mean;
      mean += d / double(count);
      m2 += d * (x - mean);
      last = x;
    }
    double std_dev() const { return count < 2 ? 0.0 : std::sqrt(m2 / double(count - 1)); }
  };
  struct Pair {
    size_t count = 0, size = 0;
    std::vector<double> mean_i, mean_j, co, m2_i, m2_j;
    explicit Pair(size_t n = 0) : size(n), mean_i(n), mean_j(n), co(n), m2_i(n), m2_j(n) {}
    void update(const std::vector<float>& gi, const std::vector<float>& gj) {
      if (gi.size() != size || gj.size() != size) return;
      ++count;
      double n = double(count);
      for (size_t k = 0; k < size; ++k) {
        double vi = gi[k], vj = gj[k];
        double di = vi - mean_i[k], dj = vj - mean_j[k];
        mean_i[k] += di / n;
        mean_j[k] += dj / n;
        double di2 = vi - mean_i[k], dj2 = vj - mean_j[k];
        m2_i[k] += di * di2;
        m2_j[k] += dj * dj2;
        co[k] += di * dj2;
      }
    }
    std::optional<float> correlation() const {
      if (count < 2) return std::nullopt;
      double s = 0;
      size_t valid = 0;
      for (size_t k = 0; k < size; ++k) {
        double vi = m2_i[k] / double(count - 1), vj = m2_j[k] / double(count - 1);
        double cov = co[k] / double(count - 1);
        double den = std::sqrt(vi * vj);
        if (den > 1e-10) {
          s += cov / den;
          ++valid;
        }
      }
      if (!valid) return std::nullopt;
      return float(s / double(valid));
    }
  };
  struct Injected { size_t count; float corr, alpha_ab, beta_ab, alpha_ba, beta_ba; };

  void update_pair(LayerId a, LayerId b) {
    auto ia = current_.find(a), ib = current_.find(b);
    if (ia == current_.end() || ib == current_.end()) return;
    if (ia->second.size() != ib->second.size()) return;
    if (a > b) {
      std::swap(a, b);
      std::swap(ia, ib);
    }
    auto it = pairs_.find({a, b});
    if (it == pairs_.end()) it = pairs_.emplace(std::make_pair(a, b), Pair(ia->second.size())).first;
    it->second.update(ia->second, ib->second);
  }

  float threshold_;
  std::map<LayerId, NormStats> stats_;
  std::map<std::pair<LayerId, LayerId>, Pair> pairs_;
  std::map<std::pair<LayerId, LayerId>, Injected> injected_;
  std::map<LayerId, std::vector<float>> current_;
  std::map<LayerId, size_t> layer_sizes_;
  size_t step_count_ = 0;
  SamplingStrategy strategy_;
  bool auto_end_step_ = true;
};

}  // namespace nangila
