// Boundary-node ("ghost") prediction: signal history, the three predictors, the classifier that
// picks one, accuracy bookkeeping and the confidence -> speculative-depth rule.
// Behavioural reference: nangila-spice/nangila-node/src/predictor.rs:27-580, ghost.rs:19-226.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace nspice {

struct SignalState {
    double value = 0, gradient = 0, second_derivative = 0, time = 0;
    std::vector<std::pair<double, double>> history;  // (time, voltage), newest last, at most 16
    double gradient_before = 0;  // slope before the newest sample was recorded (amend() needs it)
    void record(double t, double v) {
        double old = gradient;
        gradient_before = old;
        if (t > time) {
            double dt = t - time;
            gradient = (v - value) / dt;
            second_derivative = (gradient - old) / dt;
        }
        value = v;
        time = t;
        history.emplace_back(t, v);
        if (history.size() > 16) history.erase(history.begin());
    }
};

// Replaces the value of the newest sample (the first value received for a time point was a speculative one and the
// relaxation has since settled on another): slopes are taken again from the sample before it.
inline void amend_newest(SignalState& s, double v) {
    if (s.history.empty()) { s.value = v; return; }
    s.history.back().second = v;
    s.value = v;
    if (s.history.size() >= 2) {
        const auto& prev = s.history[s.history.size() - 2];
        const double dt = s.time - prev.first;
        if (dt > 0.0) {
            s.gradient = (v - prev.second) / dt;
            s.second_derivative = (s.gradient - s.gradient_before) / dt;
        }
    }
}

inline double predict_linear(const SignalState& s, double t) { return s.value + s.gradient * (t - s.time); }

inline double predict_exponential(const SignalState& s, double t, double tau, double asymptote) {
    return asymptote + (s.value - asymptote) * std::exp(-(t - s.time) / tau);
}

// Slope of the recorded history around time t (central difference over the neighbours when there are
// enough points, else the bracketing pair).
inline double history_slope(const std::vector<std::pair<double, double>>& h, double t) {
    size_t n = h.size();
    if (n < 2) return 0.0;
    size_t idx = n - 2;
    for (size_t i = 0; i + 1 < n; ++i)
        if (h[i + 1].first >= t) { idx = i; break; }
    double dt = h[idx + 1].first - h[idx].first;
    if (std::fabs(dt) < 1e-30) return 0.0;
    if (idx > 0 && idx + 2 < n) {
        double wide = h[idx + 2].first - h[idx - 1].first;
        if (std::fabs(wide) > 1e-30) return (h[idx + 2].second - h[idx - 1].second) / wide;
    }
    return (h[idx + 1].second - h[idx].second) / dt;
}

// RK4 over the slope field estimated from history; the end slope is extrapolated with the curvature.
inline double predict_rk4(const SignalState& s, double t) {
    double h = t - s.time;
    if (std::fabs(h) < 1e-30 || s.history.size() < 2) return s.value;
    double k1 = history_slope(s.history, s.time);
    double k2 = history_slope(s.history, s.time + 0.5 * h);
    double k4 = std::fabs(s.second_derivative) > 1e-20 ? k1 + s.second_derivative * h : history_slope(s.history, s.time + h);
    return s.value + h / 6.0 * (k1 + 4.0 * k2 + k4);
}

enum class SignalClass { Smooth, Decaying, Stiff, Unknown };

inline SignalClass classify_signal(const SignalState& s) {
    size_t n = s.history.size();
    if (n < 4) return SignalClass::Unknown;
    std::vector<double> g, gt;  // gradients and the dt that follows each
    for (size_t i = 1; i < n; ++i) {
        double dt = s.history[i].first - s.history[i - 1].first;
        if (std::fabs(dt) > 1e-30) g.push_back((s.history[i].second - s.history[i - 1].second) / dt);
    }
    if (g.size() < 3) return SignalClass::Unknown;
    int flips = 0;
    for (size_t i = 1; i < g.size(); ++i) if (g[i] * g[i - 1] < 0.0) ++flips;
    if (double(flips) / double(g.size() - 1) > 0.3) return SignalClass::Stiff;
    std::vector<double> c;
    for (size_t i = 1; i < g.size() && i + 1 < n; ++i) {
        double dt = s.history[i + 1].first - s.history[i].first;
        if (std::fabs(dt) > 1e-30) c.push_back((g[i] - g[i - 1]) / dt);
    }
    if (c.size() >= 2) {
        bool same_sign = true;
        for (size_t i = 1; i < c.size(); ++i) if (c[i] * c[i - 1] < 0.0) same_sign = false;
        size_t half = g.size() / 2;
        double early = 0, late = 0;
        for (size_t i = 0; i < half; ++i) early += std::fabs(g[i]);
        for (size_t i = half; i < g.size(); ++i) late += std::fabs(g[i]);
        early /= double(half);
        late /= double(g.size() - half);
        if (same_sign && late < 0.7 * early) return SignalClass::Decaying;
    }
    double grad = std::fabs(s.gradient);
    if (grad > 1e-15 && std::fabs(s.second_derivative) / (grad * grad) > 1e6) return SignalClass::Stiff;
    return SignalClass::Smooth;
}

struct Prediction { double value; const char* predictor; };

inline Prediction select_and_predict(const SignalState& s, double t, double default_tau = 10e-12) {
    switch (classify_signal(s)) {
        case SignalClass::Decaying: {
            double tau = (std::fabs(s.gradient) > 1e-15 && std::fabs(s.value) > 1e-15) ? std::fabs(s.value / s.gradient) : default_tau;
            return {predict_exponential(s, t, tau, 0.0), "Exponential"};
        }
        case SignalClass::Stiff: return {predict_rk4(s, t), "RungeKutta"};
        default: return {predict_linear(s, t), "Linear"};
    }
}

struct NodeAccuracy {
    uint64_t net_id = 0;
    std::string predictor;
    uint64_t total = 0, hits = 0;
    double sum_error = 0, max_error = 0;
    std::vector<double> recent;  // last 32 absolute errors
    void record(double predicted, double actual, double reltol) {
        double err = std::fabs(actual - predicted);
        double rel = std::fabs(actual) > 1e-15 ? err / std::fabs(actual) : err;
        ++total;
        if (rel < reltol) ++hits;
        sum_error += err;
        max_error = std::max(max_error, err);
        recent.push_back(err);
        if (recent.size() > 32) recent.erase(recent.begin());
    }
    double hit_rate() const { return total ? double(hits) / double(total) : 1.0; }
    double mean_error() const { return total ? sum_error / double(total) : 0.0; }
    // > 0 when the late half of the recent errors is larger than the early half
    double error_trend() const {
        if (recent.size() < 4) return 0.0;
        size_t h = recent.size() / 2;
        double a = 0, b = 0;
        for (size_t i = 0; i < h; ++i) a += recent[i];
        for (size_t i = h; i < recent.size(); ++i) b += recent[i];
        return b / double(recent.size() - h) - a / double(h);
    }
};

struct AccuracyLogger {
    std::vector<NodeAccuracy> nodes;
    NodeAccuracy& get(uint64_t id, const std::string& predictor) {
        auto it = index_.find(id);
        if (it != index_.end() && it->second < nodes.size() && nodes[it->second].net_id == id) {
            nodes[it->second].predictor = predictor;
            return nodes[it->second];
        }
        index_[id] = nodes.size();
        nodes.emplace_back();
        nodes.back().net_id = id;
        nodes.back().predictor = predictor;
        return nodes.back();
    }
    std::unordered_map<uint64_t, size_t> index_;
    void record(uint64_t id, const std::string& predictor, double predicted, double actual, double reltol) {
        get(id, predictor).record(predicted, actual, reltol);
    }
    double overall_hit_rate() const {
        uint64_t t = 0, h = 0;
        for (auto& n : nodes) { t += n.total; h += n.hits; }
        return t ? double(h) / double(t) : 1.0;
    }
    std::string summary() const {
        char buf[160];
        std::snprintf(buf, sizeof buf, "prediction accuracy: %zu nodes, overall hit rate %.1f%%", nodes.size(), overall_hit_rate() * 100.0);
        return buf;
    }
};

// Per-node confidence (rises slowly on hits, drops fast on misses); the least confident node scales
// the speculative depth between 0.5x and 2x of the base, clamped to [1, 3 * base].
struct AdaptiveConfidence {
    uint32_t base_depth, min_depth = 1, max_depth;
    std::vector<std::pair<uint64_t, double>> conf;
    explicit AdaptiveConfidence(uint32_t base = 5) : base_depth(base), max_depth(base * 3) {}
    void update(uint64_t id, bool accurate) {
        auto it = index_.find(id);
        if (it != index_.end() && it->second < conf.size() && conf[it->second].first == id) {
            auto& c = conf[it->second];
            c.second = accurate ? c.second * 0.9 + 0.1 : c.second * 0.7;
            c.second = std::min(1.0, std::max(0.0, c.second));
            return;
        }
        index_[id] = conf.size();
        conf.emplace_back(id, accurate ? 0.5 : 0.1);
    }
    std::unordered_map<uint64_t, size_t> index_;
    uint32_t effective_depth() const {
        if (conf.empty()) return base_depth;
        double mn = 1.0;
        for (auto& c : conf) mn = std::min(mn, c.second);
        uint32_t d = uint32_t(double(base_depth) * (0.5 + 1.5 * mn));
        return std::min(max_depth, std::max(min_depth, d));
    }
    double confidence_for(uint64_t id) const {
        for (auto& c : conf) if (c.first == id) return c.second;
        return 0.5;
    }
};

struct GhostNode {
    uint64_t net_id = 0;
    uint32_t owner = 0;
    double last_known_voltage = 0, gradient = 0, confidence = 0, last_update_time = 0;
    SignalState signal;
    std::string active_predictor = "Linear";
    GhostNode() = default;
    GhostNode(uint64_t id, uint32_t owner_) : net_id(id), owner(owner_) {}

    Prediction predict_named(double t) const {
        if (signal.history.size() >= 4) return select_and_predict(signal, t);
        return {last_known_voltage + gradient * (t - last_update_time), "Linear"};
    }
    double predict(double t) const { return predict_named(t).value; }
    // Records the true value; returns whether the prediction for that time was within reltol.
    bool apply_correction(double v, double t, double reltol) {
        double err = std::fabs(v - predict(t));
        double dt = t - last_update_time;
        if (dt > 0.0) gradient = (v - last_known_voltage) / dt;
        last_known_voltage = v;
        last_update_time = t;
        signal.record(t, v);
        double rel = std::fabs(v) > 1e-15 ? err / std::fabs(v) : err;
        confidence = std::min(1.0, std::max(0.0, 1.0 - rel));
        return rel < reltol;
    }
    // The value recorded for the newest time point is replaced by `v`; no prediction is scored.
    void amend(double v) {
        if (signal.history.size() >= 2) {
            const auto& prev = signal.history[signal.history.size() - 2];
            const double dt = last_update_time - prev.first;
            if (dt > 0.0) gradient = (v - prev.second) / dt;
        }
        last_known_voltage = v;
        amend_newest(signal, v);
    }
};

struct Correction { uint64_t net_id; double voltage; double time; };

class GhostBuffer {
public:
    std::vector<GhostNode> nodes;
    AccuracyLogger accuracy;
    AdaptiveConfidence adaptive;
    explicit GhostBuffer(uint32_t base_depth = 5) : adaptive(base_depth) {}
    void add(GhostNode n) { index_.emplace(n.net_id, nodes.size()); nodes.push_back(std::move(n)); }
    // Position of a net in `nodes`, or size() when the buffer does not hold it.
    size_t index_of(uint64_t net_id) const {
        if (index_.size() != nodes.size()) rebuild_index();  // `nodes` is public; tolerate direct pushes
        auto it = index_.find(net_id);
        return it == index_.end() ? nodes.size() : it->second;
    }
    size_t size() const { return nodes.size(); }
    std::vector<std::pair<uint64_t, double>> predict_all(double t) const {
        std::vector<std::pair<uint64_t, double>> out;
        for (auto& g : nodes) out.emplace_back(g.net_id, g.predict(t));
        return out;
    }
    bool apply_corrections(const std::vector<Correction>& cs, double reltol) {
        bool all_ok = true;
        for (auto& c : cs) {
            const size_t i = index_of(c.net_id);
            if (i >= nodes.size()) continue;
            GhostNode& g = nodes[i];
            Prediction p = g.predict_named(c.time);
            bool ok = g.apply_correction(c.voltage, c.time, reltol);
            g.active_predictor = p.predictor;
            accuracy.record(c.net_id, p.predictor, p.value, c.voltage, reltol);
            adaptive.update(c.net_id, ok);
            all_ok = all_ok && ok;
        }
        return all_ok;
    }
    uint32_t effective_depth() const { return adaptive.effective_depth(); }

private:
    mutable std::unordered_map<uint64_t, size_t> index_;
    void rebuild_index() const {
        index_.clear();
        for (size_t i = 0; i < nodes.size(); ++i) index_.emplace(nodes[i].net_id, i);
    }
};

}  // namespace nspice
