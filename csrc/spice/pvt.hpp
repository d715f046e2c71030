// Process / voltage / temperature sweeps: corner descriptions, the golden-trajectory cache with its
// binary form, and the delta solver that derives a nearby corner's waveform from the golden one.
// Behavioural reference: nangila-spice/nangila-node/src/pvt.rs:26-507. Unlike the reference, a corner
// that is too far from the golden one is really re-simulated when a simulation callback is given
// (the reference returns the golden waveform unchanged as a placeholder).
#pragma once
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <list>
#include <string>
#include <vector>

namespace nspice {

enum class ProcessCorner { TT, FF, SS, FS, SF };

inline double mobility_factor(ProcessCorner p) {
    switch (p) {
        case ProcessCorner::FF: return 1.15;
        case ProcessCorner::SS: return 0.85;
        case ProcessCorner::FS: return 1.1;
        case ProcessCorner::SF: return 0.9;
        default: return 1.0;
    }
}
inline const char* corner_name(ProcessCorner p) {
    switch (p) {
        case ProcessCorner::FF: return "FF";
        case ProcessCorner::SS: return "SS";
        case ProcessCorner::FS: return "FS";
        case ProcessCorner::SF: return "SF";
        default: return "TT";
    }
}
inline ProcessCorner corner_from_name(const std::string& s) {
    if (s == "FF" || s == "ff") return ProcessCorner::FF;
    if (s == "SS" || s == "ss") return ProcessCorner::SS;
    if (s == "FS" || s == "fs") return ProcessCorner::FS;
    if (s == "SF" || s == "sf") return ProcessCorner::SF;
    return ProcessCorner::TT;
}

struct CornerDelta {
    double delta_vdd = 0, delta_temp = 0, mobility = 1;
    // small enough for the first-order correction: < 0.3 V, < 50 C, < 20 % mobility
    bool linearisable() const { return std::fabs(delta_vdd) < 0.3 && std::fabs(delta_temp) < 50.0 && std::fabs(mobility - 1.0) < 0.2; }
};

struct CornerSpec {
    ProcessCorner process = ProcessCorner::TT;
    double vdd = 1.8, temperature = 27.0;
    std::string name = "TT_1V8_27C";
    CornerSpec() = default;
    CornerSpec(ProcessCorner p, double v, double t) : process(p), vdd(v), temperature(t) {
        char buf[64];
        std::snprintf(buf, sizeof buf, "%s_%gV_%.0fC", corner_name(p), v, t);
        name = buf;
    }
    bool is_nominal() const { return process == ProcessCorner::TT && std::fabs(vdd - 1.8) < 0.01 && std::fabs(temperature - 27.0) < 0.1; }
    double thermal_voltage() const { return 8.617e-5 * (temperature + 273.15); }
    CornerDelta delta(const CornerSpec& ref) const {
        return {vdd - ref.vdd, temperature - ref.temperature, mobility_factor(process) / mobility_factor(ref.process)};
    }
};

struct PvtPoint { double time; std::vector<double> voltages; };

struct GoldenTrajectory {
    CornerSpec corner;
    double dt = 0;
    std::vector<PvtPoint> points;
    GoldenTrajectory() = default;
    GoldenTrajectory(CornerSpec c, double dt_) : corner(std::move(c)), dt(dt_) {}
    void push(double t, std::vector<double> v) { points.push_back({t, std::move(v)}); }
    size_t size() const { return points.size(); }
    // Linear interpolation between the stored points; false outside the stored span.
    bool voltage_at(size_t node, double t, double& out) const {
        if (points.empty() || t < points.front().time || t > points.back().time) return false;
        size_t lo = 0, hi = points.size() - 1;
        while (hi - lo > 1) { size_t mid = (lo + hi) / 2; (points[mid].time <= t ? lo : hi) = mid; }
        if (node >= points[lo].voltages.size()) return false;
        double t0 = points[lo].time, t1 = points[hi].time, v0 = points[lo].voltages[node], v1 = points[hi].voltages[node];
        out = (t1 > t0) ? v0 + (v1 - v0) * (t - t0) / (t1 - t0) : v0;
        return true;
    }
    // "NZGT", u32 points, u32 nodes, f64 dt, then per point f64 time + f64 voltages[nodes]
    std::string to_bytes() const {
        std::string b("NZGT");
        auto put = [&](const void* p, size_t n) { b.append(static_cast<const char*>(p), n); };
        uint32_t np = uint32_t(points.size()), nn = points.empty() ? 0 : uint32_t(points[0].voltages.size());
        put(&np, 4); put(&nn, 4); put(&dt, 8);
        for (auto& p : points) {
            put(&p.time, 8);
            for (uint32_t i = 0; i < nn; ++i) { double v = i < p.voltages.size() ? p.voltages[i] : 0.0; put(&v, 8); }
        }
        return b;
    }
    static bool from_bytes(const std::string& b, const CornerSpec& corner, GoldenTrajectory& out) {
        if (b.size() < 20 || b.compare(0, 4, "NZGT") != 0) return false;
        uint32_t np, nn;
        double dt;
        std::memcpy(&np, b.data() + 4, 4); std::memcpy(&nn, b.data() + 8, 4); std::memcpy(&dt, b.data() + 12, 8);
        if (b.size() != 20 + uint64_t(np) * (8 + 8 * uint64_t(nn))) return false;
        out = GoldenTrajectory(corner, dt);
        size_t pos = 20;
        for (uint32_t p = 0; p < np; ++p) {
            PvtPoint pt;
            std::memcpy(&pt.time, b.data() + pos, 8); pos += 8;
            pt.voltages.resize(nn);
            std::memcpy(pt.voltages.data(), b.data() + pos, 8 * size_t(nn)); pos += 8 * size_t(nn);
            out.points.push_back(std::move(pt));
        }
        return true;
    }
};

// Least-recently-used cache of golden trajectories keyed by corner name.
class PvtCache {
public:
    struct Stats { uint64_t hits = 0, misses = 0, evictions = 0; };
    Stats stats;
    explicit PvtCache(size_t max_size) : max_(max_size ? max_size : 1) {}
    void insert(GoldenTrajectory t) {
        for (auto it = items_.begin(); it != items_.end(); ++it) if (it->corner.name == t.corner.name) { items_.erase(it); break; }
        if (items_.size() >= max_) { items_.pop_back(); ++stats.evictions; }
        items_.push_front(std::move(t));
    }
    const GoldenTrajectory* get(const std::string& name) {
        for (auto it = items_.begin(); it != items_.end(); ++it)
            if (it->corner.name == name) { items_.splice(items_.begin(), items_, it); ++stats.hits; return &items_.front(); }
        ++stats.misses;
        return nullptr;
    }
    bool contains(const std::string& name) const { for (auto& t : items_) if (t.corner.name == name) return true; return false; }
    size_t size() const { return items_.size(); }
private:
    size_t max_;
    std::list<GoldenTrajectory> items_;
};

struct DeltaSolveResult {
    CornerSpec corner;
    std::vector<PvtPoint> delta_waveform;  // corner minus golden, same time axis
    double peak_delta_v = 0, wall_time_secs = 0;
    bool used_delta_mode = false, resimulated = false;
};

class DeltaSolver {
public:
    struct Stats { uint64_t corners_solved = 0, delta_mode_used = 0, full_sim_fallback = 0; double total_wall_time = 0, speedup_estimate = 0; };
    GoldenTrajectory golden;
    Stats stats;
    // Optional full simulation for corners outside the linear range: returns the corner's points on
    // the golden time axis.
    std::function<std::vector<PvtPoint>(const CornerSpec&)> full_simulation;

    explicit DeltaSolver(GoldenTrajectory g) : golden(std::move(g)) {}

    // First-order model: node voltages follow the supply ratio times sqrt(mobility ratio), plus
    // -0.5 mV per degree.
    DeltaSolveResult solve_corner(const CornerSpec& corner) {
        auto t0 = std::chrono::steady_clock::now();
        ++stats.corners_solved;
        CornerDelta d = corner.delta(golden.corner);
        DeltaSolveResult res;
        res.corner = corner;
        res.used_delta_mode = d.linearisable();
        std::vector<PvtPoint> full;
        if (res.used_delta_mode) ++stats.delta_mode_used;
        else {
            ++stats.full_sim_fallback;
            if (full_simulation) { full = full_simulation(corner); res.resimulated = full.size() == golden.points.size(); }
        }
        const double scale = corner.vdd / golden.corner.vdd * std::sqrt(d.mobility), offset = -0.5e-3 * d.delta_temp;
        for (size_t k = 0; k < golden.points.size(); ++k) {
            const PvtPoint& g = golden.points[k];
            PvtPoint p{g.time, std::vector<double>(g.voltages.size(), 0.0)};
            for (size_t i = 0; i < g.voltages.size(); ++i) {
                double vc = g.voltages[i];
                if (res.used_delta_mode) vc = g.voltages[i] * scale + offset;
                else if (res.resimulated && i < full[k].voltages.size()) vc = full[k].voltages[i];
                p.voltages[i] = vc - g.voltages[i];
                res.peak_delta_v = std::max(res.peak_delta_v, std::fabs(p.voltages[i]));
            }
            res.delta_waveform.push_back(std::move(p));
        }
        res.wall_time_secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        stats.total_wall_time += res.wall_time_secs;
        return res;
    }
    std::vector<PvtPoint> reconstruct(const DeltaSolveResult& d) const {
        std::vector<PvtPoint> out;
        for (size_t k = 0; k < golden.points.size() && k < d.delta_waveform.size(); ++k) {
            PvtPoint p{golden.points[k].time, golden.points[k].voltages};
            for (size_t i = 0; i < p.voltages.size() && i < d.delta_waveform[k].voltages.size(); ++i) p.voltages[i] += d.delta_waveform[k].voltages[i];
            out.push_back(std::move(p));
        }
        return out;
    }
    void update_speedup(double full_sim_time_per_corner) {
        if (stats.corners_solved && stats.total_wall_time > 0)
            stats.speedup_estimate = full_sim_time_per_corner / (stats.total_wall_time / double(stats.corners_solved));
    }
};

}  // namespace nspice
