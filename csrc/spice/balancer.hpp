// Load balancing across partitions (per-partition timing, straggler detection, migration plans) and
// the synthetic benchmark circuits with their harness.
// Behavioural reference: nangila-spice/nangila-node/src/balancer.rs:21-422, benchmark.rs:24-315.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <deque>
#include <string>
#include <vector>

#include "transient.hpp"

namespace nspice {

struct PartitionMetrics {
    uint32_t partition_id = 0, element_count = 0, ghost_count = 0;
    uint64_t steps_completed = 0, rollback_count = 0;
    std::deque<double> solve_times;  // last 64
    double ewma = 0.0, alpha = 0.1;
    PartitionMetrics() = default;
    PartitionMetrics(uint32_t id, uint32_t elements, uint32_t ghosts) : partition_id(id), element_count(elements), ghost_count(ghosts) {}
    void record_solve_time(double s) {
        solve_times.push_back(s);
        if (solve_times.size() > 64) solve_times.pop_front();
        ewma = ewma == 0.0 ? s : alpha * s + (1.0 - alpha) * ewma;
        ++steps_completed;
    }
    double avg_solve_time() const { return ewma; }
    double solve_time_variance() const {
        if (solve_times.size() < 2) return 0.0;
        double mean = 0.0, var = 0.0;
        for (double t : solve_times) mean += t;
        mean /= double(solve_times.size());
        for (double t : solve_times) var += (t - mean) * (t - mean);
        return var / double(solve_times.size() - 1);
    }
    double throughput() const { return ewma > 0.0 ? double(element_count) / ewma : 0.0; }
};

struct StragglerConfig { double threshold_sigma = 1.5, min_ratio = 1.3; size_t min_samples = 10; };
struct Straggler { uint32_t partition; double ratio; };

// A partition is a straggler when its smoothed step time is above mean + sigma * stddev of all
// partitions and at least min_ratio times the fastest.
inline std::vector<Straggler> detect_stragglers(const std::vector<PartitionMetrics>& m, const StragglerConfig& cfg = {}) {
    std::vector<Straggler> out;
    if (m.size() < 2) return out;
    uint64_t min_steps = UINT64_MAX;
    for (auto& p : m) min_steps = std::min(min_steps, p.steps_completed);
    if (min_steps < cfg.min_samples) return out;
    double mean = 0.0, var = 0.0, fastest = 1e300;
    for (auto& p : m) { mean += p.avg_solve_time(); fastest = std::min(fastest, p.avg_solve_time()); }
    mean /= double(m.size());
    for (auto& p : m) var += (p.avg_solve_time() - mean) * (p.avg_solve_time() - mean);
    double threshold = mean + cfg.threshold_sigma * std::sqrt(var / double(m.size()));
    for (auto& p : m) {
        double t = p.avg_solve_time(), ratio = fastest > 0.0 ? t / fastest : 1.0;
        if (t > threshold && ratio > cfg.min_ratio) out.push_back({p.partition_id, ratio});
    }
    return out;
}

struct MigrationPlan { uint32_t from_partition, to_partition, elements_to_move; double expected_speedup; };

class WorkStealer {
public:
    double max_steal_fraction = 0.25, min_improvement = 1.1;
    struct Stats { uint64_t migrations_planned = 0, elements_migrated = 0; double total_speedup_estimate = 0; } stats;
    // Moves a share of a straggler's elements to the partition with the highest throughput.
    std::vector<MigrationPlan> plan(const std::vector<PartitionMetrics>& m, const std::vector<Straggler>& stragglers) {
        std::vector<MigrationPlan> plans;
        if (stragglers.empty() || m.size() < 2) return plans;
        double mean_tp = 0.0;
        for (auto& p : m) mean_tp += p.throughput();
        mean_tp /= double(m.size());
        const PartitionMetrics* target = nullptr;
        for (auto& p : m)
            if (p.throughput() > 1.1 * mean_tp && (!target || p.throughput() > target->throughput())) target = &p;
        if (!target) return plans;
        for (auto& s : stragglers) {
            const PartitionMetrics* src = nullptr;
            for (auto& p : m) if (p.partition_id == s.partition) src = &p;
            if (!src || src == target) continue;
            uint32_t move = uint32_t(double(src->element_count) * max_steal_fraction * (1.0 - 1.0 / s.ratio));
            double speedup = std::sqrt(s.ratio);
            if (move == 0 || speedup < min_improvement) continue;
            plans.push_back({s.partition, target->partition_id, move, speedup});
            ++stats.migrations_planned;
            stats.elements_migrated += move;
            stats.total_speedup_estimate += speedup;
        }
        return plans;
    }
};

class BalanceMonitor {
public:
    std::vector<PartitionMetrics> metrics;
    StragglerConfig detector;
    WorkStealer stealer;
    uint64_t check_interval = 50;
    std::vector<double> balance_history;
    explicit BalanceMonitor(uint32_t partitions) { for (uint32_t i = 0; i < partitions; ++i) metrics.emplace_back(i, 0, 0); }
    void set_partition_info(uint32_t id, uint32_t elements, uint32_t ghosts) {
        for (auto& m : metrics) if (m.partition_id == id) { m.element_count = elements; m.ghost_count = ghosts; }
    }
    void record(uint32_t id, double solve_time) {
        for (auto& m : metrics) if (m.partition_id == id) m.record_solve_time(solve_time);
        ++steps_;
    }
    std::vector<MigrationPlan> check_balance() {
        if (steps_ % check_interval != 0) return {};
        balance_history.push_back(balance_score());
        auto s = detect_stragglers(metrics, detector);
        if (s.empty()) return {};
        return stealer.plan(metrics, s);
    }
    // 0 = all partitions equally fast, towards 1 = one partition dominates
    double balance_score() const {
        double mx = -1e300, mn = 1e300;
        for (auto& m : metrics) { mx = std::max(mx, m.avg_solve_time()); mn = std::min(mn, m.avg_solve_time()); }
        return (metrics.empty() || mx <= 0.0) ? 0.0 : (mx - mn) / mx;
    }
    std::string summary() const {
        char buf[200];
        std::snprintf(buf, sizeof buf, "load balance: %zu partitions, %llu steps, score %.3f, %llu migrations planned", metrics.size(),
                      (unsigned long long)steps_, balance_score(), (unsigned long long)stealer.stats.migrations_planned);
        return buf;
    }
    uint64_t steps() const { return steps_; }
private:
    uint64_t steps_ = 0;
};

// ---- synthetic circuits ----------------------------------------------------------------------------

// Compute-in-memory crossbar: row drivers (row 0 at 1.8 V), a resistor per cell (1 MOhm where
// (row + col) % 3 == 0, else 10 kOhm), 100 fF on every bit line.
inline Netlist generate_cim_array(int rows, int cols) {
    Netlist n;
    n.name = "cim_" + std::to_string(rows) + "x" + std::to_string(cols);
    n.num_nodes = rows + cols;
    for (int r = 0; r < rows; ++r) n.elements.push_back(Element::vsource(r + 1, 0, SourceWaveform::make_dc(r == 0 ? 1.8 : 0.0)));
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) n.elements.push_back(Element::resistor(r + 1, rows + c + 1, (r + c) % 3 == 0 ? 1e6 : 10e3));
    for (int c = 0; c < cols; ++c) n.elements.push_back(Element::capacitor(rows + c + 1, 0, 100e-15));
    for (int r = 0; r < rows; ++r) n.node_names.push_back("wl" + std::to_string(r));
    for (int c = 0; c < cols; ++c) n.node_names.push_back("bl" + std::to_string(c));
    return n;
}
inline Netlist generate_rc_ladder(int stages, double r, double c) {
    Netlist n;
    n.name = "rc_ladder_" + std::to_string(stages);
    n.num_nodes = stages + 1;
    n.elements.push_back(Element::vsource(1, 0, SourceWaveform::make_dc(1.8)));
    for (int i = 0; i < stages; ++i) {
        n.elements.push_back(Element::resistor(i + 1, i + 2, r));
        n.elements.push_back(Element::capacitor(i + 2, 0, c));
    }
    return n;
}
// n x n grid of equal resistors, 1.8 V at one corner, 1 mA drawn from the opposite one.
inline Netlist generate_resistor_mesh(int n_side, double r) {
    Netlist n;
    n.name = "mesh_" + std::to_string(n_side);
    n.num_nodes = n_side * n_side;
    auto node = [&](int row, int col) { return row * n_side + col + 1; };
    n.elements.push_back(Element::vsource(node(0, 0), 0, SourceWaveform::make_dc(1.8)));
    n.elements.push_back(Element::isource(node(n_side - 1, n_side - 1), 0, SourceWaveform::make_dc(1e-3)));
    for (int row = 0; row < n_side; ++row)
        for (int col = 0; col + 1 < n_side; ++col) n.elements.push_back(Element::resistor(node(row, col), node(row, col + 1), r));
    for (int row = 0; row + 1 < n_side; ++row)
        for (int col = 0; col < n_side; ++col) n.elements.push_back(Element::resistor(node(row, col), node(row + 1, col), r));
    return n;
}

struct BenchmarkResult {
    std::string name;
    int num_nodes = 0;
    size_t num_elements = 0;
    uint64_t steps = 0, nr_iterations = 0;
    double wall_time_secs = 0, steps_per_sec = 0;
    bool completed = false;
    std::string summary() const {
        char buf[240];
        std::snprintf(buf, sizeof buf, "%-20s %7d nodes %8zu elements %7llu steps %9.3f s %10.0f steps/s%s", name.c_str(), num_nodes, num_elements,
                      (unsigned long long)steps, wall_time_secs, steps_per_sec, completed ? "" : "  (did not finish)");
        return buf;
    }
};

inline BenchmarkResult run_benchmark(Netlist nl, SimConfig cfg, LinearBackend backend = LinearBackend::SparseLU) {
    BenchmarkResult r;
    r.name = nl.name;
    r.num_nodes = nl.num_nodes;
    r.num_elements = nl.elements.size();
    TransientSolver s(std::move(nl), GhostBuffer(cfg.predict_depth), CommLayer(0, 1), cfg);
    s.engine().newton.linear.backend = backend;
    s.run();
    r.steps = s.stats.total_steps;
    r.wall_time_secs = s.stats.wall_time_secs;
    r.steps_per_sec = r.wall_time_secs > 0 ? double(r.steps) / r.wall_time_secs : 0.0;
    r.nr_iterations = s.engine().newton.stats.total_iterations;
    r.completed = s.stats.completed;
    return r;
}

inline std::vector<BenchmarkResult> run_benchmark_suite(int scale = 1) {
    SimConfig cfg;
    cfg.tstop = 100e-12; cfg.dt = 1e-12; cfg.record_every = 1000;
    std::vector<BenchmarkResult> out;
    out.push_back(run_benchmark(generate_rc_ladder(100 * scale, 1e3, 10e-15), cfg));
    out.push_back(run_benchmark(generate_rc_ladder(1000 * scale, 1e3, 10e-15), cfg));
    out.push_back(run_benchmark(generate_cim_array(16 * scale, 16 * scale), cfg));
    out.push_back(run_benchmark(generate_resistor_mesh(20 * scale, 1e3), cfg));
    return out;
}

}  // namespace nspice
