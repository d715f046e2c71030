// Transient loop of one partition: apply incoming residual corrections, honour rollback requests,
// predict the ghost nodes one step ahead, solve, record the waveform and keep a bounded history of
// checkpoints. Behavioural reference: nangila-spice/nangila-node/src/solver.rs:14-245.
#pragma once
#include <chrono>
#include <deque>
#include <functional>
#include <limits>
#include <memory>

#include "comm.hpp"
#include "engine.hpp"
#include "ghost.hpp"

namespace nspice {

struct SimConfig {
    double tstop = 1e-6, dt = 1e-12, reltol = 1e-3;
    uint32_t predict_depth = 5;
    size_t max_history = 100;
    // Optional cap on stored waveform points: keep every k-th step (1 = all).
    uint32_t record_every = 1;
    // Variable internal step (single-partition runs): the waveform is still written on the dt grid, but the solver
    // takes the steps the signals allow, between dt / 64 and max_step_factor * dt, lands on the corners of the sources,
    // and bounds how far a solution may depart from the straight line through the two before it (lte_reltol of the
    // larger of the values involved plus lte_abstol volts). That departure is far larger than the error of the
    // trapezoidal step itself: at 2 % the observed outputs of the logic cases stay within 3 mV of a run at a quarter of dt.
    bool adaptive = false;
    double lte_reltol = 2e-2, lte_abstol = 1e-4, max_step_factor = 64.0;
    // Unknowns (0-based) whose values the waveform keeps, in this order; empty = all of them. A deck of 100 000 nets
    // over thousands of steps is gigabytes of waveform of which a comparison reads a handful of columns.
    std::vector<uint32_t> record_nodes;
};

struct SimStats {
    uint64_t total_steps = 0, prediction_hits = 0, prediction_misses = 0, rollbacks = 0;
    uint64_t solver_steps = 0, rejected_steps = 0;  // adaptive mode: internal steps accepted / thrown away
    double wall_time_secs = 0.0;
    bool completed = false;
    double hit_rate() const {
        uint64_t t = prediction_hits + prediction_misses;
        return t ? double(prediction_hits) / double(t) : 1.0;
    }
};

struct WaveformPoint { double time; std::vector<double> values; };

class TransientSolver {
public:
    std::vector<WaveformPoint> waveform;
    SimStats stats;
    GhostBuffer ghosts;
    CommLayer comm;
    SimConfig config;

    TransientSolver(Netlist nl, GhostBuffer g, CommLayer c, SimConfig cfg)
        : ghosts(std::move(g)), comm(std::move(c)), config(cfg), engine_(new SolverEngine(std::move(nl))) {}

    SolverEngine& engine() { return *engine_; }

    // Hook called after every accepted step (time, solution); used by the partitioned runner to
    // publish boundary voltages.
    std::function<void(const PartitionState&)> on_step;

    PartitionState run() {
        if (config.adaptive && ghosts.size() == 0) return run_adaptive();
        auto t0 = std::chrono::steady_clock::now();
        PartitionState state = engine_->initial_state();
        waveform.clear();
        waveform.push_back({state.time, recorded(state.voltages)});
        history_.clear();
        uint64_t step = 0;
        // the loop counts steps instead of comparing accumulated floating-point time with tstop, so
        // tstop / dt steps are taken exactly
        const uint64_t planned = config.dt > 0 ? uint64_t(std::ceil(config.tstop / config.dt - 1e-9)) : 0;
        stats = SimStats{};
        while (step < planned) {
            for (auto& msg : comm.poll_residuals()) {
                std::vector<Correction> cs;
                for (auto& u : msg.updates) cs.push_back({u.first, u.second, msg.time});
                if (ghosts.apply_corrections(cs, config.reltol)) stats.prediction_hits += cs.size();
                else stats.prediction_misses += cs.size();
            }
            RollbackRequest rb;
            if (comm.poll_rollback(rb)) {
                PartitionState restored{0};
                if (rollback_to(rb.rollback_to_time, restored)) {
                    uint64_t back = uint64_t(std::llround((state.time - restored.time) / config.dt));
                    step = back <= step ? step - back : 0;
                    state = std::move(restored);
                    ++stats.rollbacks;
                    continue;
                }
            }
            auto predictions = ghosts.predict_all(state.time + config.dt);
            PartitionState next{0};
            if (!engine_->solve_step(state, predictions, config.dt, next)) break;
            ++step;
            next.time = double(step_origin_ + step) * config.dt;
            if (step % config.record_every == 0 || step == planned) waveform.push_back({next.time, recorded(next.voltages)});
            if (history_.size() >= config.max_history) history_.pop_front();
            history_.push_back(state);
            state = std::move(next);
            if (on_step) on_step(state);
        }
        stats.total_steps = step;
        stats.completed = step == planned;
        stats.wall_time_secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        return state;
    }

    // The columns of a solution the waveform keeps (config.record_nodes; all when that is empty).
    std::vector<double> recorded(const std::vector<double>& v) const {
        if (config.record_nodes.empty()) return v;
        std::vector<double> out(config.record_nodes.size(), 0.0);
        for (size_t k = 0; k < out.size(); ++k)
            if (config.record_nodes[k] < v.size()) out[k] = v[config.record_nodes[k]];
        return out;
    }

    // Variable-step form of run(): same waveform grid, the solver chooses its own steps in between.
    PartitionState run_adaptive() {
        auto t0 = std::chrono::steady_clock::now();
        PartitionState state = engine_->initial_state(), older{0};
        waveform.clear();
        waveform.push_back({state.time, recorded(state.voltages)});
        stats = SimStats{};
        const double dt = config.dt, tstop = config.tstop;
        const uint64_t planned = dt > 0 ? uint64_t(std::ceil(tstop / dt - 1e-9)) : 0;
        const double hmin = dt / 64.0, hmax = dt * config.max_step_factor;
        const int nodes = engine_->netlist.num_nodes;
        double t = 0.0, h = dt, h_older = 0.0;
        uint64_t emitted = 0;   // grid points written so far (beyond t = 0)
        bool have_older = false, failed = false;
        auto next_corner = [&](double now) {
            double c = std::numeric_limits<double>::infinity();
            for (auto& e : engine_->netlist.elements)
                if (e.kind == Element::VSource || e.kind == Element::ISource) c = std::min(c, e.source.next_corner_after(now));
            return c;
        };
        const std::vector<std::pair<uint64_t, double>> no_pins;
        while (emitted < planned && !failed) {
            const double t_end = double(planned) * dt;
            double step = std::min(h, t_end - t);
            const double corner = next_corner(t);
            bool lands_on_corner = false;
            if (t + step > corner - 1e-6 * dt) { step = corner - t; lands_on_corner = true; }
            if (step <= 0.0) step = hmin;
            PartitionState next{0};
            if (!engine_->solve_step(state, no_pins, step, next)) {
                if (step <= hmin * 1.0001) { failed = true; break; }
                h = std::max(hmin, 0.25 * step);
                ++stats.rejected_steps;
                continue;
            }
            double err = 0.0;
            if (have_older && h_older > 0.0) {
                const double ratio = step / h_older;
                for (int i = 0; i < nodes; ++i) {
                    const double now = state.voltages[size_t(i)], was = older.voltages[size_t(i)], got = next.voltages[size_t(i)];
                    const double line = now + (now - was) * ratio;
                    const double tol = config.lte_reltol * std::max({std::fabs(got), std::fabs(now), std::fabs(line)}) + config.lte_abstol;
                    err = std::max(err, std::fabs(got - line) / tol);
                }
                if (err > 1.0 && step > hmin * 1.0001) {
                    h = std::max(hmin, step * std::max(0.25, 0.9 / std::sqrt(err)));
                    ++stats.rejected_steps;
                    continue;
                }
            }
            // accepted: write the grid points this step covers (linear between its two ends)
            const double t_new = t + step;
            while (emitted < planned && double(emitted + 1) * dt <= t_new + 1e-9 * dt) {
                const double tg = double(emitted + 1) * dt, w = step > 0.0 ? std::min(1.0, std::max(0.0, (tg - t) / step)) : 1.0;
                ++emitted;
                if (emitted % config.record_every == 0 || emitted == planned) {
                    if (config.record_nodes.empty()) {
                        std::vector<double> v(next.voltages.size());
                        for (size_t i = 0; i < v.size(); ++i) v[i] = state.voltages[i] + w * (next.voltages[i] - state.voltages[i]);
                        waveform.push_back({tg, std::move(v)});
                    } else {
                        std::vector<double> v(config.record_nodes.size(), 0.0);
                        for (size_t k = 0; k < v.size(); ++k) {
                            const size_t i = config.record_nodes[k];
                            if (i < next.voltages.size()) v[k] = state.voltages[i] + w * (next.voltages[i] - state.voltages[i]);
                        }
                        waveform.push_back({tg, std::move(v)});
                    }
                }
            }
            ++stats.solver_steps;
            older = std::move(state);
            h_older = step;
            have_older = !lands_on_corner;   // the slope of a source changes at a corner: the straight line through it says nothing
            state = std::move(next);
            state.time = t_new;
            t = t_new;
            if (on_step) on_step(state);
            const double grow = have_older ? std::min(2.0, 0.9 / std::sqrt(std::max(err, 0.05))) : 1.0;
            h = lands_on_corner ? std::min(dt, step) : std::min(hmax, std::max(hmin, step * std::max(grow, 0.5)));
        }
        stats.total_steps = emitted;
        stats.completed = !failed && emitted == planned;
        stats.wall_time_secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        return state;
    }

private:
    std::unique_ptr<SolverEngine> engine_;
    std::deque<PartitionState> history_;
    uint64_t step_origin_ = 0;

    // Newest checkpoint at or before `t`; later checkpoints and waveform points are discarded.
    bool rollback_to(double t, PartitionState& out) {
        const double eps = 0.5 * config.dt;
        while (!history_.empty()) {
            if (history_.back().time <= t + eps * 1e-6) {
                out = history_.back();
                history_.pop_back();
                while (!waveform.empty() && waveform.back().time > out.time + eps * 1e-6) waveform.pop_back();
                return true;
            }
            history_.pop_back();
        }
        return false;
    }
};

}  // namespace nspice
