// Transient loop of one partition: apply incoming residual corrections, honour rollback requests,
// predict the ghost nodes one step ahead, solve, record the waveform and keep a bounded history of
// checkpoints. Behavioural reference: nangila-spice/nangila-node/src/solver.rs:14-245.
#pragma once
#include <chrono>
#include <deque>
#include <functional>
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
};

struct SimStats {
    uint64_t total_steps = 0, prediction_hits = 0, prediction_misses = 0, rollbacks = 0;
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
        auto t0 = std::chrono::steady_clock::now();
        PartitionState state = engine_->initial_state();
        waveform.clear();
        waveform.push_back({state.time, state.voltages});
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
            if (step % config.record_every == 0 || step == planned) waveform.push_back({next.time, next.voltages});
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
