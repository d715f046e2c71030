// One partition of a partitioned transient run as its own process; the partitions advance in lockstep over a
// SocketMesh (netfabric.hpp). The algorithm is the one of partitioned.hpp (speculative solve with predicted ghost
// voltages, exchange of the boundary voltages, block relaxation of the steps whose predictions missed), with the
// shared-memory reads replaced by messages:
//
//   set-up    every process tells every owner which of its nets it wants; from then on a values message is just the
//             time and the voltages in the order they were asked for (8 bytes per net, no identifiers)
//   window    every process runs several steps ahead on predictions, then one exchange carries the boundary voltages of
//             the whole window and one all-gathered tally says up to which step every prediction everywhere hit:
//             those steps are final, the first missed one is relaxed, the rest is discarded
//   values    one exchange per relaxation sweep between the pairs of processes that share a boundary
//   tally   one all-gather per window and per sweep (first miss, steps ready, sweep converged, failed, largest
//             change), so that all processes take the same decision
//
// The DC point is relaxed the same way (every process solves its operating point against the neighbours' last
// values, Jacobi fashion, until nothing moves). A process that fails, or whose peer went away or stays silent past
// the I/O deadline, stops with an error; the others learn of it through the tally or through their own deadline.
#pragma once
#include <map>
#include <memory>
#include <set>
#include <unordered_map>

#include "comm.hpp"
#include "engine.hpp"
#include "ghost.hpp"
#include "netfabric.hpp"
#include "parser.hpp"
#include "transient.hpp"

namespace nspice {

struct DistributedConfig {
    double tstop = 1e-9, dt = 1e-12, reltol = 1e-3, abstol = 1e-6;
    double accept_factor = 0.25;  // a prediction is a hit within accept_factor * reltol (see PartitionedConfig)
    uint32_t predict_depth = 5, record_every = 1;
    bool speculate = true;  // windows of steps between exchanges (false: one step per exchange)
    int max_sweeps = 50, max_dc_sweeps = 400, io_timeout_ms = 30000;
};

struct DistributedStats {
    uint64_t steps = 0, prediction_hits = 0, prediction_misses = 0, resolves = 0, unconverged_steps = 0, dc_sweeps = 0;
    uint64_t windows = 0, speculated_steps = 0, discarded_steps = 0, rollbacks = 0;
    double wall_time_secs = 0.0;
    bool completed = false;
    std::string error;
};

class DistributedRunner {
public:
    DistributedStats stats;
    std::vector<std::string> names;        // nets this partition owns
    std::vector<WaveformPoint> waveform;   // values in `names` order

    DistributedRunner(Netlist part, SocketMesh& mesh, DistributedConfig cfg)
        : cfg_(cfg), mesh_(mesh), ghosts_(cfg.predict_depth), depth_(cfg.predict_depth, 1, cfg.predict_depth * 3) {
        all_names_ = part.names_or_default();
        for (auto& g : part.ghost_map) {
            ghost_index_.emplace(g.net_id, ghosts_.size());
            ghosts_.add(GhostNode(g.net_id, g.owner));
            ghost_nodes_.insert(g.local_node);
            ghost_owner_.push_back(g.owner);
        }
        has_ic_ = !part.initial_conditions.empty();
        engine_.reset(new SolverEngine(std::move(part)));
        for (size_t i = 0; i < all_names_.size(); ++i)
            if (!ghost_nodes_.count(int(i) + 1)) { owned_.push_back(i); names.push_back(all_names_[i]); }
    }

    SolverEngine& engine() { return *engine_; }

    bool run() {
        auto t0 = std::chrono::steady_clock::now();
        bool ok = setup() && relax_dc() && transient();
        stats.completed = ok;
        stats.wall_time_secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        return ok;
    }

private:
    struct Tally { uint8_t ok = 1, failed = 0; uint32_t first_miss = 0xFFFFFFFFu, ready = 0xFFFFFFFFu; double change = 0.0; };

    DistributedConfig cfg_;
    SocketMesh& mesh_;
    std::unique_ptr<SolverEngine> engine_;
    GhostBuffer ghosts_;
    std::set<int> ghost_nodes_;
    std::vector<uint32_t> ghost_owner_;
    std::unordered_map<uint64_t, size_t> ghost_index_;
    std::vector<std::string> all_names_;
    std::vector<size_t> owned_;
    bool has_ic_ = false;
    std::vector<uint32_t> partners_;                       // processes this one shares a boundary with, ascending
    std::map<uint32_t, std::vector<int>> exports_;         // consumer -> local nodes, in the order the consumer asked for
    std::map<uint32_t, std::vector<size_t>> imports_;      // owner -> positions in the ghost list, in the order asked for
    PartitionState state_{0}, next_{0};
    std::vector<std::pair<uint64_t, double>> pins_, latest_;  // in ghost-list order
    std::vector<std::vector<std::pair<uint64_t, double>>> window_latest_;  // per step of the window, same order
    SpeculativeDepthController depth_;

    bool fail(const std::string& what) { if (stats.error.empty()) stats.error = what; return false; }

    bool setup() {
        const uint32_t k = mesh_.total(), me = mesh_.id();
        for (size_t g = 0; g < ghost_owner_.size(); ++g) {
            if (ghost_owner_[g] >= k || ghost_owner_[g] == me) return fail("ghost net owned by process " + std::to_string(ghost_owner_[g]) + ", which is not a peer");
            imports_[ghost_owner_[g]].push_back(g);
        }
        std::vector<uint32_t> peers;
        std::vector<std::string> out, in;
        for (uint32_t p = 0; p < k; ++p) {
            if (p == me) continue;
            peers.push_back(p);
            std::string req;
            auto it = imports_.find(p);
            if (it != imports_.end())
                for (size_t g : it->second) { uint64_t id = ghosts_.nodes[g].net_id; req.append(reinterpret_cast<const char*>(&id), 8); }
            out.push_back(std::move(req));
        }
        if (!mesh_.exchange(peers, out, in, cfg_.io_timeout_ms)) return fail("set-up: " + mesh_.error);
        std::unordered_map<uint64_t, int> mine;
        for (size_t i : owned_) mine.emplace(net_name_hash(all_names_[i]), int(i) + 1);
        for (size_t i = 0; i < peers.size(); ++i) {
            if (in[i].size() % 8) return fail("set-up: malformed request from process " + std::to_string(peers[i]));
            std::vector<int> locals;
            for (size_t o = 0; o < in[i].size(); o += 8) {
                uint64_t id;
                std::memcpy(&id, in[i].data() + o, 8);
                auto f = mine.find(id);
                if (f == mine.end()) return fail("process " + std::to_string(peers[i]) + " asks for a net this partition does not own");
                locals.push_back(f->second);
            }
            if (!locals.empty()) exports_[peers[i]] = std::move(locals);
            if (exports_.count(peers[i]) || imports_.count(peers[i])) partners_.push_back(peers[i]);
        }
        pins_.clear();
        for (auto& g : ghosts_.nodes) pins_.emplace_back(g.net_id, 0.0);
        latest_ = pins_;
        return true;
    }

    // Sends the boundary voltages of `v` to the consumers and takes in the owners' values (into latest_).
    bool swap_boundaries(const std::vector<double>& v, double t) {
        std::vector<std::string> out, in;
        for (uint32_t p : partners_) {
            std::string msg(reinterpret_cast<const char*>(&t), 8);
            auto it = exports_.find(p);
            if (it != exports_.end())
                for (int node : it->second) msg.append(reinterpret_cast<const char*>(&v[size_t(node - 1)]), 8);
            out.push_back(std::move(msg));
        }
        if (!mesh_.exchange(partners_, out, in, cfg_.io_timeout_ms)) return fail("boundary exchange: " + mesh_.error);
        for (size_t i = 0; i < partners_.size(); ++i) {
            auto it = imports_.find(partners_[i]);
            const size_t want = it == imports_.end() ? 0 : it->second.size();
            if (in[i].size() != 8 + 8 * want) return fail("process " + std::to_string(partners_[i]) + " sent " + std::to_string(in[i].size()) + " bytes, expected " + std::to_string(8 + 8 * want));
            double theirs;
            std::memcpy(&theirs, in[i].data(), 8);
            if (std::fabs(theirs - t) > 1e-3 * cfg_.dt + 1e-30) return fail("process " + std::to_string(partners_[i]) + " is at another time point: out of step");
            for (size_t j = 0; j < want; ++j) std::memcpy(&latest_[it->second[j]].second, in[i].data() + 8 + 8 * j, 8);
        }
        return true;
    }

    // Everybody's tally on the sweep; the combined one is the same in every process.
    bool agree(Tally mine, Tally& all) {
        std::vector<std::string> got;
        std::string msg(reinterpret_cast<const char*>(&mine), sizeof mine);
        if (!mesh_.all_gather(msg, got, cfg_.io_timeout_ms)) return fail("tally: " + mesh_.error);
        all = Tally{};
        for (uint32_t p = 0; p < got.size(); ++p) {
            if (got[p].size() != sizeof(Tally)) return fail("malformed tally from process " + std::to_string(p));
            Tally v;
            std::memcpy(&v, got[p].data(), sizeof v);
            all.ok = all.ok && v.ok;
            all.failed = all.failed || v.failed;
            all.change = std::max(all.change, v.change);
            all.first_miss = std::min(all.first_miss, v.first_miss);
            all.ready = std::min(all.ready, v.ready);
            if (v.failed && stats.error.empty() && p != mesh_.id()) stats.error = "process " + std::to_string(p) + " reported a failed solve";
        }
        return true;
    }

    bool relax_dc() {
        state_ = engine_->seeded_state();
        next_ = state_;
        if (!swap_boundaries(next_.voltages, 0.0)) return false;
        for (int sweep = 0; sweep < cfg_.max_dc_sweeps; ++sweep) {
            Tally mine, all;
            if (!has_ic_) {
                PartitionState seed = next_, out{0};
                seed.cap_currents.clear();
                if (engine_->solve_dc(seed, out, latest_)) {
                    for (size_t i = 0; i < out.voltages.size(); ++i) mine.change = std::max(mine.change, std::fabs(out.voltages[i] - next_.voltages[i]));
                    next_.voltages = out.voltages;
                }
            }
            ++stats.dc_sweeps;
            if (!swap_boundaries(next_.voltages, 0.0) || !agree(mine, all)) return false;
            if (all.change < 1e-9) break;
        }
        state_.voltages = next_.voltages;
        state_.cap_currents.clear();
        state_.time = 0.0;
        for (size_t g = 0; g < ghosts_.nodes.size(); ++g) ghosts_.nodes[g].apply_correction(latest_[g].second, 0.0, cfg_.reltol);
        record(0.0);
        return true;
    }

    // Sends the boundary voltages of the first `mine` states of the window and takes in the partners' windows.
    // window_latest_[d] then holds the ghost voltages of step d (ghost-list order); returns in `usable` how many steps
    // every partner and this process have.
    bool swap_window(const std::vector<PartitionState>& states, double t_first, uint32_t& usable) {
        std::vector<std::string> out, in;
        const uint32_t mine = uint32_t(states.size());
        for (uint32_t p : partners_) {
            std::string msg(reinterpret_cast<const char*>(&mine), 4);
            msg.append(reinterpret_cast<const char*>(&t_first), 8);
            auto it = exports_.find(p);
            if (it != exports_.end())
                for (auto& st : states)
                    for (int node : it->second) msg.append(reinterpret_cast<const char*>(&st.voltages[size_t(node - 1)]), 8);
            out.push_back(std::move(msg));
        }
        if (!mesh_.exchange(partners_, out, in, cfg_.io_timeout_ms)) return fail("boundary exchange: " + mesh_.error);
        usable = mine;
        window_latest_.assign(mine, pins_);  // values a partner does not cover keep whatever was pinned last
        for (size_t i = 0; i < partners_.size(); ++i) {
            auto it = imports_.find(partners_[i]);
            const size_t want = it == imports_.end() ? 0 : it->second.size();
            uint32_t theirs = 0;
            double t_theirs = 0.0;
            if (in[i].size() < 12) return fail("process " + std::to_string(partners_[i]) + " sent a short window header");
            std::memcpy(&theirs, in[i].data(), 4);
            std::memcpy(&t_theirs, in[i].data() + 4, 8);
            if (in[i].size() != 12 + 8 * want * size_t(theirs)) return fail("process " + std::to_string(partners_[i]) + " sent a window of the wrong size");
            if (std::fabs(t_theirs - t_first) > 1e-3 * cfg_.dt + 1e-30) return fail("process " + std::to_string(partners_[i]) + " is at another time point: out of step");
            usable = std::min(usable, theirs);
            for (uint32_t d = 0; d < theirs && d < mine; ++d)
                for (size_t j = 0; j < want; ++j) std::memcpy(&window_latest_[d][it->second[j]].second, in[i].data() + 12 + 8 * (size_t(d) * want + j), 8);
        }
        return true;
    }

    // Whether every ghost voltage assumed for a step is within the acceptance bound of what its owner computed
    // (the rule of GhostNode::apply_correction, without touching the predictors).
    bool window_step_hits(const std::vector<std::pair<uint64_t, double>>& assumed, const std::vector<std::pair<uint64_t, double>>& actual) const {
        const double tol = cfg_.reltol * cfg_.accept_factor;
        for (size_t g = 0; g < assumed.size() && g < actual.size(); ++g) {
            const double v = actual[g].second, err = std::fabs(v - assumed[g].second);
            const double rel = std::fabs(v) > 1e-15 ? err / std::fabs(v) : err;
            if (!(rel < tol)) return false;
        }
        return true;
    }

    bool transient() {
        const uint64_t planned = cfg_.dt > 0 ? uint64_t(std::ceil(cfg_.tstop / cfg_.dt - 1e-9)) : 0;
        uint64_t step = 0;
        std::vector<PartitionState> ahead;
        std::vector<std::vector<std::pair<uint64_t, double>>> ahead_pins;
        while (step < planned) {
            // a window of steps on predicted ghost voltages, nobody spoken to. The depth controller is fed with the outcome
            // of the whole run (every process sees the same tallies), so all processes choose the same depth: a process
            // that ran further ahead than the others would only compute steps nobody can verify
            const uint64_t depth = std::min<uint64_t>(cfg_.speculate ? std::max<uint32_t>(1, depth_.depth()) : 1, planned - step);
            ahead.clear();
            ahead_pins.clear();
            const PartitionState* cur = &state_;
            for (uint64_t d = 0; d < depth; ++d) {
                ahead_pins.push_back(ghosts_.predict_all(double(step + d + 1) * cfg_.dt));
                PartitionState next{0};
                if (!engine_->solve_step(*cur, ahead_pins.back(), cfg_.dt, next)) { ahead_pins.pop_back(); break; }
                ahead.push_back(std::move(next));
                cur = &ahead.back();
            }
            Tally mine, all;
            mine.failed = ahead.empty() ? 1 : 0;
            if (ahead.empty()) { ahead.push_back(state_); ahead_pins.push_back(ghosts_.predict_all(double(step + 1) * cfg_.dt)); }  // well-formed; the tally stops everybody
            pins_ = ahead_pins[0];
            uint32_t usable = 0;
            if (!swap_window(ahead, double(step + 1) * cfg_.dt, usable)) return false;
            uint32_t first_miss = usable;
            for (uint32_t d = 0; d < usable; ++d)
                if (!window_step_hits(ahead_pins[d], window_latest_[d])) { first_miss = d; break; }
            mine.ready = usable;
            mine.first_miss = first_miss;
            if (!agree(mine, all)) return false;
            if (all.failed) return fail("Newton did not converge at t = " + std::to_string(double(step + 1) * cfg_.dt));
            const uint32_t ready = all.ready, miss = std::min(all.first_miss, all.ready);
            if (depth > 1) { ++stats.windows; stats.speculated_steps += ready; }
            // the steps before the first miss anywhere are final as they stand
            for (uint32_t d = 0; d < miss; ++d) {
                const double t = double(step + 1) * cfg_.dt;
                commit_predictions(window_latest_[d], t);
                depth_.record_prediction(true);
                state_ = ahead[d];
                ++step;
                stats.steps = step;
                if (step % cfg_.record_every == 0 || step == planned) record(t);
            }
            if (miss >= ready) continue;  // nothing missed (a window cut short by a failed solve further ahead starts again from here)
            // the step with the miss: relaxed with the received values until two sweeps agree everywhere
            const double t_next = double(step + 1) * cfg_.dt;
            next_ = ahead[miss];
            latest_ = window_latest_[miss];
            commit_predictions(latest_, t_next);
            depth_.record_prediction(false);
            int sweeps = 0;
            all.ok = 0;
            while (!all.ok && sweeps < cfg_.max_sweeps) {
                const std::vector<double> before = next_.voltages;
                pins_ = latest_;
                mine = Tally{};
                mine.failed = engine_->solve_step(state_, pins_, cfg_.dt, next_) ? 0 : 1;
                if (mine.failed) next_ = state_;
                ++stats.resolves;
                if (!swap_boundaries(next_.voltages, t_next)) return false;
                for (size_t i = 0; i < next_.voltages.size() && i < before.size(); ++i) {
                    const double a = next_.voltages[i], b = before[i];
                    if (std::fabs(a - b) > cfg_.reltol * 0.1 * std::max(std::fabs(a), std::fabs(b)) + cfg_.abstol * 0.1) { mine.ok = 0; break; }
                }
                if (!agree(mine, all)) return false;
                if (all.failed) return fail("Newton did not converge at t = " + std::to_string(t_next));
                ++sweeps;
            }
            if (!all.ok) ++stats.unconverged_steps;
            for (size_t g = 0; g < ghosts_.nodes.size(); ++g) ghosts_.nodes[g].amend(latest_[g].second);  // what the relaxation settled on
            state_ = next_;
            ++step;
            stats.steps = step;
            if (step % cfg_.record_every == 0 || step == planned) record(t_next);
            if (miss + 1 < ready) { ++stats.rollbacks; depth_.record_rollback(); }
            if (ahead.size() > size_t(miss) + 1) stats.discarded_steps += ahead.size() - size_t(miss) - 1;
        }
        return true;
    }

    // Feeds the owners' values of one step to the predictors and scores the predictions made for it.
    void commit_predictions(const std::vector<std::pair<uint64_t, double>>& values, double t) {
        std::vector<Correction> cs;
        cs.reserve(values.size());
        for (auto& l : values) cs.push_back({l.first, l.second, t});
        const bool hit = cs.empty() || ghosts_.apply_corrections(cs, cfg_.reltol * cfg_.accept_factor);
        (hit ? stats.prediction_hits : stats.prediction_misses) += cs.size();
    }

    void record(double t) {
        WaveformPoint pt{t, {}};
        pt.values.reserve(owned_.size());
        for (size_t i : owned_) pt.values.push_back(state_.voltages[i]);
        waveform.push_back(std::move(pt));
    }
};

}  // namespace nspice
