// In-process partitioned transient simulation: every partition owns a set of nets, sees foreign
// nets as ghost nodes. A partition solves a window of steps with *predicted* ghost voltages (the window's
// depth follows the hit rate: comm.hpp, SpeculativeDepthController), then the steps are verified in order:
// the voltages of the nets a partition owns go through the fabric (delta + quantization codec against the
// receiver's prediction), and every receiver checks its predictions. A step whose predictions were all
// within tolerance is accepted as it stands; otherwise the step is solved again with the received values
// (block Gauss-Jacobi relaxation) until two sweeps agree, and the rest of the window is discarded.
//
// The reference ships this mode as an experiment that falls back to a single node
// (nangila-spice/src/nangila_spice/orchestrator.py:222-233; solver loop solver.rs:104-245); the
// message types, codec and depth controller used here are the ones of comm.hpp.
//
// Partition files must overlap on cut elements: an element between a net of partition A and a net of
// partition B appears in both, with the foreign net listed in ghost_map. Net identity across
// partitions is the node *name* (ghost net id = net_name_hash(name)).
#pragma once
#include <atomic>
#include <map>
#include <memory>
#include <set>
#include <thread>
#include <unordered_map>

#include "parser.hpp"
#include "transient.hpp"

namespace nspice {

// Persistent worker threads for the per-partition solves of one sweep. Workers spin briefly on a
// generation counter and then yield, because a sweep is often only microseconds of work.
class SweepPool {
public:
    explicit SweepPool(unsigned threads) {
        for (unsigned i = 1; i < threads; ++i) workers_.emplace_back([this] { loop(); });
        nthreads_ = threads ? threads : 1;
    }
    ~SweepPool() {
        stop_.store(true);
        gen_.fetch_add(1);
        for (auto& t : workers_) t.join();
    }
    // Calls fn(i) for i in [0, count); the caller's thread takes part.
    void run(unsigned count, const std::function<void(unsigned)>& fn) {
        if (nthreads_ <= 1 || count <= 1) { for (unsigned i = 0; i < count; ++i) fn(i); return; }
        fn_ = &fn;
        count_ = count;
        next_.store(0);
        pending_.store(int(workers_.size()));
        gen_.fetch_add(1);
        work();
        int spins = 0;
        while (pending_.load(std::memory_order_acquire) != 0) { if (++spins > 200) std::this_thread::yield(); }
    }
    unsigned threads() const { return nthreads_; }
private:
    std::vector<std::thread> workers_;
    unsigned nthreads_ = 1, count_ = 0;
    const std::function<void(unsigned)>* fn_ = nullptr;
    std::atomic<unsigned> next_{0};
    std::atomic<int> pending_{0};
    std::atomic<uint64_t> gen_{0};
    std::atomic<bool> stop_{false};
    void work() {
        for (unsigned i = next_.fetch_add(1); i < count_; i = next_.fetch_add(1)) (*fn_)(i);
    }
    void loop() {
        uint64_t seen = 0;
        while (true) {
            int spins = 0;
            while (gen_.load(std::memory_order_acquire) == seen) {
                if (++spins > 2000) { std::this_thread::sleep_for(std::chrono::microseconds(20)); spins = 1000; }
                else if (spins > 200) std::this_thread::yield();
            }
            seen = gen_.load();
            if (stop_.load()) return;
            work();
            pending_.fetch_sub(1, std::memory_order_release);
        }
    }
};

struct PartitionedConfig {
    unsigned threads = 1;  // worker threads for the per-partition solves (1 = all on the calling thread)
    size_t min_unknowns_per_thread = 400;  // smaller partitions are solved on the calling thread whatever `threads` says
    double tstop = 1e-9, dt = 1e-12, reltol = 1e-3, abstol = 1e-6;
    uint32_t predict_depth = 5;
    int max_sweeps = 50;
    uint32_t record_every = 1;
    bool compress = true;
    // A prediction counts as a hit within accept_factor * reltol of the owner's value. A gate amplifies an error on its
    // input, so the bound on a boundary net has to be tighter than the accuracy wanted of the outputs: at 1.0 an 8-bit
    // adder was 14 mV (41 mV with windows) off the single-matrix run, at 0.25 it is 0.8 mV for 15 % more relaxed steps.
    double accept_factor = 0.25;
    bool speculate = true;  // run predict_depth-controlled windows of steps ahead between exchanges (false: one step at a time)
};

struct PartitionedStats {
    uint64_t steps = 0, prediction_hits = 0, prediction_misses = 0, resolves = 0, messages = 0, bytes_sent = 0, unconverged_steps = 0;
    uint64_t windows = 0, speculated_steps = 0, discarded_steps = 0, rollbacks = 0;  // windows deeper than one step
    double wall_time_secs = 0, codec_ratio = 1.0;
    bool completed = false;
    uint32_t final_depth = 0;
};

class PartitionedRunner {
public:
    PartitionedStats stats;
    std::vector<std::string> names;            // merged net names (owned nets of every partition)
    std::vector<WaveformPoint> waveform;       // merged, values in `names` order

    PartitionedRunner(std::vector<Netlist> parts, PartitionedConfig cfg)
        : cfg_(cfg), depth_(cfg.predict_depth, 1, cfg.predict_depth * 3), pool_(worker_count(cfg, parts)) {
        const uint32_t k = uint32_t(parts.size());
        FabricConfig fc;
        fc.compress = cfg.compress;
        mesh_ = create_mesh(k, fc);
        for (uint32_t p = 0; p < k; ++p) {
            Part part;
            part.names = parts[p].names_or_default();
            for (auto& g : parts[p].ghost_map) {
                part.ghost_index.emplace(g.net_id, part.ghosts.size());
                part.ghosts.add(GhostNode(g.net_id, g.owner));
                part.ghost_nodes.insert(g.local_node);
            }
            part.engine.reset(new SolverEngine(std::move(parts[p])));
            parts_.push_back(std::move(part));
        }
        // exports: for every ghost link of q owned by p, find p's local node of that name
        for (uint32_t q = 0; q < k; ++q)
            for (auto& g : parts_[q].engine->netlist.ghost_map) {
                if (g.owner >= k) throw std::runtime_error("ghost owner outside the partition set");
                Part& owner = parts_[g.owner];
                if (owner.owned_by_hash.empty())
                    for (size_t i = 0; i < owner.names.size(); ++i)
                        if (!owner.ghost_nodes.count(int(i) + 1)) owner.owned_by_hash.emplace(net_name_hash(owner.names[i]), int(i) + 1);
                auto found = owner.owned_by_hash.find(g.net_id);
                const int local = found == owner.owned_by_hash.end() ? -1 : found->second;
                if (local < 0) throw std::runtime_error("partition " + std::to_string(g.owner) + " does not own a net that partition " + std::to_string(q) + " lists as ghost");
                owner.exports[q].emplace_back(g.net_id, local);
                parts_[q].ghost_src.push_back({g.owner, local});
            }
        for (uint32_t p = 0; p < k; ++p)
            for (size_t i = 0; i < parts_[p].names.size(); ++i)
                if (!parts_[p].ghost_nodes.count(int(i) + 1)) { merged_.push_back({p, i}); names.push_back(parts_[p].names[i]); }
    }

    void run() {
        auto t0 = std::chrono::steady_clock::now();
        const uint32_t k = uint32_t(parts_.size());
        for (auto& p : parts_) p.state = p.engine->seeded_state();
        // consistent start: relax the DC point (or the seeded state when .ic lines exist) across partitions
        relax_dc();
        record(0.0);
        const uint64_t planned = cfg_.dt > 0 ? uint64_t(std::ceil(cfg_.tstop / cfg_.dt - 1e-9)) : 0;
        uint64_t step = 0;
        bool failed = false;
        while (step < planned && !failed) {
            // Every partition runs `depth` steps ahead on predicted ghost voltages without talking to anybody; then the
            // steps are checked in order against what the owners computed. A step whose predictions all hit is final as
            // it stands. The first step with a miss is relaxed the lockstep way, and what was computed beyond it is thrown
            // away (a rollback): those steps started from a state that has just changed.
            const uint64_t depth = std::min<uint64_t>(cfg_.speculate ? std::max<uint32_t>(1, depth_.depth()) : 1, planned - step);
            std::atomic<bool> bad{false};
            pool_.run(k, [&](unsigned p) {
                Part& part = parts_[p];
                part.ahead_states.clear();
                part.ahead_pins.clear();
                const PartitionState* cur = &part.state;
                for (uint64_t d = 0; d < depth; ++d) {
                    part.ahead_pins.push_back(part.ghosts.predict_all(double(step + d + 1) * cfg_.dt));
                    PartitionState next{0};
                    if (!part.engine->solve_step(*cur, part.ahead_pins.back(), cfg_.dt, next)) {
                        if (d == 0) bad.store(true);  // further ahead a failure only shortens the window
                        part.ahead_pins.pop_back();
                        break;
                    }
                    part.ahead_states.push_back(std::move(next));
                    cur = &part.ahead_states.back();
                }
            });
            failed = bad.load();
            if (failed) break;
            uint64_t ready = depth;
            for (auto& part : parts_) ready = std::min<uint64_t>(ready, part.ahead_states.size());
            if (depth > 1) { ++stats.windows; stats.speculated_steps += ready; }
            for (uint64_t d = 0; d < ready && !failed; ++d) {
                const double t_next = double(step + 1) * cfg_.dt;
                for (auto& part : parts_) { part.next = part.ahead_states[d]; part.pins = part.ahead_pins[d]; }
                bool all_ok = exchange(t_next, /*count=*/true);
                int sweeps = 0;
                while (!all_ok && sweeps < cfg_.max_sweeps) {
                    // solve again with the received (true, as of the last sweep) ghost values
                    std::vector<std::vector<double>> before;
                    for (auto& part : parts_) before.push_back(part.next.voltages);
                    pool_.run(k, [&](unsigned p) {
                        Part& part = parts_[p];
                        part.pins = part.latest;
                        if (!part.engine->solve_step(part.state, part.pins, cfg_.dt, part.next)) bad.store(true);
                    });
                    stats.resolves += k;
                    failed = bad.load();
                    if (failed) break;
                    exchange(t_next, /*count=*/false);
                    all_ok = true;
                    for (uint32_t p = 0; p < k; ++p)
                        for (size_t i = 0; i < parts_[p].next.voltages.size() && i < before[p].size(); ++i) {
                            double a = parts_[p].next.voltages[i], b = before[p][i];
                            if (std::fabs(a - b) > cfg_.reltol * 0.1 * std::max(std::fabs(a), std::fabs(b)) + cfg_.abstol * 0.1) { all_ok = false; break; }
                        }
                    ++sweeps;
                }
                if (failed) break;
                if (!all_ok) ++stats.unconverged_steps;
                if (sweeps > 0)  // the predictors learn from what the relaxation settled on, not from the first speculative values
                    for (auto& part : parts_)
                        for (size_t g = 0; g < part.ghosts.nodes.size() && g < part.latest.size(); ++g) part.ghosts.nodes[g].amend(part.latest[g].second);
                for (auto& part : parts_) part.state = part.next;
                ++step;
                if (step % cfg_.record_every == 0 || step == planned) record(t_next);
                if (sweeps > 0) {
                    if (d + 1 < ready) { ++stats.rollbacks; stats.discarded_steps += ready - d - 1; depth_.record_rollback(); }
                    break;
                }
            }
        }
        stats.steps = step;
        stats.completed = !failed && step == planned;
        stats.final_depth = depth_.depth();
        uint64_t raw = 0, comp = 0;
        for (auto& n : mesh_) { stats.messages += n->stats.sent; stats.bytes_sent += n->stats.bytes_sent; raw += n->codec.stats.raw_bytes; comp += n->codec.stats.compressed_bytes; }
        stats.codec_ratio = comp ? double(raw) / double(comp) : 1.0;
        stats.wall_time_secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    }

private:
    // Threads pay for themselves only when a sweep is real work: below min_unknowns_per_thread unknowns per partition the
    // hand-over between threads (and, on a busy machine, waiting to be scheduled) costs more than the solves.
    static unsigned worker_count(const PartitionedConfig& cfg, const std::vector<Netlist>& parts) {
        size_t largest = 0;
        for (auto& p : parts) largest = std::max(largest, size_t(std::max(p.num_nodes, 0)));
        if (largest < cfg.min_unknowns_per_thread) return 1;
        return std::min<unsigned>(std::max(1u, cfg.threads), unsigned(parts.size()));
    }

    struct Part {
        std::unique_ptr<SolverEngine> engine;
        GhostBuffer ghosts;
        std::set<int> ghost_nodes;
        std::vector<std::string> names;
        std::map<uint32_t, std::vector<std::pair<uint64_t, int>>> exports;  // consumer -> (net id, local node)
        PartitionState state{0}, next{0};
        std::vector<std::pair<uint64_t, double>> pins, latest;              // in the order of ghosts.nodes
        std::vector<PartitionState> ahead_states;                             // the window: states after each speculative step
        std::vector<std::vector<std::pair<uint64_t, double>>> ahead_pins;     // and the ghost voltages each of them assumed
        struct GhostSrc { uint32_t owner; int local; };
        std::vector<GhostSrc> ghost_src;                                      // where each ghost's value lives, same order
        std::unordered_map<uint64_t, size_t> ghost_index;                     // net id -> position in ghosts.nodes
        std::unordered_map<uint64_t, int> owned_by_hash;                      // name hash -> local node of the nets this partition owns
    };
    struct MergedRef { uint32_t part; size_t index; };
    PartitionedConfig cfg_;
    std::vector<Part> parts_;
    std::vector<std::unique_ptr<FabricNode>> mesh_;
    std::vector<MergedRef> merged_;
    SpeculativeDepthController depth_;
    SweepPool pool_;

    // Every owner publishes its boundary voltages of `next`; receivers decode, remember them and
    // (when count is set) score their predictions. Returns whether every prediction was a hit.
    bool exchange(double t, bool count) {
        const uint32_t k = uint32_t(parts_.size());
        // `pins` and `latest` are in the order of the partition's ghost list; a value that no message corrects
        // (its delta was below the codec's floor) stays what was pinned
        for (auto& part : parts_) part.latest = part.pins;
        for (uint32_t p = 0; p < k; ++p)
            for (auto& ex : parts_[p].exports) {
                ResidualMessage m;
                m.from = p; m.to = ex.first; m.time = t;
                // the sender encodes against what the receiver pinned, which both sides know after the
                // previous exchange; on the first sweep that is the receiver's prediction
                const Part& to = parts_[ex.first];
                std::vector<std::pair<uint64_t, double>> base;
                base.reserve(ex.second.size());
                for (auto& e : ex.second) {
                    m.updates.emplace_back(e.first, parts_[p].next.voltages[size_t(e.second - 1)]);
                    auto it = to.ghost_index.find(e.first);
                    if (it != to.ghost_index.end() && it->second < to.pins.size()) base.push_back(to.pins[it->second]);
                }
                mesh_[p]->send_residual(m, base);
            }
        bool all_ok = true;
        for (uint32_t q = 0; q < k; ++q) {
            Part& part = parts_[q];
            for (auto& fm : mesh_[q]->drain_inbox()) {
                if (fm.kind != FabricMessage::Residual) continue;
                ResidualMessage m = mesh_[q]->decode_residual(fm.residual);
                for (auto& u : m.updates) {
                    auto it = part.ghost_index.find(u.first);
                    if (it != part.ghost_index.end() && it->second < part.latest.size()) part.latest[it->second].second = u.second;
                }
                if (count) {
                    std::vector<Correction> cs;
                    for (auto& u : m.updates) cs.push_back({u.first, u.second, t});
                    bool ok = part.ghosts.apply_corrections(cs, cfg_.reltol * cfg_.accept_factor);
                    (ok ? stats.prediction_hits : stats.prediction_misses) += cs.size();
                    depth_.record_prediction(ok);
                    all_ok = all_ok && ok;
                }
            }
        }
        return all_ok;
    }
    // Block relaxation of the DC point: each partition solves its operating point with the ghosts
    // pinned to the neighbours' latest values.
    void relax_dc() {
        const uint32_t k = uint32_t(parts_.size());
        for (auto& part : parts_) { part.next = part.state; part.pins.clear(); part.latest.clear(); }
        for (int sweep = 0; sweep < 200; ++sweep) {
            double change = 0.0;
            for (uint32_t p = 0; p < k; ++p) {
                Part& part = parts_[p];
                if (!part.engine->netlist.initial_conditions.empty()) continue;
                // ghosts pinned to what their owners hold now; the partition's own DC solve may step its conductance
                PartitionState out{0};
                std::vector<std::pair<uint64_t, double>> pins;
                pins.reserve(part.ghost_src.size());
                for (size_t g = 0; g < part.ghost_src.size(); ++g)
                    pins.emplace_back(part.ghosts.nodes[g].net_id, parts_[part.ghost_src[g].owner].next.voltages[size_t(part.ghost_src[g].local - 1)]);
                PartitionState seed = part.next;
                seed.cap_currents.clear();
                if (part.engine->solve_dc(seed, out, pins)) {
                    for (size_t i = 0; i < out.voltages.size(); ++i) change = std::max(change, std::fabs(out.voltages[i] - part.next.voltages[i]));
                    part.next.voltages = out.voltages;
                }
            }
            if (change < 1e-9) break;
        }
        for (auto& part : parts_) {
            part.state.voltages = part.next.voltages;
            part.state.cap_currents.clear();
            part.state.time = 0.0;
            // ghosts start from the neighbours' initial values
        }
        for (auto& part : parts_)
            for (size_t g = 0; g < part.ghost_src.size(); ++g)
                part.ghosts.nodes[g].apply_correction(parts_[part.ghost_src[g].owner].state.voltages[size_t(part.ghost_src[g].local - 1)], 0.0, cfg_.reltol);
    }
    void record(double t) {
        WaveformPoint pt{t, {}};
        for (auto& r : merged_) pt.values.push_back(parts_[r.part].state.voltages[r.index]);
        waveform.push_back(std::move(pt));
    }
};

}  // namespace nspice
