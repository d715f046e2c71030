// Modified nodal analysis, Newton-Raphson and the per-step solver of one partition.
//
// What it covers of the reference: MnaSystem stamping (nangila-spice/nangila-node/src/mna.rs:108-492),
// NewtonSolver (newton.rs:24-227), SolverEngine::solve_builtin / DC operating point
// (ngspice_ffi.rs:156-400). Differences by design: the matrix pattern is built once per engine and
// every Newton iteration only rewrites values through precomputed slots (the reference rebuilds a
// dense N x N matrix and densifies it again for every iteration); the linear solve is sparse.
//
// Unknown ordering: node voltages (num_nodes), then one branch current per voltage source, then one
// per inductor — the same ordering as the reference, so state vectors are interchangeable.
#pragma once
#include <array>
#include <cstdint>
#include <map>
#include <tuple>
#include <unordered_map>

#include "circuit.hpp"
#include "sparse.hpp"

namespace nspice {

enum class Integration { BackwardEuler, Trapezoidal };

struct PartitionState {
    std::vector<double> voltages;      // full solution vector (nodes, then branch currents)
    std::vector<double> cap_currents;  // one per capacitor, in element order; empty before the first step
    std::vector<double> slopes;        // d/dt of every unknown over the step that led here; empty before the first step
    double time = 0.0;
    bool validated = false;
    explicit PartitionState(size_t n = 0) : voltages(n, 0.0) {}
};

struct NrConfig {
    int max_iter = 150;
    double reltol = 1e-3;
    double abstol = 1e-6;
    double damping = 1.0;
    // Largest change of one node voltage per iteration; the exponential and square-law devices are only
    // linearised locally, so an unlimited update can jump into a region from which the iteration oscillates.
    double max_dv = 0.6;
    // How often solve_step may halve a step that did not converge (2^k sub-steps at most).
    int max_cuts = 8;
};

struct NrStats {
    uint64_t total_iterations = 0, converged_count = 0, failed_count = 0, linear_solves = 0;
    double avg_iterations() const { return converged_count ? double(total_iterations) / double(converged_count + failed_count) : 0.0; }
};

struct NrOutcome {
    std::vector<double> x;
    int iterations = 0;
    bool converged = false;
    double final_error = 0.0;
};

// Newton iteration over a callback that fills the system for the current guess.
class NewtonSolver {
public:
    NrConfig config;
    NrStats stats;
    LinearSolver linear;

    // The first `limited` unknowns are node voltages and get the per-iteration step limit. A system that does
    // not depend on the guess (`linear_system`) is solved once: the first solution is exact.
    template <class Build>
    NrOutcome solve(std::vector<double> guess, CsrMatrix& m, Build&& build, int limited = 0, bool linear_system = false) {
        NrOutcome out;
        out.x = std::move(guess);
        out.x.resize(size_t(m.n), 0.0);
        for (int it = 0; it < config.max_iter; ++it) {
            build(out.x, m);
            ++stats.linear_solves;
            if (!linear.solve(m)) break;
            double max_err = 0.0;
            for (int i = 0; i < m.n; ++i) {
                double vn = m.solution[size_t(i)], vo = out.x[size_t(i)];
                double tol = config.reltol * std::max(std::fabs(vn), std::fabs(vo)) + config.abstol;
                max_err = std::max(max_err, std::fabs(vn - vo) / std::max(tol, config.abstol));
                double step = config.damping * (vn - vo);
                if (i < limited && config.max_dv > 0.0) step = std::max(-config.max_dv, std::min(config.max_dv, step));
                out.x[size_t(i)] = vo + step;
            }
            out.iterations = it + 1;
            out.final_error = max_err;
            if (max_err < 1.0 || (linear_system && config.damping == 1.0)) { out.converged = true; break; }
        }
        stats.total_iterations += uint64_t(out.iterations);
        if (out.converged) ++stats.converged_count; else ++stats.failed_count;
        return out;
    }
};

// Pattern-once MNA assembler.
class Assembler {
public:
    int num_nodes = 0, num_vs = 0, num_ind = 0, size = 0;
    CsrMatrix m;
    static constexpr double kGhostG = 1e12;
    double gmin = 1e-12;  // tiny conductance from every node to ground; keeps floating nodes solvable

    Assembler() = default;
    Assembler(const Netlist& nl) { build(nl); }

    void build(const Netlist& nl) {
        net_ = &nl;
        num_nodes = nl.num_nodes;
        num_vs = num_ind = 0;
        for (auto& e : nl.elements) {
            if (e.kind == Element::VSource) ++num_vs;
            if (e.kind == Element::Inductor) ++num_ind;
        }
        size = num_nodes + num_vs + num_ind;
        std::vector<std::tuple<int, int, double>> t;
        auto add = [&](int r, int c) { if (r >= 0 && c >= 0) t.emplace_back(r, c, 0.0); };
        // every node row and every inductor row has a diagonal entry; the branch row of a voltage source has none
        // (it reads v(a) - v(b) = V), which lets the factorisation take source rows and columns as free pivots
        for (int i = 0; i < num_nodes; ++i) add(i, i);
        for (int i = num_nodes + num_vs; i < size; ++i) add(i, i);
        int vs = 0, ind = 0;
        for (auto& e : nl.elements) {
            switch (e.kind) {
                case Element::Resistor: case Element::Capacitor: case Element::Diode: {
                    int a = e.a - 1, b = e.b - 1;
                    add(a, a); add(a, b); add(b, a); add(b, b);
                    break;
                }
                case Element::VSource: case Element::Inductor: {
                    int br = e.kind == Element::VSource ? num_nodes + vs++ : num_nodes + num_vs + ind++;
                    int a = e.a - 1, b = e.b - 1;
                    add(a, br); add(br, a); add(b, br); add(br, b);
                    break;
                }
                case Element::Mosfet: {
                    int d = e.d - 1, g = e.g - 1, s = e.s - 1;
                    for (int r : {d, s}) for (int c : {d, g, s}) add(r, c);
                    break;
                }
                default: break;
            }
        }
        m = CsrMatrix::from_triplets(size, t, -1.0);
        // slots
        slots_.assign(nl.elements.size(), {});
        vs = ind = 0;
        for (size_t k = 0; k < nl.elements.size(); ++k) {
            auto& e = nl.elements[k];
            auto& s = slots_[k];
            s.fill(-1);
            auto S = [&](int r, int c) { return (r >= 0 && c >= 0) ? m.slot(r, c) : -1; };
            switch (e.kind) {
                case Element::Resistor: case Element::Capacitor: case Element::Diode: {
                    int a = e.a - 1, b = e.b - 1;
                    s[0] = S(a, a); s[1] = S(a, b); s[2] = S(b, a); s[3] = S(b, b);
                    break;
                }
                case Element::VSource: case Element::Inductor: {
                    int br = e.kind == Element::VSource ? num_nodes + vs++ : num_nodes + num_vs + ind++;
                    int a = e.a - 1, b = e.b - 1;
                    s[0] = S(a, br); s[1] = S(br, a); s[2] = S(b, br); s[3] = S(br, b); s[4] = e.kind == Element::Inductor ? S(br, br) : -1; s[5] = br;
                    break;
                }
                case Element::Mosfet: {
                    int d = e.d - 1, g = e.g - 1, sn = e.s - 1;
                    s[0] = S(d, g); s[1] = S(d, d); s[2] = S(d, sn); s[3] = S(sn, g); s[4] = S(sn, d); s[5] = S(sn, sn);
                    break;
                }
                case Element::Ghost: s[0] = S(e.a - 1, e.a - 1); break;
                default: break;
            }
        }
        diag_.resize(size_t(num_nodes));
        for (int i = 0; i < num_nodes; ++i) diag_[size_t(i)] = m.slot(i, i);
    }

    // Linear (guess-independent) part: everything but diodes and MOSFETs. dt <= 0 is the DC form:
    // capacitors open, inductors a 0 V source.
    void stamp_linear(const std::vector<double>& prev, const std::vector<double>& prev_ic, double dt, double time,
                      Integration method, const std::vector<std::pair<int, double>>& ghosts) {
        std::fill(m.val.begin(), m.val.end(), 0.0);
        std::fill(m.rhs.begin(), m.rhs.end(), 0.0);
        auto V = [&](int node) { return (node > 0 && size_t(node - 1) < prev.size()) ? prev[size_t(node - 1)] : 0.0; };
        for (int i = 0; i < num_nodes; ++i) m.val[size_t(diag_[size_t(i)])] += gmin;
        size_t cap = 0;
        const Netlist& nl = *net_;
        for (size_t k = 0; k < nl.elements.size(); ++k) {
            auto& e = nl.elements[k];
            auto& s = slots_[k];
            switch (e.kind) {
                case Element::Resistor: conduct(s, 1.0 / e.value); break;
                case Element::Capacitor: {
                    double ic = cap < prev_ic.size() ? prev_ic[cap] : 0.0;
                    ++cap;
                    if (dt <= 0.0) break;
                    double g = (method == Integration::Trapezoidal ? 2.0 : 1.0) * e.value / dt;
                    double ieq = g * (V(e.a) - V(e.b)) + (method == Integration::Trapezoidal ? ic : 0.0);
                    conduct(s, g);
                    if (e.a > 0) m.rhs[size_t(e.a - 1)] += ieq;
                    if (e.b > 0) m.rhs[size_t(e.b - 1)] -= ieq;
                    break;
                }
                case Element::VSource: branch(s, e.source.value_at(time), 0.0); break;
                case Element::Inductor: {
                    if (dt <= 0.0) { branch(s, 0.0, 0.0); break; }
                    int br = s[5];
                    double iprev = size_t(br) < prev.size() ? prev[size_t(br)] : 0.0;
                    if (method == Integration::Trapezoidal) {
                        double r = -2.0 * e.value / dt;
                        branch(s, r * iprev - (V(e.a) - V(e.b)), r);
                    } else {
                        double r = -e.value / dt;
                        branch(s, r * iprev, r);
                    }
                    break;
                }
                case Element::ISource: {
                    double i = e.source.value_at(time);
                    if (e.a > 0) m.rhs[size_t(e.a - 1)] -= i;
                    if (e.b > 0) m.rhs[size_t(e.b - 1)] += i;
                    break;
                }
                case Element::Ghost: pin(e.a, e.value); break;
                default: break;
            }
        }
        for (auto& g : ghosts) pin(g.first, g.second);
        lin_val_ = m.val;
        lin_rhs_ = m.rhs;
    }

    // Adds the linearised nonlinear devices around `guess` on top of the saved linear part.
    void stamp_nonlinear(const std::vector<double>& guess) {
        m.val = lin_val_;
        m.rhs = lin_rhs_;
        auto V = [&](int node) { return (node > 0 && size_t(node - 1) < guess.size()) ? guess[size_t(node - 1)] : 0.0; };
        const Netlist& nl = *net_;
        for (size_t k = 0; k < nl.elements.size(); ++k) {
            auto& e = nl.elements[k];
            auto& s = slots_[k];
            if (e.kind == Element::Diode) {
                double g, ieq;
                e.diode.companion(V(e.a) - V(e.b), g, ieq);
                conduct(s, g);
                if (e.a > 0) m.rhs[size_t(e.a - 1)] -= ieq;
                if (e.b > 0) m.rhs[size_t(e.b - 1)] += ieq;
            } else if (e.kind == Element::Mosfet) {
                double gm, gds, ieq;
                e.mos.companion(V(e.g) - V(e.s), V(e.d) - V(e.s), gm, gds, ieq);
                // drain row: +id ; source row: -id, with id = gm (vg - vs) + gds (vd - vs) + ieq
                if (s[0] >= 0) m.val[size_t(s[0])] += gm;
                if (s[1] >= 0) m.val[size_t(s[1])] += gds;
                if (s[2] >= 0) m.val[size_t(s[2])] -= gm + gds;
                if (s[3] >= 0) m.val[size_t(s[3])] -= gm;
                if (s[4] >= 0) m.val[size_t(s[4])] -= gds;
                if (s[5] >= 0) m.val[size_t(s[5])] += gm + gds;
                if (e.d > 0) m.rhs[size_t(e.d - 1)] -= ieq;
                if (e.s > 0) m.rhs[size_t(e.s - 1)] += ieq;
            }
        }
    }

    bool has_nonlinear() const {
        for (auto& e : net_->elements) if (e.kind == Element::Diode || e.kind == Element::Mosfet) return true;
        return false;
    }

private:
    const Netlist* net_ = nullptr;
    std::vector<std::array<int, 6>> slots_;
    std::vector<int> diag_;
    std::vector<double> lin_val_, lin_rhs_;

    void conduct(const std::array<int, 6>& s, double g) {
        if (s[0] >= 0) m.val[size_t(s[0])] += g;
        if (s[1] >= 0) m.val[size_t(s[1])] -= g;
        if (s[2] >= 0) m.val[size_t(s[2])] -= g;
        if (s[3] >= 0) m.val[size_t(s[3])] += g;
    }
    void branch(const std::array<int, 6>& s, double rhs, double r) {
        if (s[0] >= 0) m.val[size_t(s[0])] += 1.0;
        if (s[1] >= 0) m.val[size_t(s[1])] += 1.0;
        if (s[2] >= 0) m.val[size_t(s[2])] -= 1.0;
        if (s[3] >= 0) m.val[size_t(s[3])] -= 1.0;
        if (s[4] >= 0) m.val[size_t(s[4])] += r;
        m.rhs[size_t(s[5])] += rhs;
    }
    void pin(int node, double v) {
        if (node <= 0 || node > num_nodes) return;
        m.val[size_t(diag_[size_t(node - 1)])] += kGhostG;
        m.rhs[size_t(node - 1)] += kGhostG * v;
    }
};

class SolverEngine {
public:
    Netlist netlist;
    NewtonSolver newton;

    explicit SolverEngine(Netlist nl) : netlist(std::move(nl)), asm_(netlist) {}
    SolverEngine(const SolverEngine&) = delete;

    int size() const { return asm_.size; }
    const Assembler& assembler() const { return asm_; }

    // Sources at t = 0 and `.ic` values, everything else 0.
    PartitionState seeded_state() const {
        PartitionState st{size_t(size())};
        for (auto& e : netlist.elements)
            if (e.kind == Element::VSource) {
                double v = e.source.value_at(0.0);
                if (e.a > 0 && e.b == 0) st.voltages[size_t(e.a - 1)] = v;
                else if (e.b > 0 && e.a == 0) st.voltages[size_t(e.b - 1)] = -v;
            }
        for (auto& ic : netlist.initial_conditions)
            if (ic.first > 0 && ic.first <= netlist.num_nodes) st.voltages[size_t(ic.first - 1)] = ic.second;
        return st;
    }

    // With `.ic` lines the seeded state is the start; otherwise the DC operating point.
    PartitionState initial_state() {
        PartitionState seeded = seeded_state();
        if (!netlist.initial_conditions.empty()) return seeded;
        PartitionState dc{0};
        return solve_dc(seeded, dc) ? dc : seeded;
    }

    // Plain Newton from the seeded state first; if that fails, conductance stepping: solve with a large
    // conductance from every node to ground, then lower it by decades with the last solution as the guess.
    // `ghost_voltages` pins foreign nets of a partition.
    bool solve_dc(const PartitionState& seeded, PartitionState& out, const std::vector<std::pair<uint64_t, double>>& ghost_voltages = {}) {
        const std::vector<std::pair<int, double>> pins = node_pins(ghost_voltages);
        NrOutcome r = run_newton(seeded, pins, 0.0, 0.0, Integration::BackwardEuler);
        if (!r.converged) {
            const double target = asm_.gmin;
            PartitionState g = seeded;
            bool ok = true;
            for (double gm = 1e-2; ok && gm > target * 1.5; gm *= 0.1) {
                asm_.gmin = gm;
                r = run_newton(g, pins, 0.0, 0.0, Integration::BackwardEuler);
                ok = r.converged;
                if (ok) g.voltages = r.x;
            }
            asm_.gmin = target;
            if (ok) r = run_newton(g, pins, 0.0, 0.0, Integration::BackwardEuler);
            ++dc_gmin_stepping;
        }
        if (!r.converged) return false;
        out = PartitionState{0};
        out.voltages = r.x;
        out.time = 0.0;
        return true;
    }

    // One step of size dt from `cur`; ghost nodes are pinned to the given voltages. Trapezoidal when
    // capacitor currents are known, Backward-Euler on the first step and as the retry when the
    // trapezoidal Newton does not converge. A step that still does not converge is taken as two half
    // steps (recursively, NrConfig::max_cuts deep) with the pins held.
    bool solve_step(const PartitionState& cur, const std::vector<std::pair<uint64_t, double>>& ghost_voltages, double dt,
                    PartitionState& out) {
        return advance(cur, node_pins(ghost_voltages), dt, 0, out);
    }

    uint64_t be_fallbacks = 0, step_cuts = 0, dc_gmin_stepping = 0;
    bool extrapolate_guess = true;

private:
    Assembler asm_;
    std::unordered_map<uint64_t, int> ghost_node_;  // net id -> local node, built on first use

    std::vector<std::pair<int, double>> node_pins(const std::vector<std::pair<uint64_t, double>>& ghost_voltages) {
        std::vector<std::pair<int, double>> pins;
        if (ghost_voltages.empty()) return pins;
        if (ghost_node_.size() != netlist.ghost_map.size()) {
            ghost_node_.clear();
            for (auto& link : netlist.ghost_map) ghost_node_.emplace(link.net_id, link.local_node);
        }
        pins.reserve(ghost_voltages.size());
        for (auto& gv : ghost_voltages) {
            auto it = ghost_node_.find(gv.first);
            if (it != ghost_node_.end()) pins.emplace_back(it->second, gv.second);
        }
        return pins;
    }

    bool advance(const PartitionState& cur, const std::vector<std::pair<int, double>>& pins, double dt, int depth, PartitionState& out) {
        if (single_step(cur, pins, dt, out)) return true;
        if (depth >= newton.config.max_cuts || dt <= 0.0) return false;
        ++step_cuts;
        PartitionState mid{0};
        return advance(cur, pins, 0.5 * dt, depth + 1, mid) && advance(mid, pins, 0.5 * dt, depth + 1, out);
    }

    bool single_step(const PartitionState& cur, const std::vector<std::pair<int, double>>& pins, double dt, PartitionState& out) {
        Integration method = cur.cap_currents.empty() ? Integration::BackwardEuler : Integration::Trapezoidal;
        NrOutcome r = run_newton(cur, pins, dt, cur.time + dt, method);
        if (!r.converged && method == Integration::Trapezoidal) {
            ++be_fallbacks;
            method = Integration::BackwardEuler;
            r = run_newton(cur, pins, dt, cur.time + dt, method);
        }
        if (!r.converged) return false;
        out = PartitionState{0};
        out.voltages = std::move(r.x);
        out.time = cur.time + dt;
        if (dt > 0.0 && out.voltages.size() == cur.voltages.size()) {
            out.slopes.resize(out.voltages.size());
            for (size_t i = 0; i < out.slopes.size(); ++i) out.slopes[i] = (out.voltages[i] - cur.voltages[i]) / dt;
        }
        auto V = [](const std::vector<double>& v, int node) { return (node > 0 && size_t(node - 1) < v.size()) ? v[size_t(node - 1)] : 0.0; };
        size_t cap = 0;
        for (auto& e : netlist.elements) {
            if (e.kind != Element::Capacitor) continue;
            double dv = (V(out.voltages, e.a) - V(out.voltages, e.b)) - (V(cur.voltages, e.a) - V(cur.voltages, e.b));
            double prev_ic = cap < cur.cap_currents.size() ? cur.cap_currents[cap] : 0.0;
            double ic = dt > 0.0 ? (method == Integration::Trapezoidal ? 2.0 * e.value / dt * dv - prev_ic : e.value / dt * dv) : 0.0;
            out.cap_currents.push_back(ic);
            ++cap;
        }
        return true;
    }

    NrOutcome run_newton(const PartitionState& cur, const std::vector<std::pair<int, double>>& pins, double dt, double t,
                         Integration method) {
        asm_.stamp_linear(cur.voltages, cur.cap_currents, dt, t, method, pins);
        const bool nonlinear = asm_.has_nonlinear();
        // Newton starts from the straight line through the last step (nonlinear transient steps only: a linear system
        // needs no guess, and the DC solve has no time)
        std::vector<double> guess = cur.voltages;
        if (nonlinear && extrapolate_guess && dt > 0.0 && cur.slopes.size() == guess.size())
            for (int i = 0; i < asm_.num_nodes; ++i) guess[size_t(i)] += cur.slopes[size_t(i)] * dt;
        return newton.solve(std::move(guess), asm_.m, [&](const std::vector<double>& x, CsrMatrix&) {
            if (nonlinear) asm_.stamp_nonlinear(x);
        }, nonlinear ? asm_.num_nodes : 0, !nonlinear);
    }
};

}  // namespace nspice
