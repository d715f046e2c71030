// Python module nangila_spice._native: the simulator core for tests, the orchestrator and notebooks.
// Netlists cross the boundary as JSON text (the partition-file form), numeric data as lists.
#include <algorithm>
#include <unordered_map>

#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "balancer.hpp"
#include "nz.hpp"
#include "parser.hpp"
#include "partitioned.hpp"
#include "pvt.hpp"
#include "transient.hpp"

namespace py = pybind11;
using namespace nspice;

static LinearBackend backend_of(const std::string& s) {
    if (s == "dense") return LinearBackend::Dense;
    if (s == "krylov") return LinearBackend::Krylov;
    if (s == "cuda") return LinearBackend::Cuda;
    if (s == "lu" || s.empty()) return LinearBackend::SparseLU;
    throw std::invalid_argument("solver must be 'lu', 'dense', 'krylov' or 'cuda'");
}

static py::dict stats_dict(const SimStats& s) {
    py::dict d;
    d["total_steps"] = s.total_steps; d["wall_time_secs"] = s.wall_time_secs; d["prediction_hits"] = s.prediction_hits;
    d["prediction_misses"] = s.prediction_misses; d["rollbacks"] = s.rollbacks; d["completed"] = s.completed;
    d["hit_rate"] = s.hit_rate(); d["solver_steps"] = s.solver_steps; d["rejected_steps"] = s.rejected_steps;
    return d;
}

static const char* class_name(SignalClass c) {
    switch (c) {
        case SignalClass::Smooth: return "Smooth";
        case SignalClass::Decaying: return "Decaying";
        case SignalClass::Stiff: return "Stiff";
        default: return "Unknown";
    }
}

// Waveform samples as one (points x nets) float64 array: a list of lists costs a Python float per sample.
static py::array_t<double> waveform_array(const std::vector<WaveformPoint>& w) {
    const py::ssize_t rows = py::ssize_t(w.size()), cols = rows ? py::ssize_t(w[0].values.size()) : 0;
    py::array_t<double> a({rows, cols});
    double* dst = a.mutable_data();
    for (py::ssize_t r = 0; r < rows; ++r) {
        const auto& v = w[size_t(r)].values;
        for (py::ssize_t c = 0; c < cols; ++c) dst[r * cols + c] = size_t(c) < v.size() ? v[size_t(c)] : 0.0;
    }
    return a;
}

PYBIND11_MODULE(_native, m) {
    m.doc() = "nangila-spice native core";

    m.def("parse_scaled", [](const std::string& s) -> py::object { double v; if (!parse_scaled(s, v)) return py::none(); return py::float_(v); });
    m.def("net_name_hash", &net_name_hash);
    m.def("set_cuda_library", &CudaKrylov::set_library, "path of libnangila_kernels.so for solver='cuda'");
    m.def("parse_spice", [](const std::string& text, const std::string& name, const std::string& process, double vdd, double temp) {
        Corner c; c.process = process; c.vdd = vdd; c.temp_c = temp;
        SpiceParser p(c);
        Netlist nl = p.parse_text(text, name);
        return py::make_tuple(nl.to_json().dump(), p.warnings);
    }, py::arg("text"), py::arg("name") = "netlist", py::arg("process") = "TT", py::arg("vdd") = 1.8, py::arg("temp") = 27.0);
    m.def("expand_includes", &SpiceParser::expand, py::arg("text"), py::arg("directory"), py::arg("deck_path") = "",
          "deck text with every readable `.include <file>` / `.lib <file> [section]` replaced by what it names (paths relative to `directory`)");
    m.def("netlist_roundtrip", [](const std::string& js) { return Netlist::from_json(Json::parse(js)).to_json().dump(); });
    m.def("source_value", [](const std::string& js, double t) { return SourceWaveform::from_json(Json::parse(js)).value_at(t); });

    // ---- simulation ---------------------------------------------------------------------------
    m.def("simulate", [](const std::string& netlist_json, double tstop, double dt, double reltol, const std::string& solver, uint32_t record_every,
                         uint32_t predict_depth, std::vector<std::tuple<uint32_t, double, std::vector<std::pair<uint64_t, double>>>> inject,
                         std::vector<double> rollbacks, bool adaptive, double lte_reltol, double max_step_factor, std::vector<std::string> record_nodes) {
        Netlist nl = Netlist::from_json(Json::parse(netlist_json));
        std::vector<std::string> names = nl.names_or_default();
        std::vector<uint32_t> keep;
        if (!record_nodes.empty()) {  // names compared without case; unknown names are skipped
            auto lower = [](std::string v) { for (auto& c : v) c = char(std::tolower((unsigned char)c)); return v; };
            std::unordered_map<std::string, uint32_t> at;
            for (uint32_t i = 0; i < names.size(); ++i) at.emplace(lower(names[i]), i);
            std::vector<std::string> kept;
            for (auto& want : record_nodes) {
                auto it = at.find(lower(want));
                if (it != at.end() && std::find(keep.begin(), keep.end(), it->second) == keep.end()) { keep.push_back(it->second); kept.push_back(names[it->second]); }
            }
            names = kept;
        }
        GhostBuffer ghosts(predict_depth);
        for (auto& g : nl.ghost_map) ghosts.add(GhostNode(g.net_id, g.owner));
        SimConfig cfg;
        cfg.tstop = tstop; cfg.dt = dt; cfg.reltol = reltol; cfg.record_every = std::max(1u, record_every); cfg.predict_depth = predict_depth;
        cfg.adaptive = adaptive; cfg.lte_reltol = lte_reltol; cfg.max_step_factor = max_step_factor;
        cfg.record_nodes = keep;
        CommLayer comm(0, 1);
        for (auto& msg : inject) { ResidualMessage r; r.from = std::get<0>(msg); r.time = std::get<1>(msg); r.updates = std::get<2>(msg); comm.inject_message(r); }
        for (double t : rollbacks) comm.inject_rollback({1, t});
        TransientSolver s(std::move(nl), std::move(ghosts), std::move(comm), cfg);
        s.engine().newton.config.reltol = reltol;
        s.engine().newton.linear.backend = backend_of(solver);
        PartitionState fin(0);
        {
            py::gil_scoped_release rel;
            fin = s.run();
        }
        std::vector<double> t;
        for (auto& p : s.waveform) t.push_back(p.time);
        py::array_t<double> v = waveform_array(s.waveform);
        py::dict out;
        out["node_names"] = names; out["time"] = t; out["values"] = v; out["final"] = fin.voltages; out["stats"] = stats_dict(s.stats);
        py::dict nr;
        nr["total_iterations"] = s.engine().newton.stats.total_iterations; nr["linear_solves"] = s.engine().newton.stats.linear_solves;
        nr["failed"] = s.engine().newton.stats.failed_count; nr["be_fallbacks"] = s.engine().be_fallbacks;
        { auto& lu = s.engine().newton.linear.lu.stats;
          nr["lu_analyses"] = lu.analyses; nr["lu_refactors"] = lu.refactors; nr["lu_reuses"] = lu.reuses; nr["lu_repivots"] = lu.repivots;
          nr["lu_refinement_rounds"] = lu.refinement_rounds; nr["lu_factor_nnz"] = lu.factor_nnz; nr["lu_singletons"] = lu.singletons;
          nr["lu_fallbacks"] = s.engine().newton.linear.stats.lu_fallbacks; }
        nr["step_cuts"] = s.engine().step_cuts; nr["dc_gmin_stepping"] = s.engine().dc_gmin_stepping;
        nr["device_solves"] = s.engine().newton.linear.stats.device_solves; nr["krylov_iterations"] = s.engine().newton.linear.stats.krylov_iterations;
        nr["krylov_fallbacks"] = s.engine().newton.linear.stats.krylov_fallbacks; nr["cuda_error"] = s.engine().newton.linear.cuda_error;
        out["newton"] = nr;
        return out;
    }, py::arg("netlist_json"), py::arg("tstop"), py::arg("dt"), py::arg("reltol") = 1e-3, py::arg("solver") = "lu", py::arg("record_every") = 1,
       py::arg("predict_depth") = 5, py::arg("inject") = std::vector<std::tuple<uint32_t, double, std::vector<std::pair<uint64_t, double>>>>{},
       py::arg("rollbacks") = std::vector<double>{}, py::arg("adaptive") = false, py::arg("lte_reltol") = 2e-2, py::arg("max_step_factor") = 64.0,
       py::arg("record_nodes") = std::vector<std::string>{});

    m.def("dc_operating_point", [](const std::string& netlist_json) {
        SolverEngine e(Netlist::from_json(Json::parse(netlist_json)));
        PartitionState out(0);
        bool ok = e.solve_dc(e.seeded_state(), out);
        return py::make_tuple(ok, ok ? out.voltages : e.seeded_state().voltages);
    });

    // DC transfer curve: the voltage source between `node` and ground takes each of `values` in turn; every point starts
    // Newton from the previous solution (continuation), which is what carries a bistable or steep circuit along its curve.
    m.def("dc_sweep", [](const std::string& netlist_json, const std::string& node, std::vector<double> values) {
        Netlist base = Netlist::from_json(Json::parse(netlist_json));
        std::vector<std::string> names = base.names_or_default();
        auto lower = [](std::string v) { for (auto& c : v) c = char(std::tolower((unsigned char)c)); return v; };
        int idx = -1;
        for (size_t i = 0; i < names.size(); ++i) if (lower(names[i]) == lower(node)) idx = int(i) + 1;
        if (idx < 0) throw std::invalid_argument("dc_sweep: no net named '" + node + "'");
        int which = -1;
        double sign = 1.0;
        for (size_t k = 0; k < base.elements.size(); ++k) {
            const Element& e = base.elements[k];
            if (e.kind != Element::VSource) continue;
            if (e.a == idx && e.b == 0) { which = int(k); sign = 1.0; }
            else if (e.b == idx && e.a == 0) { which = int(k); sign = -1.0; }
        }
        if (which < 0) throw std::invalid_argument("dc_sweep: no voltage source between '" + node + "' and ground");
        const size_t n = size_t(base.num_nodes);
        py::array_t<double> out({values.size(), n});
        auto o = out.mutable_unchecked<2>();
        std::vector<bool> converged;
        std::vector<double> prev;
        {
            for (size_t p = 0; p < values.size(); ++p) {
                Netlist nl = base;
                nl.initial_conditions.clear();
                nl.elements[size_t(which)].source = SourceWaveform::make_dc(sign * values[p]);
                SolverEngine e(std::move(nl));
                PartitionState seed = e.seeded_state(), sol(0);
                if (!prev.empty()) {
                    for (size_t i = 0; i < prev.size() && i < seed.voltages.size(); ++i) seed.voltages[i] = prev[i];
                    seed.voltages[size_t(idx - 1)] = values[p];
                }
                bool ok = e.solve_dc(seed, sol);
                converged.push_back(ok);
                if (ok) prev = sol.voltages;
                for (size_t i = 0; i < n; ++i) o(p, i) = ok && i < sol.voltages.size() ? sol.voltages[i] : std::nan("");
            }
        }
        py::dict r;
        r["node_names"] = names; r["sweep"] = values; r["values"] = out; r["converged"] = converged;
        return r;
    }, py::arg("netlist_json"), py::arg("node"), py::arg("values"),
       "operating points over a swept source: {node_names, sweep, values[point, net], converged[point]}");

    m.def("simulate_partitioned", [](std::vector<std::string> parts_json, double tstop, double dt, double reltol, uint32_t predict_depth, bool compress,
                                     uint32_t record_every, unsigned threads, bool speculate) {
        std::vector<Netlist> parts;
        for (auto& js : parts_json) parts.push_back(Netlist::from_json(Json::parse(js)));
        PartitionedConfig cfg;
        cfg.tstop = tstop; cfg.dt = dt; cfg.reltol = reltol; cfg.predict_depth = predict_depth; cfg.compress = compress; cfg.record_every = std::max(1u, record_every); cfg.threads = threads; cfg.speculate = speculate;
        PartitionedRunner r(std::move(parts), cfg);
        {
            py::gil_scoped_release rel;
            r.run();
        }
        std::vector<double> t;
        for (auto& p : r.waveform) t.push_back(p.time);
        py::array_t<double> v = waveform_array(r.waveform);
        py::dict st;
        st["steps"] = r.stats.steps; st["prediction_hits"] = r.stats.prediction_hits; st["prediction_misses"] = r.stats.prediction_misses;
        st["resolves"] = r.stats.resolves; st["messages"] = r.stats.messages; st["bytes_sent"] = r.stats.bytes_sent; st["codec_ratio"] = r.stats.codec_ratio;
        st["completed"] = r.stats.completed; st["wall_time_secs"] = r.stats.wall_time_secs; st["unconverged_steps"] = r.stats.unconverged_steps;
        st["final_depth"] = r.stats.final_depth;
        st["windows"] = r.stats.windows; st["speculated_steps"] = r.stats.speculated_steps; st["discarded_steps"] = r.stats.discarded_steps;
        st["rollbacks"] = r.stats.rollbacks;
        py::dict out;
        out["node_names"] = r.names; out["time"] = t; out["values"] = v; out["stats"] = st;
        return out;
    }, py::arg("partitions"), py::arg("tstop"), py::arg("dt"), py::arg("reltol") = 1e-3, py::arg("predict_depth") = 5, py::arg("compress") = true,
       py::arg("record_every") = 1, py::arg("threads") = 1, py::arg("speculate") = true);

    // ---- linear algebra -----------------------------------------------------------------------
    m.def("solve_csr", [](int n, std::vector<int> row_ptr, std::vector<int> col, std::vector<double> val, std::vector<double> rhs, const std::string& solver) {
        CsrMatrix a(n);
        a.row_ptr = std::move(row_ptr); a.col = std::move(col); a.val = std::move(val); a.rhs = std::move(rhs);
        if (int(a.row_ptr.size()) != n + 1 || a.col.size() != a.val.size() || int(a.rhs.size()) != n) throw std::invalid_argument("inconsistent CSR arrays");
        LinearSolver s;
        s.backend = backend_of(solver);
        bool ok = s.solve(a);
        return py::make_tuple(ok, a.solution, s.stats.krylov_iterations);
    }, py::arg("n"), py::arg("row_ptr"), py::arg("col"), py::arg("val"), py::arg("rhs"), py::arg("solver") = "lu");
    py::class_<FactoredLU>(m, "FactoredLU", "sparse LU that keeps its ordering and pattern between solves of one sparsity pattern")
        .def(py::init<>())
        .def("solve", [](FactoredLU& lu, int n, const std::vector<int>& row_ptr, const std::vector<int>& col, const std::vector<double>& val,
                         const std::vector<double>& rhs) {
            if (int(row_ptr.size()) != n + 1 || col.size() != val.size() || int(rhs.size()) != n) throw std::invalid_argument("inconsistent CSR arrays");
            std::vector<double> x;
            bool ok = lu.solve(n, row_ptr, col, val, rhs, x);
            return py::make_tuple(ok, x);
        })
        .def("stats", [](const FactoredLU& lu) {
            py::dict d;
            d["orderings"] = lu.stats.orderings; d["analyses"] = lu.stats.analyses; d["refactors"] = lu.stats.refactors; d["reuses"] = lu.stats.reuses; d["repivots"] = lu.stats.repivots;
            d["refinement_rounds"] = lu.stats.refinement_rounds; d["factor_nnz"] = lu.stats.factor_nnz; d["singletons"] = lu.stats.singletons;
            return d;
        });
    m.def("singleton_pivots", [](int n, const std::vector<int>& row_ptr, const std::vector<int>& col) { return singleton_pivots(n, row_ptr, col); });
    m.def("minimum_degree_order", [](int n, const std::vector<int>& row_ptr, const std::vector<int>& col) { return minimum_degree_order(n, row_ptr, col); });
    m.def("csr_spmv", [](int n, std::vector<int> row_ptr, std::vector<int> col, std::vector<double> val, std::vector<double> x) {
        CsrMatrix a(n);
        a.row_ptr = std::move(row_ptr); a.col = std::move(col); a.val = std::move(val);
        return a.spmv(x);
    });
    m.def("mna_matrix", [](const std::string& netlist_json, double dt, double time, std::vector<double> guess) {
        Netlist nl = Netlist::from_json(Json::parse(netlist_json));
        Assembler as(nl);
        guess.resize(size_t(as.size), 0.0);
        as.stamp_linear(guess, {}, dt, time, Integration::BackwardEuler, {});
        as.stamp_nonlinear(guess);
        return py::make_tuple(as.size, as.m.row_ptr, as.m.col, as.m.val, as.m.rhs);
    }, py::arg("netlist_json"), py::arg("dt"), py::arg("time"), py::arg("guess") = std::vector<double>{});

    // ---- devices ------------------------------------------------------------------------------
    m.def("diode_eval", [](double vd, double is, double n, double vt) { DiodeModel d; d.is = is; d.n = n; d.vt = vt; double i, g; d.eval(vd, i, g); return py::make_tuple(i, g); },
          py::arg("vd"), py::arg("is_") = 1e-14, py::arg("n") = 1.0, py::arg("vt") = 0.02585);
    m.def("mosfet_eval", [](double vgs, double vds, bool pmos, double vth, double beta, double lambda) {
        MosfetLevel1 f; f.kind = pmos ? MosType::Pmos : MosType::Nmos; f.vth = vth; f.beta = beta; f.lambda = lambda;
        double id, gm, gds; MosRegion r;
        f.evaluate(vgs, vds, id, gm, gds, r);
        return py::make_tuple(id, gm, gds, r == MosRegion::Cutoff ? "Cutoff" : r == MosRegion::Linear ? "Linear" : "Saturation");
    }, py::arg("vgs"), py::arg("vds"), py::arg("pmos") = false, py::arg("vth") = 0.5, py::arg("beta") = 1e-3, py::arg("lambda_") = 0.1);

    // ---- prediction ---------------------------------------------------------------------------
    py::class_<GhostNode>(m, "GhostNode")
        .def(py::init<uint64_t, uint32_t>())
        .def("predict", &GhostNode::predict)
        .def("predict_named", [](const GhostNode& g, double t) { Prediction p = g.predict_named(t); return py::make_tuple(p.value, std::string(p.predictor)); })
        .def("apply_correction", &GhostNode::apply_correction)
        .def("signal_class", [](const GhostNode& g) { return std::string(class_name(classify_signal(g.signal))); })
        .def_readonly("confidence", &GhostNode::confidence)
        .def_readonly("gradient", &GhostNode::gradient)
        .def_readonly("last_known_voltage", &GhostNode::last_known_voltage);
    py::class_<AdaptiveConfidence>(m, "AdaptiveConfidence")
        .def(py::init<uint32_t>(), py::arg("base_depth") = 5)
        .def("update", &AdaptiveConfidence::update)
        .def("effective_depth", &AdaptiveConfidence::effective_depth)
        .def("confidence_for", &AdaptiveConfidence::confidence_for);
    py::class_<SpeculativeDepthController>(m, "SpeculativeDepthController")
        .def(py::init<uint32_t, uint32_t, uint32_t>())
        .def("record_prediction", &SpeculativeDepthController::record_prediction)
        .def("record_rollback", &SpeculativeDepthController::record_rollback)
        .def("depth", &SpeculativeDepthController::depth);

    // ---- codec --------------------------------------------------------------------------------
    m.def("codec_roundtrip", [](std::vector<std::pair<uint64_t, double>> updates, std::vector<std::pair<uint64_t, double>> predicted, int quant_bits) {
        ResidualCodec c;
        c.quant_bits = quant_bits;
        ResidualMessage msg;
        msg.from = 0; msg.to = 1; msg.time = 1e-9; msg.updates = std::move(updates);
        std::string bytes = c.encode_to_bytes(msg, predicted);
        ResidualMessage out;
        bool ok = c.decode_from_bytes(bytes, out);
        py::dict d;
        d["ok"] = ok; d["updates"] = out.updates; d["bytes"] = py::bytes(bytes); d["ratio"] = c.stats.compression_ratio(); d["skipped"] = c.stats.skipped;
        return d;
    }, py::arg("updates"), py::arg("predicted"), py::arg("quant_bits") = 16);
    m.def("fabric_selftest", [](uint32_t n, int rounds) {
        // every node sends one residual to every other node per round, from its own thread
        auto mesh = create_mesh(n);
        std::vector<std::thread> th;
        for (uint32_t i = 0; i < n; ++i)
            th.emplace_back([&, i] {
                for (int r = 0; r < rounds; ++r)
                    for (uint32_t j = 0; j < n; ++j)
                        if (j != i) { ResidualMessage msg; msg.from = i; msg.to = j; msg.time = r; msg.updates = {{uint64_t(i), double(r) + 0.5}}; mesh[i]->send_residual(msg, {{uint64_t(i), double(r)}}); }
                mesh[i]->broadcast_done();
            });
        for (auto& t : th) t.join();
        uint64_t residuals = 0, done = 0;
        double sum = 0;
        for (uint32_t i = 0; i < n; ++i)
            for (auto& fm : mesh[i]->drain_inbox()) {
                if (fm.kind == FabricMessage::Done) ++done;
                else if (fm.kind == FabricMessage::Residual) { ++residuals; for (auto& u : mesh[i]->decode_residual(fm.residual).updates) sum += u.second; }
            }
        return py::make_tuple(residuals, done, sum);
    });

    // ---- .nz ----------------------------------------------------------------------------------
    m.def("nz_compress", [](std::vector<std::string> names, std::vector<double> time, std::vector<std::vector<double>> signals, double error_bound) {
        NzWriter w(error_bound);
        std::string bytes = NzWriter::to_bytes(w.compress(names, time, signals));
        py::dict st;
        st["compression_ratio"] = w.stats.compression_ratio(); st["prediction_rate"] = w.stats.prediction_rate();
        st["predicted_blocks"] = w.stats.predicted_blocks; st["raw_blocks"] = w.stats.raw_blocks;
        return py::make_tuple(py::bytes(bytes), st);
    }, py::arg("names"), py::arg("time"), py::arg("signals"), py::arg("error_bound") = 1e-6);
    m.def("nz_decompress", [](const std::string& bytes) {
        NzFile f = NzReader::from_bytes(bytes);
        py::dict h;
        h["version"] = f.version; h["t_start"] = f.t_start; h["t_end"] = f.t_end; h["error_bound"] = f.error_bound; h["num_blocks"] = f.blocks.size();
        return py::make_tuple(f.names, f.time, NzReader::decompress(f), h);
    });

    // ---- PVT ----------------------------------------------------------------------------------
    m.def("pvt_delta", [](std::vector<double> time, std::vector<std::vector<double>> golden, const std::string& process, double vdd, double temp) {
        GoldenTrajectory g(CornerSpec(), time.size() > 1 ? time[1] - time[0] : 0.0);
        for (size_t k = 0; k < time.size(); ++k) g.push(time[k], golden[k]);
        std::string bytes = g.to_bytes();
        GoldenTrajectory back;
        bool rt = GoldenTrajectory::from_bytes(bytes, g.corner, back) && back.points.size() == g.points.size();
        DeltaSolver s(std::move(g));
        CornerSpec c(corner_from_name(process), vdd, temp);
        DeltaSolveResult r = s.solve_corner(c);
        std::vector<std::vector<double>> rec;
        for (auto& p : s.reconstruct(r)) rec.push_back(p.voltages);
        py::dict d;
        d["name"] = c.name; d["used_delta_mode"] = r.used_delta_mode; d["peak_delta_v"] = r.peak_delta_v; d["waveform"] = rec; d["bytes_roundtrip"] = rt;
        return d;
    });
    // The golden run is handed over once; every corner after that is one call with three numbers.
    py::class_<DeltaSolver>(m, "PvtDeltaSolver", "delta reconstruction of corner waveforms from one golden run")
        .def(py::init([](const std::vector<double>& time, py::array_t<double, py::array::c_style | py::array::forcecast> golden) {
            if (golden.ndim() != 2 || size_t(golden.shape(0)) != time.size()) throw std::invalid_argument("golden must be (len(time), nets)");
            GoldenTrajectory g(CornerSpec(), time.size() > 1 ? time[1] - time[0] : 0.0);
            const py::ssize_t cols = golden.shape(1);
            const double* src = golden.data();
            for (size_t k = 0; k < time.size(); ++k) g.push(time[k], std::vector<double>(src + py::ssize_t(k) * cols, src + (py::ssize_t(k) + 1) * cols));
            return new DeltaSolver(std::move(g));
        }), py::arg("time"), py::arg("golden"))
        .def("solve", [](DeltaSolver& s, const std::string& process, double vdd, double temp, bool want_waveform) {
            CornerSpec c(corner_from_name(process), vdd, temp);
            DeltaSolveResult r = s.solve_corner(c);
            py::dict d;
            d["name"] = c.name; d["used_delta_mode"] = r.used_delta_mode; d["peak_delta_v"] = r.peak_delta_v;
            if (want_waveform) {
                std::vector<WaveformPoint> w;
                for (auto& p : s.reconstruct(r)) w.push_back({p.time, std::move(p.voltages)});
                d["waveform"] = waveform_array(w);
            }
            return d;
        }, py::arg("process"), py::arg("vdd"), py::arg("temp"), py::arg("want_waveform") = true)
        .def("stats", [](const DeltaSolver& s) {
            py::dict d;
            d["corners_solved"] = s.stats.corners_solved; d["delta_mode_used"] = s.stats.delta_mode_used; d["full_sim_fallback"] = s.stats.full_sim_fallback;
            d["total_wall_time"] = s.stats.total_wall_time;
            return d;
        });
    m.def("pvt_cache_selftest", [](size_t cap, std::vector<std::string> inserts, std::vector<std::string> lookups) {
        PvtCache c(cap);
        for (auto& n : inserts) { GoldenTrajectory g; g.corner.name = n; c.insert(std::move(g)); }
        std::vector<bool> found;
        for (auto& n : lookups) found.push_back(c.get(n) != nullptr);
        return py::make_tuple(found, c.size(), c.stats.hits, c.stats.misses, c.stats.evictions);
    });

    // ---- balancer / benchmarks ----------------------------------------------------------------
    m.def("balance_plan", [](std::vector<std::tuple<uint32_t, uint32_t, std::vector<double>>> partitions) {
        // (partition id, element count, step times) -> (stragglers, plans, score)
        BalanceMonitor mon{uint32_t(partitions.size())};
        mon.check_interval = 1;
        for (size_t i = 0; i < partitions.size(); ++i) {
            mon.metrics[i].partition_id = std::get<0>(partitions[i]);
            mon.metrics[i].element_count = std::get<1>(partitions[i]);
            for (double t : std::get<2>(partitions[i])) mon.metrics[i].record_solve_time(t);
        }
        std::vector<std::pair<uint32_t, double>> st;
        for (auto& s : detect_stragglers(mon.metrics, mon.detector)) st.emplace_back(s.partition, s.ratio);
        std::vector<std::tuple<uint32_t, uint32_t, uint32_t, double>> plans;
        for (auto& p : mon.check_balance()) plans.emplace_back(p.from_partition, p.to_partition, p.elements_to_move, p.expected_speedup);
        return py::make_tuple(st, plans, mon.balance_score());
    });
    m.def("generate_circuit", [](const std::string& kind, int a, int b, double r, double c) {
        if (kind == "rc_ladder") return generate_rc_ladder(a, r, c).to_json().dump();
        if (kind == "cim_array") return generate_cim_array(a, b).to_json().dump();
        if (kind == "resistor_mesh") return generate_resistor_mesh(a, r).to_json().dump();
        throw std::invalid_argument("kind must be rc_ladder, cim_array or resistor_mesh");
    }, py::arg("kind"), py::arg("a"), py::arg("b") = 0, py::arg("r") = 1e3, py::arg("c") = 10e-15);
    m.def("run_benchmark_suite", [](int scale) {
        std::vector<py::dict> out;
        for (auto& r : run_benchmark_suite(scale)) {
            py::dict d;
            d["name"] = r.name; d["num_nodes"] = r.num_nodes; d["num_elements"] = r.num_elements; d["steps"] = r.steps; d["wall_time_secs"] = r.wall_time_secs;
            d["steps_per_sec"] = r.steps_per_sec; d["completed"] = r.completed; d["summary"] = r.summary();
            out.push_back(d);
        }
        return out;
    }, py::arg("scale") = 1);
}
