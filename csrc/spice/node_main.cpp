// nangila-node: solver process of one partition.
//
//   nangila-node --partition deck.sp|part.json [--node-id N] [-k TOTAL] [--predict-depth D]
//                [--reltol R] [--tstop T] [--dt DT] [--process TT|FF|SS|FS|SF] [--vdd V] [--temp C]
//                [--waveform-json out.json] [--waveform-nz out.nz] [--solver lu|dense|krylov|cuda]
//                [--record-every K] [--record-nodes A,B,...] [--adaptive] [--demo]
//                [--rendezvous DIR [--bind HOST] [--connect-timeout-ms T] [--io-timeout-ms T]]
//
// With --rendezvous and -k > 1 the process is one of TOTAL that advance in lockstep and exchange boundary voltages
// over TCP (distributed.hpp); its waveform file then holds the nets this partition owns. DIR must be empty of earlier
// runs' address files; the processes must run on machines of one byte order.
//
// Flag set and the waveform JSON layout ({netlist, node_names, waveform: [{time, voltages{}}],
// stats{}}) follow the reference's CLI (nangila-spice/nangila-node/src/main.rs:21-132).
#include <algorithm>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <iostream>

#include "balancer.hpp"
#include "distributed.hpp"
#include "nz.hpp"
#include "parser.hpp"
#include "partitioned.hpp"
#include "transient.hpp"

using namespace nspice;

struct Args {
    std::string partition, partitions, process = "TT", waveform_json, waveform_nz, solver = "lu", rendezvous, bind_host = "127.0.0.1";
    int connect_timeout_ms = 30000, io_timeout_ms = 30000;
    uint32_t node_id = 0, total = 1, predict_depth = 5, record_every = 1, threads = 1;
    double reltol = 1e-3, tstop = 1e-6, dt = 1e-12, vdd = 1.8, temp = 27.0, nz_tol = 1e-6;
    std::string record_nodes;                    // comma-separated net names: the waveform keeps these only (single partition)
    bool tstop_given = false, dt_given = false;  // a deck's `.tran` card fills in whichever was not given
    bool demo = false, bench = false, lockstep = false, adaptive = false;
};

static void usage() {
    std::fprintf(stderr,
                 "usage: nangila-node [--partition FILE | --demo] [--node-id N] [-k TOTAL] [--predict-depth D]\n"
                 "                    [--reltol R] [--tstop T] [--dt DT] [--process P] [--vdd V] [--temp C]\n"
                 "                    [--waveform-json OUT] [--waveform-nz OUT] [--nz-tol E] [--solver lu|dense|krylov|cuda]\n"
                 "                    [--record-every K] [--record-nodes A,B,...] [--adaptive] [--partitions A.json,B.json,... [--threads T]] [--bench]\n"
                 "                    [--rendezvous DIR [--bind HOST] [--connect-timeout-ms T] [--io-timeout-ms T] [--lockstep]]\n");
}

static bool parse_args(int argc, char** argv, Args& a) {
    for (int i = 1; i < argc; ++i) {
        std::string f = argv[i];
        auto need = [&](const char* name) -> const char* {
            if (i + 1 >= argc) { std::fprintf(stderr, "missing value for %s\n", name); return nullptr; }
            return argv[++i];
        };
        const char* v = nullptr;
        if (f == "--demo") a.demo = true;
        else if (f == "--bench") a.bench = true;
        else if (f == "--lockstep") a.lockstep = true;
        else if (f == "--adaptive") a.adaptive = true;
        else if (f == "--record-nodes") { if (!(v = need("--record-nodes"))) return false; a.record_nodes = v; }
        else if (f == "--partitions") { if (!(v = need("--partitions"))) return false; a.partitions = v; }
        else if (f == "-h" || f == "--help") { usage(); std::exit(0); }
        else if (f == "--partition" || f == "-p") { if (!(v = need("--partition"))) return false; a.partition = v; }
        else if (f == "--node-id" || f == "-n") { if (!(v = need("--node-id"))) return false; a.node_id = uint32_t(std::atoi(v)); }
        else if (f == "-k" || f == "--total-partitions") { if (!(v = need("-k"))) return false; a.total = uint32_t(std::atoi(v)); }
        else if (f == "--predict-depth") { if (!(v = need("--predict-depth"))) return false; a.predict_depth = uint32_t(std::atoi(v)); }
        else if (f == "--threads") { if (!(v = need("--threads"))) return false; a.threads = uint32_t(std::max(1, std::atoi(v))); }
        else if (f == "--record-every") { if (!(v = need("--record-every"))) return false; a.record_every = std::max(1, std::atoi(v)); }
        else if (f == "--reltol") { if (!(v = need("--reltol"))) return false; a.reltol = std::atof(v); }
        else if (f == "--tstop") { if (!(v = need("--tstop"))) return false; a.tstop = std::atof(v); a.tstop_given = true; }
        else if (f == "--dt") { if (!(v = need("--dt"))) return false; a.dt = std::atof(v); a.dt_given = true; }
        else if (f == "--vdd") { if (!(v = need("--vdd"))) return false; a.vdd = std::atof(v); }
        else if (f == "--temp") { if (!(v = need("--temp"))) return false; a.temp = std::atof(v); }
        else if (f == "--nz-tol") { if (!(v = need("--nz-tol"))) return false; a.nz_tol = std::atof(v); }
        else if (f == "--process") { if (!(v = need("--process"))) return false; a.process = v; }
        else if (f == "--solver") { if (!(v = need("--solver"))) return false; a.solver = v; }
        else if (f == "--waveform-json") { if (!(v = need("--waveform-json"))) return false; a.waveform_json = v; }
        else if (f == "--rendezvous") { if (!(v = need("--rendezvous"))) return false; a.rendezvous = v; }
        else if (f == "--bind") { if (!(v = need("--bind"))) return false; a.bind_host = v; }
        else if (f == "--connect-timeout-ms") { if (!(v = need("--connect-timeout-ms"))) return false; a.connect_timeout_ms = std::atoi(v); }
        else if (f == "--io-timeout-ms") { if (!(v = need("--io-timeout-ms"))) return false; a.io_timeout_ms = std::atoi(v); }
        else if (f == "--waveform-nz") { if (!(v = need("--waveform-nz"))) return false; a.waveform_nz = v; }
        else { std::fprintf(stderr, "unknown flag %s\n", f.c_str()); return false; }
    }
    return true;
}

static Netlist demo_netlist() {
    Netlist n;
    n.name = "RC Demo";
    n.num_nodes = 2;
    n.elements = {Element::vsource(1, 0, SourceWaveform::make_dc(1.8)), Element::resistor(1, 2, 1000.0), Element::capacitor(2, 0, 10e-15)};
    n.node_names = {"vdd", "cap"};
    // start from a discharged capacitor so the demo shows the charging curve
    n.initial_conditions = {{1, 1.8}, {2, 0.0}};
    return n;
}

static void write_json(const std::string& path, const std::string& name, const std::vector<std::string>& names,
                       const std::vector<WaveformPoint>& wf, const SimStats& st) {
    std::ofstream f(path);
    if (!f) throw std::runtime_error("cannot write '" + path + "'");
    // streamed by hand: a waveform can hold millions of points
    f << "{\n  \"netlist\": " << Json(name).dump() << ",\n  \"node_names\": [";
    for (size_t i = 0; i < names.size(); ++i) f << (i ? ", " : "") << Json(names[i]).dump();
    f << "],\n  \"waveform\": [";
    char buf[64];
    for (size_t p = 0; p < wf.size(); ++p) {
        std::snprintf(buf, sizeof buf, "%.17g", wf[p].time);
        f << (p ? ",\n    " : "\n    ") << "{\"time\": " << buf << ", \"voltages\": {";
        size_t n = std::min(names.size(), wf[p].values.size());
        for (size_t i = 0; i < n; ++i) {
            std::snprintf(buf, sizeof buf, "%.17g", wf[p].values[i]);
            f << (i ? ", " : "") << Json(names[i]).dump() << ": " << buf;
        }
        f << "}}";
    }
    f << "\n  ],\n  \"stats\": {\"total_steps\": " << st.total_steps;
    std::snprintf(buf, sizeof buf, "%.9g", st.wall_time_secs);
    f << ", \"wall_time_secs\": " << buf << ", \"prediction_hits\": " << st.prediction_hits << ", \"prediction_misses\": "
      << st.prediction_misses << ", \"rollbacks\": " << st.rollbacks << ", \"completed\": " << (st.completed ? "true" : "false") << "}\n}\n";
}

static void write_nz(const std::string& path, const std::vector<std::string>& names, const std::vector<WaveformPoint>& wf, double tol) {
    std::vector<double> t;
    std::vector<std::vector<double>> sig(names.size());
    for (auto& p : wf) {
        t.push_back(p.time);
        for (size_t i = 0; i < names.size(); ++i) sig[i].push_back(i < p.values.size() ? p.values[i] : 0.0);
    }
    NzWriter w(tol);
    w.write_file(path, names, t, sig);
}

static Netlist load_any(const std::string& path, const Args& a) {
    std::ifstream f(path);
    if (!f) throw std::runtime_error("cannot open '" + path + "'");
    std::stringstream ss;
    ss << f.rdbuf();
    if (path.size() > 5 && path.substr(path.size() - 5) == ".json") return Netlist::from_json(Json::parse(ss.str()));
    Corner c;
    c.process = a.process; c.vdd = a.vdd; c.temp_c = a.temp;
    SpiceParser p(c);
    p.follow_includes_from(SpiceParser::directory_of(path), path);
    return p.parse_text(ss.str(), path.substr(path.find_last_of('/') == std::string::npos ? 0 : path.find_last_of('/') + 1));
}

// All partitions of a design in one process: --partitions p0.json,p1.json,...
static int run_partitioned(const Args& a) {
    std::vector<Netlist> parts;
    try {
        size_t pos = 0;
        while (pos <= a.partitions.size()) {
            size_t comma = a.partitions.find(',', pos);
            std::string one = a.partitions.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
            if (!one.empty()) parts.push_back(load_any(one, a));
            if (comma == std::string::npos) break;
            pos = comma + 1;
        }
        PartitionedConfig cfg;
        cfg.tstop = a.tstop; cfg.dt = a.dt; cfg.reltol = a.reltol; cfg.predict_depth = a.predict_depth; cfg.record_every = a.record_every;
        cfg.threads = a.threads;
        if (a.threads > 1) cfg.min_unknowns_per_thread = 0;   // --threads was asked for: take it literally
        cfg.speculate = !a.lockstep;
        PartitionedRunner runner(std::move(parts), cfg);
        runner.run();
        const PartitionedStats& st = runner.stats;
        std::fprintf(stderr, "partitioned run: %llu steps%s, %.3f s, hits %llu, misses %llu, extra solves %llu, messages %llu (%llu bytes, codec ratio %.2f), depth %u\n",
                     (unsigned long long)st.steps, st.completed ? "" : " (stopped early)", st.wall_time_secs, (unsigned long long)st.prediction_hits,
                     (unsigned long long)st.prediction_misses, (unsigned long long)st.resolves, (unsigned long long)st.messages,
                     (unsigned long long)st.bytes_sent, st.codec_ratio, st.final_depth);
        SimStats ss;
        ss.total_steps = st.steps; ss.wall_time_secs = st.wall_time_secs; ss.prediction_hits = st.prediction_hits;
        ss.prediction_misses = st.prediction_misses; ss.rollbacks = st.resolves; ss.completed = st.completed;
        if (!a.waveform_json.empty()) write_json(a.waveform_json, "partitioned", runner.names, runner.waveform, ss);
        if (!a.waveform_nz.empty()) write_nz(a.waveform_nz, runner.names, runner.waveform, a.nz_tol);
        return st.completed ? 0 : 3;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ERROR: %s\n", e.what());
        return 1;
    }
}

// One of several processes of a partitioned run: --partition part.json --node-id N -k TOTAL --rendezvous DIR
static int run_distributed(const Args& a) {
    try {
        Netlist nl = load_any(a.partition, a);
        std::string name = nl.name;
        SocketMesh mesh(a.node_id, a.total, a.rendezvous, a.bind_host);
        if (!mesh.connect_all(a.connect_timeout_ms)) { std::fprintf(stderr, "ERROR: process %u: %s\n", a.node_id, mesh.error.c_str()); return 4; }
        DistributedConfig cfg;
        cfg.tstop = a.tstop; cfg.dt = a.dt; cfg.reltol = a.reltol; cfg.predict_depth = a.predict_depth; cfg.record_every = a.record_every;
        cfg.io_timeout_ms = a.io_timeout_ms;
        cfg.speculate = !a.lockstep;
        DistributedRunner runner(std::move(nl), mesh, cfg);
        runner.engine().newton.config.reltol = a.reltol;
        if (a.solver == "dense") runner.engine().newton.linear.backend = LinearBackend::Dense;
        else if (a.solver == "krylov") runner.engine().newton.linear.backend = LinearBackend::Krylov;
        const bool ok = runner.run();
        const DistributedStats& st = runner.stats;
        std::fprintf(stderr, "process %u of %u: %llu steps%s, %.3f s, %llu DC sweeps, %llu windows (%llu steps ahead, %llu discarded), hits %llu, misses %llu, extra solves %llu, %llu messages (%llu bytes)%s%s\n",
                     a.node_id, a.total, (unsigned long long)st.steps, ok ? "" : " (stopped early)", st.wall_time_secs, (unsigned long long)st.dc_sweeps,
                     (unsigned long long)st.windows, (unsigned long long)st.speculated_steps, (unsigned long long)st.discarded_steps,
                     (unsigned long long)st.prediction_hits, (unsigned long long)st.prediction_misses, (unsigned long long)st.resolves,
                     (unsigned long long)mesh.stats.messages_sent, (unsigned long long)mesh.stats.bytes_sent, st.error.empty() ? "" : ": ", st.error.c_str());
        SimStats ss;
        ss.total_steps = st.steps; ss.wall_time_secs = st.wall_time_secs; ss.prediction_hits = st.prediction_hits;
        ss.prediction_misses = st.prediction_misses; ss.rollbacks = st.resolves; ss.completed = ok;
        if (!a.waveform_json.empty()) write_json(a.waveform_json, name, runner.names, runner.waveform, ss);
        if (!a.waveform_nz.empty()) write_nz(a.waveform_nz, runner.names, runner.waveform, a.nz_tol);
        // 3: this partition's solve failed; 5: the run stopped because of a peer or the network
        return ok ? 0 : (st.error.find("Newton") != std::string::npos ? 3 : 5);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ERROR: process %u: %s\n", a.node_id, e.what());
        return 1;
    }
}

static int run(int argc, char** argv);

int main(int argc, char** argv) {
    try {
        return run(argc, argv);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ERROR: %s\n", e.what());
        return 1;
    }
}

static int run(int argc, char** argv) {
    Args a;
    if (!parse_args(argc, argv, a)) { usage(); return 2; }
    if (a.bench) {
        for (auto& r : run_benchmark_suite()) std::printf("%s\n", r.summary().c_str());
        return 0;
    }
    if (!a.partitions.empty()) return run_partitioned(a);
    if (!a.rendezvous.empty() && a.total > 1) {
        if (a.partition.empty()) { std::fprintf(stderr, "--rendezvous needs --partition FILE\n"); return 2; }
        return run_distributed(a);
    }
    Netlist nl;
    try {
        if (a.demo) nl = demo_netlist();
        else if (a.partition.empty()) { std::fprintf(stderr, "nothing to do: give --partition FILE or --demo\n"); return 0; }
        else if (a.partition.size() > 5 && a.partition.substr(a.partition.size() - 5) == ".json") {
            std::ifstream f(a.partition);
            if (!f) throw std::runtime_error("cannot open '" + a.partition + "'");
            std::stringstream ss;
            ss << f.rdbuf();
            nl = Netlist::from_json(Json::parse(ss.str()));
        } else {
            Corner c;
            c.process = a.process; c.vdd = a.vdd; c.temp_c = a.temp;
            SpiceParser p(c);
            std::ifstream f(a.partition);
            if (!f) throw std::runtime_error("cannot open '" + a.partition + "'");
            std::stringstream ss;
            ss << f.rdbuf();
            std::string base = a.partition.substr(a.partition.find_last_of('/') == std::string::npos ? 0 : a.partition.find_last_of('/') + 1);
            p.follow_includes_from(SpiceParser::directory_of(a.partition), a.partition);
            nl = p.parse_text(ss.str(), base);
            if (!a.tstop_given && p.tran_stop > 0.0) a.tstop = p.tran_stop;
            if (!a.dt_given && p.tran_step > 0.0) a.dt = p.tran_step;
            for (auto& w : p.warnings) std::fprintf(stderr, "warning: %s\n", w.c_str());
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ERROR: failed to load netlist '%s': %s\n", a.partition.c_str(), e.what());
        return 1;
    }
    std::fprintf(stderr, "nangila-node %u of %u: '%s', %d nodes, %zu elements, %zu ghost nodes\n", a.node_id, a.total, nl.name.c_str(),
                 nl.num_nodes, nl.elements.size(), nl.ghost_map.size());
    GhostBuffer ghosts(a.predict_depth);
    for (auto& g : nl.ghost_map) ghosts.add(GhostNode(g.net_id, g.owner));
    SimConfig cfg;
    cfg.tstop = a.tstop; cfg.dt = a.dt; cfg.reltol = a.reltol; cfg.predict_depth = a.predict_depth; cfg.record_every = a.record_every;
    cfg.adaptive = a.adaptive;   // variable internal step, waveform still on the dt grid (single partition only)
    std::vector<std::string> names = nl.names_or_default();
    const std::vector<std::string> all_names = names;
    if (!a.record_nodes.empty()) {
        // the waveform keeps the named nets only (compared without case; names the deck does not have are skipped)
        auto lower = [](std::string v) { for (auto& c : v) c = char(std::tolower((unsigned char)c)); return v; };
        std::vector<std::string> kept;
        std::stringstream list(a.record_nodes);
        std::string want;
        while (std::getline(list, want, ',')) {
            for (uint32_t i = 0; i < names.size(); ++i)
                if (lower(names[i]) == lower(want) && std::find(cfg.record_nodes.begin(), cfg.record_nodes.end(), i) == cfg.record_nodes.end()) {
                    cfg.record_nodes.push_back(i);
                    kept.push_back(names[i]);
                    break;
                }
        }
        if (cfg.record_nodes.empty()) std::fprintf(stderr, "warning: --record-nodes names no net of this deck; the waveform keeps all of them\n");
        else names = kept;
    }
    std::string name = nl.name;
    TransientSolver solver(std::move(nl), std::move(ghosts), CommLayer(a.node_id, a.total), cfg);
    solver.engine().newton.config.reltol = a.reltol;
    if (a.solver == "dense") solver.engine().newton.linear.backend = LinearBackend::Dense;
    else if (a.solver == "krylov") solver.engine().newton.linear.backend = LinearBackend::Krylov;
    else if (a.solver == "cuda") {
        // the kernel library: $NANGILA_KERNELS_LIB, else the in-tree build next to this executable's package
        if (!std::getenv("NANGILA_KERNELS_LIB")) {
            char buf[4096];
            ssize_t len = readlink("/proc/self/exe", buf, sizeof buf - 1);
            if (len > 0) {
                std::string exe(buf, size_t(len));
                size_t cut = exe.rfind("/nangila_spice/bin/");
                if (cut != std::string::npos) CudaKrylov::set_library(exe.substr(0, cut) + "/nangila/libnangila_kernels.so");
            }
        }
        solver.engine().newton.linear.backend = LinearBackend::Cuda;
    }
    PartitionState fin = solver.run();
    const SimStats& st = solver.stats;
    std::fprintf(stderr, "steps %llu%s, wall %.3f s, NR iterations/step %.2f, hit rate %.1f%%, rollbacks %llu\n",
                 (unsigned long long)st.total_steps, st.completed ? "" : " (stopped early: Newton did not converge)", st.wall_time_secs,
                 st.total_steps ? double(solver.engine().newton.stats.total_iterations) / double(st.total_steps) : 0.0, st.hit_rate() * 100.0,
                 (unsigned long long)st.rollbacks);
    if (a.solver == "cuda") {
        const auto& ls = solver.engine().newton.linear;
        std::fprintf(stderr, "device linear solver: %llu solves on the GPU, %llu fell back to the sparse LU%s\n", (unsigned long long)ls.stats.device_solves,
                     (unsigned long long)ls.stats.krylov_fallbacks, ls.cuda_error ? " (kernel library not usable: every solve ran on the host)" : "");
    }
    for (size_t i = 0; i < all_names.size() && i < fin.voltages.size() && i < 16; ++i) std::fprintf(stderr, "  V(%s) = %.6f\n", all_names[i].c_str(), fin.voltages[i]);
    try {
        if (!a.waveform_json.empty()) write_json(a.waveform_json, name, names, solver.waveform, st);
        if (!a.waveform_nz.empty()) write_nz(a.waveform_nz, names, solver.waveform, a.nz_tol);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ERROR: %s\n", e.what());
        return 1;
    }
    return st.completed ? 0 : 3;
}
