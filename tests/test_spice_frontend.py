"""CPU tests of the circuit simulator's Python front end: text-level parser, circuit graph,
partitioner, in-process and process-per-partition runs, merging, correctness contract, PVT sweep,
.nz reader, gate-level synthesis, report and command line. Plan modelled on the reference's
``nangila-spice/src/tests`` suites (partitioner, integration, correctness, PVT orchestrator)."""
import json
import time
import math
import os
import subprocess
import sys

import numpy as np
import pytest

pytest.importorskip("nangila_spice._native")

import nangila_spice as ns  # noqa: E402
from nangila_spice import _native as N  # noqa: E402
from nangila_spice.benchmark import generate_cim_netlist, generate_rc_ladder_netlist, run_scaling_study  # noqa: E402
from nangila_spice.parser import parse_netlist_text  # noqa: E402
from nangila_spice.partitioner import partition_flat  # noqa: E402

LATCH = """* cross-coupled inverters plus a passive tail
VDD vdd 0 DC 1.8
M1 q qb vdd vdd pch w=2u l=180n
M2 q qb 0 0 nch w=1u l=180n
M3 qb q vdd vdd pch w=2u l=180n
M4 qb q 0 0 nch w=1u l=180n
R1 q t1 20k
C1 t1 0 5f
R2 t1 t2 1k
C2 t2 0 5f
R3 t2 t3 1k
C3 t3 0 5f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
.ic V(q)=1.8 V(qb)=0 V(t1)=0 V(t2)=0 V(t3)=0
.end
"""


def _write(tmp_path, name, text):
    p = tmp_path / name
    p.write_text(text)
    return str(p)


def test_text_parser_and_flatten():
    nl = parse_netlist_text("""title
.global vdd
.subckt inv a y
M1 y a vdd vdd pch w=2u l=180n
M2 y a 0 0 nch
.ends
X1 in mid inv
X2 mid out inv
R1 out 0 10k
C1 out 0 1f
""")
    assert nl.title == "title" and nl.num_devices == 4 and "INV" in nl.subcircuits and nl.global_nodes == {"vdd"}
    flat = nl.flatten()
    assert [d.name for d in flat.devices] == ["X1.M1", "X1.M2", "X2.M1", "X2.M2", "R1", "C1"]   # names keep their case
    assert flat.devices[0].nodes == ["mid", "in", "vdd", "vdd"] and flat.devices[0].params == {"w": "2u", "l": "180n"}
    assert flat.devices[2].nodes[0] == "out" and flat.devices[1].model == "nch"
    assert flat.num_nodes == 5  # in, mid, out, vdd, 0
    with pytest.raises(FileNotFoundError):
        ns.parse_netlist("/nonexistent/deck.sp")


def test_circuit_graph_and_feedback_detection():
    nl = parse_netlist_text(LATCH)
    cg = ns.build_circuit_graph(nl)
    assert cg.num_devices == 11 and cg.num_nets == 7 and cg.num_edges > 20
    assert len(cg.feedback_groups) == 1 and cg.feedback_groups[0] == {"M1", "M2", "M3", "M4"}
    assert cg.graph["D:M1"]["N:qb"]["weight"] == 10 and cg.graph["D:M1"]["N:vdd"]["weight"] == 2  # source + bulk on the supply
    ladder = ns.build_circuit_graph(parse_netlist_text(generate_rc_ladder_netlist(20)))
    assert ladder.feedback_groups == []


@pytest.mark.parametrize("method", ["spectral", "bisect"])
def test_partitioner_properties(method):
    flat = json.loads(N.generate_circuit("rc_ladder", 63))
    res = partition_flat(flat, 4, method)
    assert len(res.partitions) == 4 and res.method == method
    owned = [p.internal_nodes for p in res.partitions]
    assert sum(len(o) for o in owned) == 63 and len(set().union(*owned)) == 63  # node_1 is held by the source and replicated
    assert max(len(o) for o in owned) - min(len(o) for o in owned) <= 2
    assert res.total_cut_edges == 3 and res.total_boundary_nodes == 6  # a chain cut three times
    assert 1.0 <= res.balance_ratio < 1.15
    for p in res.partitions:
        nl = p.netlist
        assert nl["num_nodes"] == len(nl["node_names"]) == len(p.internal_nodes) + len(p.boundary_nodes) + (1 if "node_1" in nl["node_names"] else 0)
        for net_id, local, owner in nl["ghost_map"]:
            name = nl["node_names"][local - 1]
            assert net_id == N.net_name_hash(name) and name in res.partitions[owner].internal_nodes
    assert "Partitions: 4" in res.summary()
    with pytest.raises(ValueError):
        partition_flat(flat, 0)
    assert len(partition_flat(flat, 1).partitions) == 1


def test_partitioner_keeps_feedback_loop_together(tmp_path):
    res = ns.partition_netlist(ns.parse_netlist(_write(tmp_path, "latch.sp", LATCH)), 2, "spectral")
    assert res.feedback_groups_enforced == 1
    assert res.net_assignment["q"] == res.net_assignment["qb"]
    assert {"M1", "M2", "M3", "M4"} <= set(res.partitions[res.net_assignment["q"]].device_names)


@pytest.mark.parametrize("k", [2, 3, 5])
def test_partitioned_run_matches_single_matrix(tmp_path, k):
    path = _write(tmp_path, "ladder.sp", generate_rc_ladder_netlist(40, 1e3, 10e-15))
    res = ns.simulate(path, partitions=k, tstop=300e-12, dt=1e-12, method="bisect")
    assert res.success and res.validation_status == "partitioned_validated", res.summary()
    assert res.reference_comparison.max_abs_error < 5e-5 and len(res.partition_result.partitions) == k  # accepted predictions are within 0.25e-3 relative
    assert res.waveform.num_nodes == 41 and res.waveform.num_points == 301
    st = res.solver_stats["stats"]
    assert st["messages"] > 0 and st["codec_ratio"] > 1.0 and st["unconverged_steps"] == 0
    assert "partitioned_validated" in res.summary()


def test_partitioned_nonlinear_latch_with_tail(tmp_path):
    res = ns.simulate(_write(tmp_path, "latch.sp", LATCH), partitions=2, tstop=200e-12, dt=0.5e-12, method="spectral")
    assert res.success and res.validation_status == "partitioned_validated", res.summary()
    assert res.waveform.voltage("q", 200e-12) > 1.6 and res.waveform.voltage("t3", 200e-12) > 0.5
    assert res.waveform.voltage("nope", 0.0) is None and res.waveform.voltage("q", 1.0) is None


def test_single_partition_exports_and_processes_mode(tmp_path):
    path = _write(tmp_path, "cim.sp", generate_cim_netlist(4, 4))
    out = tmp_path / "out"
    res = ns.simulate(path, partitions=1, tstop=1e-9, dt=5e-12, output_dir=str(out), output_format="csv")
    assert res.success and res.validation_status == "validated_single_node"
    rows = (out / "cim.csv").read_text().splitlines()
    assert rows[0].split(",")[0] == "time" and len(rows) == 202
    ns.export_json(res.waveform, str(out / "w.json"))
    assert json.loads((out / "w.json").read_text())["num_points"] == 201
    # one solver process per partition
    res2 = ns.simulate(path, partitions=2, tstop=1e-9, dt=5e-12, mode="processes", method="bisect")
    assert res2.success and res2.validation_status == "partitioned_validated", res2.summary()
    assert res2.reference_comparison is not None and res2.reference_comparison.max_abs_error < 1e-6


def test_merge_prefers_owner_over_ghost_copy():
    from nangila_spice.merger import PartitionWaveform, merge_waveforms

    a = PartitionWaveform(0, [0.0, 1.0, 2.0], {"x": [0.0, 1.0, 2.0], "g": [9.0, 9.0, 9.0]}, {"g"})
    b = PartitionWaveform(1, [0.0, 2.0], {"g": [0.0, 4.0], "y": [1.0, 3.0]}, set())
    w = merge_waveforms([a, b])
    assert w.node_names == ["x", "g", "y"] or set(w.node_names) == {"x", "g", "y"}
    assert w.traces["g"].tolist() == [0.0, 2.0, 4.0] and w.traces["y"].tolist() == [1.0, 2.0, 3.0]
    assert w.time_range == (0.0, 2.0) and w.voltage("x", 0.5) == 0.5 and len(w.points) == 3


def test_correctness_contract():
    t = np.linspace(0, 1e-9, 101)
    ref = ns.WaveformData("ref", "", ["a"], t.tolist(), {"a": (1.8 * t / 1e-9).tolist()})
    good = ns.WaveformData("c", "", ["a"], t.tolist(), {"a": (1.8 * t / 1e-9 + 2e-4).tolist()})
    late = ns.WaveformData("c", "", ["a"], t.tolist(), {"a": (1.8 * np.clip(t - 30e-12, 0, None) / 1e-9).tolist()})
    c = ns.compare_waveforms(ref, good)
    assert math.isclose(c.max_abs_error, 2e-4, rel_tol=1e-6) and c.sample_count == 101 and c.max_edge_timing_error < 1e-12
    assert ns.within_v1_contract(c, nonlinear=False)[0]
    c2 = ns.compare_waveforms(ref, late)
    assert math.isclose(c2.max_edge_timing_error, 30e-12, rel_tol=1e-3)
    assert not ns.within_v1_contract(c2, nonlinear=True)[0]
    assert ns.v1_tolerance_profile(nonlinear=True).edge_tol == 10e-12 and math.isclose(ns.v1_tolerance_profile(nonlinear=False).max_abs_tol, 1.8e-3)
    empty = ns.compare_waveforms(ref, ns.WaveformData("c", "", ["b"], t.tolist(), {"b": t.tolist()}))
    assert empty.sample_count == 0 and not empty.within_tolerance(max_abs_tol=1, rms_tol=1, final_abs_tol=1)
    assert ns.find_nangila_binary() is not None


def test_solver_binary_json_and_nz_outputs(tmp_path):
    exe = ns.find_nangila_binary()
    deck = _write(tmp_path, "rc.sp", "* rc\nV1 vdd 0 DC 1.8\nR1 vdd out 1k\nC1 out 0 10f\n.ic V(out)=0\n.end\n")
    wj, wz = tmp_path / "w.json", tmp_path / "w.nz"
    proc = subprocess.run([exe, "--partition", deck, "--tstop", "1e-10", "--dt", "1e-12", "--waveform-json", str(wj), "--waveform-nz", str(wz),
                           "--nz-tol", "1e-6"], capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    d = json.loads(wj.read_text())
    assert d["node_names"] == ["vdd", "out"] and len(d["waveform"]) == 101 and d["stats"]["total_steps"] == 100
    nz = ns.read_nz(str(wz))
    assert nz.header.version == 2 and nz.node_names == ["vdd", "out"] and nz.header.num_points == 101
    direct = np.array([p["voltages"]["out"] for p in d["waveform"]])
    assert np.abs(nz.signals["out"] - direct).max() <= 1e-6 * (1 + 1e-9)
    from nangila_spice.nz_viewer import compare_waveforms, plot_nz

    assert compare_waveforms(nz, {"out": direct})["within_bound"]
    assert "out" in plot_nz(str(wz), ["out"], output=str(tmp_path / "p.png")) or os.path.exists(tmp_path / "p.png")
    # the reference's calling forms: a loaded waveform as the source, its keyword names, one net against its original
    text = plot_nz(nz, nodes=["out", "nosuch"], title="rc", show_error_bound=True, output_path=str(tmp_path / "p.txt"), time_scale="ps")
    assert os.path.exists(tmp_path / "p.txt") or os.path.exists(tmp_path / "p.png") or "rc" in text
    times = [p["time"] for p in d["waveform"]]
    one = compare_waveforms(times, direct, str(wz), "out", title="t", output_path=str(tmp_path / "c.png"))
    assert one["within_bound"] and set(one["per_node"]) == {"out"}
    coarse = compare_waveforms(times[::2], direct[::2], nz, node="out")   # another time axis: interpolated onto the file's
    assert coarse["max_abs_error"] < 0.05 and not coarse["within_bound"]
    with pytest.raises(KeyError):
        compare_waveforms(times, direct, nz, "nosuch")
    with pytest.raises(TypeError):
        plot_nz(42)
    assert subprocess.run([exe, "--partition", "/nonexistent.sp"], capture_output=True).returncode == 1
    assert subprocess.run([exe, "--bogus"], capture_output=True).returncode == 2
    demo = subprocess.run([exe, "--demo", "--tstop", "5e-11"], capture_output=True, text=True)
    assert demo.returncode == 0 and "V(cap)" in demo.stderr
    # every partition of a design in one solver process
    flat = json.loads(N.generate_circuit("rc_ladder", 12))
    files = []
    for i, text in enumerate(partition_flat(flat, 2, "bisect").partition_files()):
        files.append(_write(tmp_path, f"p{i}.json", text))
    out = tmp_path / "merged.json"
    proc = subprocess.run([exe, "--partitions", ",".join(files), "--tstop", "2e-11", "--dt", "1e-12", "--waveform-json", str(out)], capture_output=True, text=True)
    assert proc.returncode == 0 and "partitioned run: 20 steps" in proc.stderr
    assert len(json.loads(out.read_text())["waveform"]) == 21


def test_pvt_sweep(tmp_path):
    grid = ns.generate_corner_grid()
    assert len(grid) == 200 and grid[0].name == "TT_1.62V_-40C"
    from nangila_spice.pvt_orchestrator import generate_1000_corner_grid

    assert len(generate_1000_corner_grid()) == 1000
    nominal = ns.CornerSpec.nominal()
    assert nominal.is_nominal and math.isclose(nominal.thermal_voltage, 8.617e-5 * 300.15)
    far = ns.CornerSpec(ns.ProcessCorner.SS, 1.2, 125.0)
    assert not far.is_linearisable(nominal) and ns.CornerSpec(ns.ProcessCorner.FF, 1.89, 40.0).is_linearisable(nominal)
    corners = [ns.CornerSpec(ns.ProcessCorner.FF, 1.89, 40.0), ns.CornerSpec(ns.ProcessCorner.TT, 1.71, 27.0), far]
    res = ns.PvtOrchestrator(ns.SweepConfig(max_workers=2, tstop=50e-12)).run_sweep(corners)
    assert res.total_corners == 4 and res.completed == 4 and res.failed == 0
    assert res.delta_mode_used == 2 and res.full_sim_used == 2 and res.peak_delta_v > 0.05
    assert "4/4 corners" in res.summary() and res.success_rate == 1.0
    res.to_json(str(tmp_path / "sweep.json"))
    assert json.loads((tmp_path / "sweep.json").read_text())["completed"] == 4
    # the delta model against a real simulation of the same corner: supply scaling is exact for a passive stage
    golden = ns.simulate_corner(nominal, None, False, None, 50e-12, 1e-12)
    c = ns.CornerSpec(ns.ProcessCorner.TT, 1.71, 27.0)
    approx = ns.simulate_corner(c, golden, True, None, 50e-12, 1e-12)
    exact = ns.simulate_corner(c, golden, False, None, 50e-12, 1e-12)
    assert approx["used_delta"] and not exact["used_delta"]
    assert np.abs(np.array(approx["values"]) - np.array(exact["values"])).max() < 1e-9


def test_gate_level_synthesis_computes_c17(tmp_path):
    from nangila_spice.synth import C17_BENCH, bench_to_spice

    def nand(a, b):
        return 1 - (a & b)

    for bits in ((0, 0, 0, 0, 0), (1, 1, 1, 1, 1), (1, 0, 1, 1, 0), (0, 1, 0, 1, 1)):
        i1, i2, i3, i6, i7 = bits
        stim = [f"VIN{k} n{name} 0 DC {1.8 * b}" for k, (name, b) in enumerate(zip(("1", "2", "3", "6", "7"), bits))]
        deck = bench_to_spice(C17_BENCH, "c17", stimulus=stim)
        js, warnings = N.parse_spice(deck, "c17")
        ok, v = N.dc_operating_point(js)
        names = json.loads(js)["node_names"]
        g10, g11 = nand(i1, i3), nand(i3, i6)
        g16, g19 = nand(i2, g11), nand(g11, i7)
        want = {"n22": nand(g10, g16), "n23": nand(g16, g19)}
        assert ok and warnings == []
        for net, bit in want.items():
            assert abs(v[names.index(net)] - 1.8 * bit) < 0.05, (bits, net)
    xor = bench_to_spice("INPUT(a)\nINPUT(b)\nOUTPUT(y)\nOUTPUT(z)\ny = XOR(a, b)\nz = NOR(a, b)\n",
                         stimulus=["VA na 0 DC 1.8", "VB nb 0 DC 0"])
    js, _ = N.parse_spice(xor)
    ok, v = N.dc_operating_point(js)
    names = json.loads(js)["node_names"]
    assert ok and v[names.index("ny")] > 1.75 and v[names.index("nz")] < 0.05


def test_scaling_study_report_and_cli(tmp_path):
    suite = run_scaling_study(generate_rc_ladder_netlist(30, 1e3, 10e-15), "ladder30", [1, 2], tstop=100e-12, dt=1e-12, method="bisect")
    assert [r.partition_count for r in suite.results] == [1, 2] and suite.results[1].max_abs_error_vs_single < 1e-5
    from nangila_spice.benchmark import generate_performance_report

    md = generate_performance_report(suite, str(tmp_path / "perf"))
    assert os.path.exists(md) and "ladder30_k2" in open(md).read() and "Average speedup" in suite.summary()
    # the reference's form: a generator, sizes, partition counts; here every combination is really simulated
    study = run_scaling_study(generate_rc_ladder_netlist, [10, 20], [1, 2], label="RC study", tstop=40e-12)
    assert [(r.element_count, r.partition_count) for r in study.results] == [(21, 1), (22, 2), (41, 1), (42, 2)] and study.name == "RC study"
    assert all(r.timesteps == 40 and r.wall_time_secs > 0 for r in study.results)
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    deck = _write(tmp_path, "rc.sp", generate_rc_ladder_netlist(8, 1e3, 10e-15))
    run = subprocess.run([sys.executable, "-m", "nangila_spice.cli", "run", deck, "--partitions", "2", "--tstop", "5e-11", "--method", "bisect",
                          "--output-dir", str(tmp_path / "o"), "--output-format", "json"], capture_output=True, text=True, env=env)
    assert run.returncode == 0 and "partitioned_validated" in run.stdout, run.stdout + run.stderr
    assert os.path.exists(tmp_path / "o" / "rc.json")
    synth = subprocess.run([sys.executable, "-m", "nangila_spice.cli", "synth"], capture_output=True, text=True, env=env)
    assert synth.returncode == 0 and synth.stdout.count("\nM") == 24  # six two-input NANDs
    rep = subprocess.run([sys.executable, "-m", "nangila_spice.cli", "phase1-report", "--output-json", str(tmp_path / "r.json"), "--output-md",
                          str(tmp_path / "r.md")], capture_output=True, text=True, env=env)
    assert rep.returncode == 0, rep.stdout + rep.stderr
    report = json.loads((tmp_path / "r.json").read_text())
    assert report["all_passed"] and len(report["cases"]) == 13 and report["blocked"] == []
    assert sum(c["logic_levels_checked"] for c in report["cases"]) >= 18
    from nangila_spice.visualizer import visualize_partitions

    nl = ns.parse_netlist(deck)
    dot = visualize_partitions(nl, ns.partition_netlist(nl, 2, "bisect"))
    assert dot.startswith("graph partitions {") and "style=dashed" in dot
    # the reference's form: the circuit graph first, a title, devices only; an image request without matplotlib falls back to DOT
    pr = ns.partition_netlist(nl, 2, "bisect")
    cg = ns.build_circuit_graph(nl.flatten())
    devices_only = visualize_partitions(cg, pr, title="two parts", show_nets=False)
    assert 'label="two parts"' in devices_only and "shape=ellipse" not in devices_only and "shape=box" in devices_only
    written = visualize_partitions(cg, pr, output_path=str(tmp_path / "parts.png"), figsize=(6, 4))
    assert os.path.exists(written) and written.endswith((".png", ".dot"))
    hw = ns.discover_hardware()
    assert hw.cpu_count >= 1 and "cores" in hw.summary()


def test_small_api_members_of_the_reference_front_end(tmp_path):
    from nangila_spice import cli
    from nangila_spice.nz_reader import read_nz
    from nangila_spice.pvt_orchestrator import ProcessCorner

    assert os.path.isdir(os.path.join(cli.get_project_root(), "csrc", "spice"))
    assert ProcessCorner.TT.is_nominal and not ProcessCorner.SS.is_nominal
    deck = _write(tmp_path, "rc.sp", "* rc\nV1 in 0 DC 1.0\nR1 in out 1k\nC1 out 0 10f\n.ic V(out)=0\n.end\n")
    out = tmp_path / "w.nz"
    from nangila_spice.correctness import find_nangila_binary

    run = subprocess.run([find_nangila_binary(), "--partition", deck, "--tstop", "1e-10", "--dt", "1e-12", "--waveform-nz", str(out)],
                         capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
    w = read_nz(str(out))
    assert w.num_points == 101 and abs(w.voltage("in") - 1.0) < 1e-5
    tau = 10e-12
    assert abs(w.voltage("out", 20e-12) - (1 - math.exp(-20e-12 / tau))) < 5e-3
    assert w.voltage("out", -1.0) == w.signals["out"][0] and w.voltage("out", 1.0) == w.signals["out"][-1]
    with pytest.raises(KeyError):
        w.voltage("nope")


def _partition_files(tmp_path, text, k, method="spectral"):
    nl = ns.parse_netlist(_write(tmp_path, "deck.sp", text))
    pr = ns.partition_netlist(nl, k, method)
    files = []
    for i, js in enumerate(pr.partition_files()):
        path = tmp_path / f"p{i}.json"
        path.write_text(js)
        files.append(str(path))
    return files


def test_partitions_as_processes_exchange_boundaries_over_tcp(tmp_path):
    deck = _write(tmp_path, "ladder.sp", generate_rc_ladder_netlist(45, 1e3, 10e-15))
    res = ns.simulate(deck, partitions=3, tstop=150e-12, dt=1e-12, mode="processes", method="bisect", output_dir=str(tmp_path / "run"))
    assert res.success and res.validation_status == "partitioned_validated", (res.error, res.warnings)
    assert res.reference_comparison.max_abs_error < 1e-6
    assert res.solver_stats["stats"]["processes"] == 3 and "messages" in res.solver_stats["stats"]["log_tail"][0]
    # transistor-level logic across four processes
    from nangila_spice import correctness as cx

    case = next(c for c in cx.official_correctness_cases() if c.name == "adder2")
    path = case.materialize(str(tmp_path))
    res = ns.simulate(path, partitions=4, tstop=0.6e-9, dt=1e-12, mode="processes", output_dir=str(tmp_path / "run2"))
    assert res.success and res.validation_status == "partitioned_validated", (res.error, res.warnings)
    assert res.reference_comparison.max_abs_error < 5e-3


def test_process_mesh_notices_absent_and_dead_peers(tmp_path):
    from nangila_spice.correctness import find_nangila_binary

    exe = find_nangila_binary()
    files = _partition_files(tmp_path, generate_rc_ladder_netlist(60, 1e3, 10e-15), 3, "bisect")
    common = ["-k", "3", "--dt", "1e-12"]
    # a peer that never starts: the others give up at the connection deadline
    rv = tmp_path / "rv_absent"
    procs = [subprocess.Popen([exe, "--partition", files[i], "--node-id", str(i), *common, "--tstop", "1e-10", "--rendezvous", str(rv),
                               "--connect-timeout-ms", "700"], stderr=subprocess.PIPE, text=True) for i in (0, 2)]
    errs = [p.communicate(timeout=30)[1] for p in procs]
    assert [p.returncode for p in procs] == [4, 4], errs
    assert "process 1" in errs[1] or "never connected" in errs[0]
    # a peer that dies in the middle of a long run: the others stop with an error that names it, well inside their I/O deadline
    rv = tmp_path / "rv_dead"
    procs = [subprocess.Popen([exe, "--partition", files[i], "--node-id", str(i), *common, "--tstop", "1e-6", "--rendezvous", str(rv),
                               "--io-timeout-ms", "5000", "--waveform-json", str(tmp_path / f"dead{i}.json")], stderr=subprocess.PIPE, text=True)
             for i in range(3)]
    time.sleep(1.0)
    assert all(p.poll() is None for p in procs), "the run ended before the fault was injected"
    procs[1].kill()
    t0 = time.time()
    errs = [p.communicate(timeout=30)[1] for p in procs]
    assert time.time() - t0 < 8.0
    assert procs[0].returncode == 5 and procs[2].returncode == 5, errs
    assert any("process 1" in e for e in (errs[0], errs[2])) and all("stopped early" in e for e in (errs[0], errs[2]))
    # what the survivors had computed up to then is on disk
    partial = json.loads((tmp_path / "dead0.json").read_text())
    assert partial["stats"]["completed"] is False and len(partial["waveform"]) > 10


def test_speculative_windows_roll_back_on_a_miss_and_keep_the_answer(tmp_path):
    """Partitions run several steps ahead on predictions; a missed prediction relaxes that step and discards the rest."""
    from nangila_spice import correctness as cx

    # a smooth line: once the input edge has passed, predictions hit and whole windows are accepted
    files = _partition_files(tmp_path, generate_rc_ladder_netlist(120, 1e3, 10e-15), 3, "bisect")
    texts = [open(f).read() for f in files]
    lock = N.simulate_partitioned(texts, 300e-12, 1e-12, 1e-3, 5, True, 1, 1, False)
    spec = N.simulate_partitioned(texts, 300e-12, 1e-12, 1e-3, 5, True, 1, 1, True)
    assert lock["stats"]["windows"] == 0 and lock["stats"]["completed"] and spec["stats"]["completed"]
    assert spec["stats"]["windows"] > 5 and spec["stats"]["speculated_steps"] >= 100
    assert np.abs(np.asarray(lock["values"]) - np.asarray(spec["values"])).max() < 1e-4
    # switching logic: predictions miss at every edge, so windows are cut (rollbacks) and the depth controller backs off,
    # and the result still agrees with the single matrix
    case = next(c for c in cx.extended_phase1_correctness_cases() if c.name == "alu2")
    path = case.materialize(str(tmp_path))
    nl = ns.parse_netlist(path)
    pr = ns.partition_netlist(nl, 4, "spectral")
    flat = nl.to_native()
    flat.pop("warnings", None)
    single = N.simulate(json.dumps(flat), 0.8e-9, 1e-12)
    part = N.simulate_partitioned(pr.partition_files(), 0.8e-9, 1e-12, 1e-3, 5, True, 1, 2, True)
    st = part["stats"]
    assert st["completed"] and st["rollbacks"] > 0 and st["discarded_steps"] > 0 and st["unconverged_steps"] == 0
    a, names = np.asarray(single["values"]), single["node_names"]
    b = np.asarray(part["values"])
    idx = [names.index(n) for n in part["node_names"]]
    assert np.abs(a[:, idx] - b).max() < 2e-3


def test_ngspice_oracle_plumbing_with_a_stand_in(tmp_path):
    """ngspice is not installed where these tests run, so a stand-in executable takes its place: it reads the deck and
    the ``.control`` block the harness wrote (``tran <dt> <tstop> [uic]``, ``wrdata <file> v(a) v(b)``), solves the deck
    with this package and writes the columns ``wrdata`` would. What is checked is the harness: the deck it hands over, the
    control block, the parsing of the data file and the comparison that follows."""
    import stat
    import sys

    from nangila_spice.correctness import compare_waveforms, run_nangila_waveform, run_ngspice_waveform, within_v1_contract

    fake = tmp_path / "ngspice"
    fake.write_text(f"""#!{sys.executable}
import re, sys
sys.path.insert(0, {repr(str(__import__('pathlib').Path(__file__).resolve().parents[1]))})
assert sys.argv[1] == "-b"
text = open(sys.argv[2]).read()
ctl = text[text.lower().index(".control"):text.lower().index(".endc")]
m = re.search(r"tran\\s+(\\S+)\\s+(\\S+)(\\s+uic)?", ctl)
dt, tstop, uic = float(m.group(1)), float(m.group(2)), bool(m.group(3))
w = re.search(r"wrdata\\s+(\\S+)\\s+(.*)", ctl)
nodes = re.findall(r"v\\(([^)]+)\\)", w.group(2))
deck = text[:text.lower().index(".control")] + ".end\\n"
if not uic:
    deck = "\\n".join(l for l in deck.splitlines() if not l.strip().lower().startswith(".ic")) + "\\n"
open(sys.argv[2] + ".plain.sp", "w").write(deck)
from nangila_spice.correctness import run_nangila_waveform
wf = run_nangila_waveform(sys.argv[2] + ".plain.sp", tstop=tstop, dt=dt, in_process=True)
with open(w.group(1), "w") as out:
    for i, t in enumerate(wf.times):
        out.write(" ".join([repr(float(t))] + [repr(float(wf.traces[n][i])) for n in nodes]) + "\\n")
""")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    deck = tmp_path / "rc.sp"
    deck.write_text("* rc\nV1 vdd 0 DC 1.8\nR1 vdd out 1k\nC1 out 0 10f\n.ic v(out)=0\n.end\n")
    with_ic = run_ngspice_waveform(str(deck), ["vdd", "out"], tstop=50e-12, dt=1e-12, binary=str(fake), use_initial_conditions=True)
    assert with_ic.tool == "ngspice" and len(with_ic.times) == 51 and with_ic.traces["out"][0] == 0.0 and with_ic.traces["out"][-1] > 1.7
    from_dc = run_ngspice_waveform(str(deck), ["out"], tstop=50e-12, dt=1e-12, binary=str(fake))
    assert abs(from_dc.traces["out"][0] - 1.8) < 1e-6  # without `uic` the run starts from the operating point
    cmp_ = compare_waveforms(with_ic, run_nangila_waveform(str(deck), tstop=50e-12, dt=1e-12), vdd=1.8)
    ok, profile = within_v1_contract(cmp_, nonlinear=False, vdd=1.8)
    assert ok and cmp_.sample_count == 102 and cmp_.max_abs_error < 1e-9
    with pytest.raises(RuntimeError, match="ngspice failed"):
        run_ngspice_waveform(str(deck), ["out"], tstop=1e-11, dt=1e-12, binary=sys.executable)  # "python -b deck" writes no data file


def test_simulate_keeps_the_requested_nets_only():
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "reference_circuits")
    res = ns.simulate(os.path.join(root, "inverter.sp"), tstop=2e-10, dt=1e-12, record_nodes=["OUT"])
    assert res.success and res.waveform.node_names == ["out"] and res.waveform.num_points == 201
    full = ns.simulate(os.path.join(root, "inverter.sp"), tstop=2e-10, dt=1e-12)
    assert np.array_equal(res.waveform.traces["out"], full.waveform.traces["out"]) and len(full.waveform.node_names) == 4


def test_dc_sweep_transfer_curves(tmp_path):
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "reference_circuits")
    vtc = ns.dc_sweep(os.path.join(root, "inverter.sp"), "in", 0.0, 1.8, 0.05)
    vin, out = vtc.times, vtc.traces["out"]
    assert len(vin) == 37 and out[0] > 1.79 and abs(out[-1]) < 1e-6 and np.all(np.diff(out) <= 1e-9) and not np.isnan(out).any()
    assert abs(vin[np.argmin(np.abs(out - 0.9))] - 0.9) < 0.051   # the deck's pull-up and pull-down are matched
    gain = np.abs(np.diff(out) / np.diff(vin)).max()
    assert gain > 5.0                                             # and the curve is steep at the threshold
    # a linear divider follows the source exactly; a downward sweep works too
    deck = tmp_path / "div.sp"
    deck.write_text("* divider\nV1 a 0 DC 1\nR1 a b 3k\nR2 b 0 1k\n.end\n")
    lin = ns.dc_sweep(str(deck), "A", 2.0, -2.0, -0.5)
    assert np.allclose(lin.traces["b"], 0.25 * lin.times, atol=1e-9) and list(lin.times[:2]) == [2.0, 1.5] and len(lin.times) == 9
    with pytest.raises(ValueError):
        ns.dc_sweep(str(deck), "b", 0.0, 1.0, 0.1)    # b is not held by a source
    with pytest.raises(ValueError):
        ns.dc_sweep(str(deck), "a", 0.0, 1.0, -0.1)   # the step points away from stop
    run = subprocess.run([sys.executable, "-m", "nangila_spice.cli", "dc", os.path.join(root, "inverter.sp"), "--source", "in", "--step", "0.1",
                          "--output", str(tmp_path / "vtc.csv")], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "dc sweep of in" in run.stdout, run.stdout + run.stderr
    rows = (tmp_path / "vtc.csv").read_text().splitlines()
    assert rows[0].startswith("time,") and "V(out)" in rows[0] and len(rows) == 20
