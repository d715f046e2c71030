"""Waveform comparison and the accuracy contract, plus runners for the two tools being compared.

API counterpart: ``nangila-spice/src/nangila_spice/correctness.py:26-799`` of the reference. The
oracle there is ``ngspice``; where it is not installed ``run_ngspice_waveform`` raises and callers
fall back to the dense-solver run of this simulator (``run_nangila_waveform(solver="dense")``) or to
closed-form solutions.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import subprocess
import tempfile
from dataclasses import dataclass
from math import sqrt
from pathlib import Path
from typing import Optional

import numpy as np


@dataclass
class WaveformData:
    tool: str
    netlist: str
    node_names: list[str]
    times: list[float]
    traces: dict[str, list[float]]


@dataclass
class WaveformComparison:
    shared_nodes: list[str]
    sample_count: int
    max_abs_error: float
    rms_error: float
    final_abs_error: float
    max_edge_timing_error: Optional[float]

    def within_tolerance(self, *, max_abs_tol: float, rms_tol: float, final_abs_tol: float, edge_tol: Optional[float] = None) -> bool:
        if self.sample_count == 0:
            return False
        if self.max_abs_error > max_abs_tol or self.rms_error > rms_tol or self.final_abs_error > final_abs_tol:
            return False
        if edge_tol is not None and self.max_edge_timing_error is not None and self.max_edge_timing_error > edge_tol:
            return False
        return True


@dataclass(frozen=True)
class V1ToleranceProfile:
    circuit_class: str
    max_abs_tol: float
    rms_tol: float
    final_abs_tol: float
    edge_tol: Optional[float] = None


def v1_tolerance_profile(*, nonlinear: bool, vdd: float = 1.8) -> V1ToleranceProfile:
    """Passive circuits: 1 mV peak / 0.5 mV RMS (or 0.1 % / 0.05 % of the supply). Nonlinear: 25 mV
    / 10 mV (2 % / 1 %) and 10 ps on the first half-supply crossing."""
    if nonlinear:
        return V1ToleranceProfile("nonlinear", max(25e-3, 0.02 * vdd), max(10e-3, 0.01 * vdd), max(10e-3, 0.01 * vdd), 10e-12)
    return V1ToleranceProfile("passive", max(1e-3, 0.001 * vdd), max(0.5e-3, 0.0005 * vdd), max(1e-3, 0.001 * vdd), None)


def within_v1_contract(comparison: WaveformComparison, *, nonlinear: bool, vdd: float = 1.8) -> tuple[bool, V1ToleranceProfile]:
    p = v1_tolerance_profile(nonlinear=nonlinear, vdd=vdd)
    return comparison.within_tolerance(max_abs_tol=p.max_abs_tol, rms_tol=p.rms_tol, final_abs_tol=p.final_abs_tol, edge_tol=p.edge_tol), p


def _first_crossing_time(t: np.ndarray, v: np.ndarray, threshold: float) -> Optional[float]:
    s = v - threshold
    idx = np.flatnonzero(s[:-1] * s[1:] <= 0.0)
    for i in idx:
        if s[i] == s[i + 1]:
            continue
        return float(t[i] + (t[i + 1] - t[i]) * (-s[i]) / (s[i + 1] - s[i]))
    return None


def compare_waveforms(reference: WaveformData, candidate: WaveformData, *, vdd: float = 1.8) -> WaveformComparison:
    """Errors of ``candidate`` on the reference's time points (candidate interpolated linearly)."""
    shared = sorted(set(reference.node_names) & set(candidate.node_names))
    if not shared or not len(reference.times) or not len(candidate.times):
        return WaveformComparison(shared, 0, float("inf"), float("inf"), float("inf"), None)
    rt, ct = np.asarray(reference.times, float), np.asarray(candidate.times, float)
    sum_sq, max_abs, final_abs, count = 0.0, 0.0, 0.0, 0
    edges: list[float] = []
    t_final = min(rt[-1], ct[-1])
    same_axis = rt.shape == ct.shape and np.array_equal(rt, ct)
    for node in shared:
        rv, cv = np.asarray(reference.traces[node], float), np.asarray(candidate.traces[node], float)
        err = np.abs((cv if same_axis else np.interp(rt, ct, cv)) - rv)
        max_abs = max(max_abs, float(err.max()))
        sum_sq += float(err @ err)
        count += err.size
        final_abs = max(final_abs, float(err[-1]) if same_axis else abs(float(np.interp(t_final, ct, cv)) - float(np.interp(t_final, rt, rv))))
        re, ce = _first_crossing_time(rt, rv, 0.5 * vdd), _first_crossing_time(ct, cv, 0.5 * vdd)
        if re is not None and ce is not None:
            edges.append(abs(ce - re))
    return WaveformComparison(shared, count, max_abs, sqrt(sum_sq / count) if count else float("inf"), final_abs,
                              max(edges) if edges else None)


def find_nangila_binary() -> Optional[str]:
    """The solver process built in-tree (``nangila_spice/bin/nangila-node``), else one on PATH."""
    env = os.environ.get("NANGILA_NODE_BIN")
    if env and os.path.exists(env):
        return env
    here = Path(__file__).resolve().parent / "bin" / "nangila-node"
    if here.exists():
        return str(here)
    return shutil.which("nangila-node")


def find_ngspice_binary() -> Optional[str]:
    return shutil.which("ngspice")


def run_nangila_waveform(netlist_path: str, *, tstop: float, dt: float, reltol: float = 1e-3, process: str = "TT", vdd: float = 1.8,
                         temp: float = 27.0, solver: str = "lu", binary: Optional[str] = None, in_process: bool = False,
                         record_every: int = 1, allow_partial: bool = False, adaptive: bool = False,
                         nodes: Optional[list] = None) -> WaveformData:
    """Runs this simulator on a deck: through the ``nangila-node`` process (default) or in-process. A run that
    stops before ``tstop`` (Newton did not converge even after step cutting) raises unless ``allow_partial``.
    ``adaptive``: the solver chooses its own steps between the points of the ``dt`` grid the waveform is written on.
    ``nodes``: keep these nets only (names compared without case); a deck of 100 000 nets over thousands of samples
    is gigabytes as Python lists, and a comparison looks at a handful of them."""
    if in_process:
        from . import _native

        text = Path(netlist_path).read_text()
        js, _ = _native.parse_spice(text, Path(netlist_path).name, process, vdd, temp)
        r = _native.simulate(js, tstop, dt, reltol, solver, record_every, adaptive=adaptive, record_nodes=list(nodes or []))
        if not r["stats"]["completed"] and not allow_partial:
            raise RuntimeError(f"{netlist_path}: stopped at t = {r['time'][-1]:.4g} s of {tstop:.4g} s: Newton did not converge")
        vals = np.asarray(r["values"], float)
        wanted = None if nodes is None else {n.lower() for n in nodes}
        names = [n for j, n in enumerate(r["node_names"]) if j < vals.shape[1] and (wanted is None or n.lower() in wanted)]
        col = {n: j for j, n in enumerate(r["node_names"])}
        return WaveformData("nangila", netlist_path, names, list(r["time"]), {n: vals[:, col[n]].tolist() for n in names})
    exe = binary or find_nangila_binary()
    if exe is None:
        raise FileNotFoundError("nangila-node is not built: run `python -m nangila._build --spice`")
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "wave.json")
        cmd = [exe, "--partition", netlist_path, "--tstop", repr(tstop), "--dt", repr(dt), "--reltol", repr(reltol), "--process", process,
               "--vdd", repr(vdd), "--temp", repr(temp), "--solver", solver, "--record-every", str(record_every), "--waveform-json", out]
        if adaptive:
            cmd.append("--adaptive")
        if nodes:
            cmd += ["--record-nodes", ",".join(nodes)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode == 3 and not allow_partial:
            raise RuntimeError(f"{netlist_path}: stopped before tstop: {proc.stderr[-300:]}")
        if proc.returncode not in (0, 3) or not os.path.exists(out):
            raise RuntimeError(f"nangila-node failed ({proc.returncode}): {proc.stderr[-500:]}")
        with open(out) as f:
            d = json.load(f)
    wanted = None if nodes is None else {n.lower() for n in nodes}
    names = [n for n in d["node_names"] if wanted is None or n.lower() in wanted]
    pts = d["waveform"]
    return WaveformData("nangila", netlist_path, names, [p["time"] for p in pts], {n: [p["voltages"].get(n, 0.0) for p in pts] for n in names})


def run_ngspice_waveform(netlist_path: str, nodes: list[str], *, tstop: float, dt: float, binary: Optional[str] = None,
                         use_initial_conditions: bool = False) -> WaveformData:
    """Runs ``ngspice -b`` with a ``.control`` block that writes the listed nets; needs ngspice on PATH (or ``binary``).
    ``use_initial_conditions`` starts the transient from the deck's ``.ic`` values (``uic``) instead of the DC point."""
    exe = binary or find_ngspice_binary()
    if exe is None:
        raise FileNotFoundError("ngspice is not installed")
    text = Path(netlist_path).read_text()
    with tempfile.TemporaryDirectory() as tmp:
        data = os.path.join(tmp, "out.data")
        vec = " ".join(f"v({n})" for n in nodes)
        control = f".control\nset wr_singlescale\ntran {dt!r} {tstop!r}{" uic" if use_initial_conditions else ""}\nwrdata {data} {vec}\nquit\n.endc\n"
        lines = [ln for ln in text.splitlines() if ln.strip().lower() != ".end"]
        deck = os.path.join(tmp, "deck.sp")
        Path(deck).write_text("\n".join(lines) + "\n" + control + ".end\n")
        proc = subprocess.run([exe, "-b", deck], capture_output=True, text=True)
        if proc.returncode != 0 or not os.path.exists(data):
            raise RuntimeError(f"ngspice failed: {proc.stderr[-500:]}")
        arr = np.loadtxt(data, ndmin=2)
    return WaveformData("ngspice", netlist_path, list(nodes), arr[:, 0].tolist(), {n: arr[:, j + 1].tolist() for j, n in enumerate(nodes)})


def waveform_to_data(waveform, tool: str = "nangila", netlist: str = "") -> WaveformData:
    """``merger.Waveform`` -> ``WaveformData``."""
    # the arrays themselves: a list per trace costs a Python float per sample, and every consumer goes through numpy anyway
    return WaveformData(tool, netlist, waveform.node_names, waveform.times, dict(waveform.traces))


# ---- case registry ------------------------------------------------------------------------------------------
# The reference keeps its correctness cases as lists of deck paths inside its repository
# (correctness.py:112-420: official, phase-1 automated, extended and blocked cases). The decks here are
# generated (benchmark.py, benchcircuits.py), so a case carries its deck text; ``materialize`` writes it out.
@dataclass(frozen=True)
class CorrectnessCase:
    """One deck with what to observe and how to step it. ``expected_levels`` (net -> 0 / 1) is the logic-level
    oracle of a synthesised case: the settled voltage of those nets must sit at the matching rail."""
    name: str
    deck: str
    nodes: tuple
    tstop: float
    dt: float
    nonlinear: bool
    tier: str = "passive"
    use_initial_conditions: bool = False
    vdd: float = 1.8
    expected_levels: tuple = ()

    def materialize(self, directory: str) -> str:
        """Writes the deck to ``directory/<name>.sp`` and returns the path."""
        os.makedirs(directory, exist_ok=True)
        path = os.path.join(directory, self.name + ".sp")
        with open(path, "w") as fh:
            fh.write(self.deck)
        return path

    @property
    def netlist_path(self) -> str:
        """The deck as a file (the reference's cases are files of its repository; these are generated, and written to a
        per-user directory under the system's temporary directory the first time the path is asked for)."""
        return self.materialize(_case_directory())


@dataclass(frozen=True)
class BlockedCorrectnessCase:
    name: str
    reason: str

    @property
    def netlist_path(self) -> str:
        """The deck of the suite entry, generated on first use (see ``CorrectnessCase.netlist_path``)."""
        from . import benchcircuits as bc

        path = os.path.join(_case_directory(), self.name + ".sp")
        if not os.path.exists(path):
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "w") as fh:
                fh.write(bc.deck(self.name, cload="20f"))
        return path


def _case_directory() -> str:
    return os.path.join(tempfile.gettempdir(), f"nangila_spice_cases_{os.getuid() if hasattr(os, 'getuid') else 0}")


def check_logic_levels(case: CorrectnessCase, waveform: "WaveformData", margin: float = 0.1) -> list:
    """Nets of ``case.expected_levels`` whose last sample is further than ``margin * vdd`` from the expected rail,
    as ``(net, expected volts, measured volts)``."""
    bad = []
    for net, bit in case.expected_levels:
        if net not in waveform.traces:
            bad.append((net, bit * case.vdd, float("nan")))
            continue
        v = float(waveform.traces[net][-1])
        if abs(v - bit * case.vdd) > margin * case.vdd:
            bad.append((net, bit * case.vdd, v))
    return bad


def _logic_case(name: str, bench: str, title: str, inputs: dict, observe: list, tstop: float = 2e-9, dt: float = 1e-12,
                held: tuple = ()) -> CorrectnessCase:
    """A synthesised block whose inputs step from 0 to their value at 50 ps; the observed outputs must settle to the
    levels the gate-level description gives. Every gate drives 20 fF, which puts some twenty 1 ps steps on an edge:
    with the 2 fF default an edge lasts three steps and the comparison measures the step size, not the solver."""
    from .benchcircuits import evaluate_bench
    from .synth import bench_to_spice

    # inputs in `held` sit at their level from t = 0; the others step to it at 50 ps
    stim = [f"VS{k} n{net} 0 DC {1.8 * bit!r}" if net in held else f"VS{k} n{net} 0 PULSE(0 {1.8 * bit!r} 50p 20p 20p 1 2)"
            for k, (net, bit) in enumerate(inputs.items())]
    levels = evaluate_bench(bench, inputs)
    if observe is None:
        observe = re.findall(r"OUTPUT\(\s*([^)\s]+)\s*\)", bench)
    return CorrectnessCase(name, bench_to_spice(bench, title, stimulus=stim, cload="20f"), tuple("n" + o for o in observe), tstop, dt, True, tier="logic",
                           expected_levels=tuple(("n" + o, int(levels[o])) for o in observe))


def _bits(prefix: str, value: int, n: int) -> dict:
    return {f"{prefix}{i}": (value >> i) & 1 for i in range(n)}


def _suite_case(name: str) -> CorrectnessCase:
    """``<name>_auto``: a suite entry (``benchcircuits.SUITE``) at transistor level. Every input and every flip-flop output
    steps to a pseudo-random level (seeded by the name), and up to 16 outputs (nets that change level first, then primary
    outputs, then next-state nets) have to settle to what the gate list computes. The time-step oracle of these is the sparse solver at half the
    step (the dense one is cubic in the circuit size)."""
    import random
    import zlib

    from . import benchcircuits as bc

    bench = bc.S27_BENCH if name == "s27" else bc.bench_text(name)
    rng = random.Random(zlib.crc32(name.encode()))
    inputs = re.findall(r"INPUT\(\s*([^)\s]+)\s*\)", bench)
    outputs = re.findall(r"OUTPUT\(\s*([^)\s]+)\s*\)", bench)
    flops = re.findall(r"^\s*(\S+)\s*=\s*DFF\(\s*(\S+?)\s*\)", bench, re.M)
    vector = {net: rng.randint(0, 1) for net in inputs + [q for q, _ in flops]}
    # what to watch: primary outputs first, then next-state nets; not the nets the stimulus drives itself (a next-state net
    # of a shift stage is the previous stage's output, which both runs of a comparison hold exactly), and with the nets
    # that change level under this vector ahead of the ones that stay (up to eight of them), so that every case has edges
    driven = set(vector)
    candidates = [n for n in dict.fromkeys(outputs + [d for _, d in flops]) if n not in driven]
    before, after = bc.evaluate_bench(bench, {k: 0 for k in vector}), bc.evaluate_bench(bench, vector)
    moving = [n for n in candidates if before[n] != after[n]][:8]
    if len(moving) < 4:  # outputs that all hold their level say nothing about the time step: add internal nets that switch
        inner = [n for n in after if n not in driven and n not in moving and before.get(n) != after[n]]
        moving += inner[:8 - len(moving)]
    observe = list(dict.fromkeys(moving + candidates))[:16]
    # the two with the steepest internal edges need the finer step to stay inside the pointwise bound
    # and the array multiplier's carry chains make runt pulses that only an eighth of a picosecond resolves the same way
    # at two step sizes (largest difference to the half-step run: 1.8 V at 1 ps, 0.15 V at 0.25 ps, 0.7 mV at 0.125 ps)
    step = 0.5e-12 if name in ("c432", "c7552") else 0.125e-12 if name == "c6288" else 1e-12
    title = "s27 with the flip-flops cut" if name == "s27" else f"{name} ({bc.SUITE[name][2]})"
    case = _logic_case(name + "_auto", bench, title, vector, observe, tstop=1e-9 if name == "s27" else 3e-9, dt=step)
    return CorrectnessCase(**{**case.__dict__, "tier": "logic" if name == "s27" else "large"})


def official_correctness_cases(repo_root: Optional[str] = None) -> list:
    """The mandatory suite (13 cases, as many as the reference's and with its names where it has a counterpart): passive
    networks with a closed form or a half-step oracle, single devices, the hand-written circuits, s27, and the suite's
    c432 / s382 / s641 entries at transistor level. ``repo_root`` is accepted for the reference's signature: its cases are
    files below that directory, these are generated (``case.deck``; ``case.netlist_path`` writes it out)."""
    from . import benchcircuits as bc
    from .benchmark import generate_cim_netlist, generate_rc_ladder_netlist

    del repo_root
    ref = bc.reference_circuits()
    rc_step = "* RC step\nV1 vdd 0 DC 1.8\nR1 vdd out 1k\nC1 out 0 10f\n.ic V(out)=0\n.end\n"
    diode = ("* diode clamp\nV1 in 0 PULSE(0 1.8 0 100p 100p 500p 2n)\nR1 in out 1k\nD1 out 0 dm\nC1 out 0 5f\n"
             ".model dm D (is=1e-14 n=1)\n.end\n")
    return [
        CorrectnessCase("rc_step", rc_step, ("out",), 100e-12, 0.25e-12, False, use_initial_conditions=True),
        CorrectnessCase("rc_ladder_50", generate_rc_ladder_netlist(50, 1e3, 10e-15), ("n1", "n25", "n50"), 500e-12, 0.25e-12, False),
        CorrectnessCase("cim_8x8", generate_cim_netlist(8, 8), ("bl0", "bl3", "bl7"), 2e-9, 5e-12, False),
        CorrectnessCase("diode_clamp", diode, ("out",), 1e-9, 1e-12, True, tier="nonlinear"),
        CorrectnessCase("cmos_inverter", ref["inverter"], ("out",), 1e-9, 1e-12, True, tier="nonlinear"),
        CorrectnessCase("sram_6t", ref["sram_6t"], ("q", "qb"), 2e-9, 1e-12, True, tier="nonlinear", use_initial_conditions=True),
        CorrectnessCase("c17_synth", ref["c17_synth"], ("n22", "n23"), 0.5e-9, 1e-12, True, tier="nonlinear",
                        expected_levels=tuple(("n" + o, bc.evaluate_bench(bc.C17_BENCH, {k: 1 for k in "12367"})[o]) for o in ("22", "23"))),
        CorrectnessCase("c17_full", ref["c17_full"], ("n22", "n23"), 4e-9, 0.5e-12, True, tier="nonlinear"),
        _suite_case("s27"),
        _logic_case("adder2", bc.adder(2), "2-bit adder", {**_bits("a", 3, 2), **_bits("b", 1, 2), "cin": 0}, ["s0", "s1", "cout"]),
        _suite_case("c432"),
        _suite_case("s382"),
        _suite_case("s641"),
    ]


def phase1_automated_correctness_cases(repo_root: Optional[str] = None) -> list:
    """What the automated report runs by default: the mandatory suite."""
    return official_correctness_cases(repo_root)


def extended_phase1_correctness_cases(repo_root: Optional[str] = None) -> list:
    """Larger cases for ``--include-extended``: a long ladder, a wider array, generated logic blocks of a few hundred
    transistors and the suite's c880 / c1355 / c1908 entries."""
    from . import benchcircuits as bc
    from .benchmark import generate_cim_netlist, generate_rc_ladder_netlist

    del repo_root
    return [
        CorrectnessCase("rc_ladder_400", generate_rc_ladder_netlist(400, 1e3, 10e-15), ("n1", "n200", "n400"), 500e-12, 0.25e-12, False),
        CorrectnessCase("cim_16x16", generate_cim_netlist(16, 16), ("bl0", "bl7", "bl15"), 2e-9, 5e-12, False),
        _logic_case("priority4", bc.priority(4), "4-channel priority encoder", {**_bits("req", 0b1010, 4), **_bits("en", 0b1111, 4)},
                    ["idx0", "idx1", "any"], dt=0.5e-12),
        _logic_case("sec4", bc.parity_sec(4), "4-bit single-error corrector", {**_bits("d", 0b1101, 4), **_bits("r", 0b010, 3), "en": 1},
                    ["q0", "q1", "q2", "q3"]),
        _logic_case("alu2", bc.alu(2), "2-bit ALU", {**_bits("a", 1, 2), **_bits("b", 3, 2), **_bits("op", 3, 2), "cin": 0},
                    ["y0", "y1", "zero", "carry"]),
        _logic_case("adder8", bc.adder(8), "8-bit adder", {**_bits("a", 0xB5, 8), **_bits("b", 0x6E, 8), "cin": 1},
                    [f"s{i}" for i in range(8)] + ["cout"], tstop=3e-9, dt=0.5e-12),
        _logic_case("mult3", bc.multiplier(3), "3 x 3 multiplier", {**_bits("a", 5, 3), **_bits("b", 6, 3)}, [f"p{i}" for i in range(6)],
                    tstop=3e-9, dt=0.5e-12),
        _logic_case("mult4", bc.multiplier(4), "4 x 4 multiplier", {**_bits("a", 11, 4), **_bits("b", 13, 4)}, [f"p{i}" for i in range(8)],
                    tstop=3e-9, dt=0.5e-12),
        _logic_case("priority8", bc.priority(8), "8-channel priority encoder", {**_bits("req", 0b01001101, 8), **_bits("en", 0b00101000, 8)},
                    ["idx0", "idx1", "idx2", "any"], tstop=3e-9, dt=0.5e-12),
        _logic_case("comparator_adder4", bc.comparator_adder(4), "4-bit comparator and adder", {**_bits("a", 0b1011, 4), **_bits("b", 0b1100, 4), "cin": 0},
                    None, tstop=3e-9, dt=0.5e-12),
        _suite_case("c880"),
        _suite_case("c1355"),
        _suite_case("c1908"),
    ]


# suite entries with a correctness case: three in the mandatory list, three in the extended one, the rest in the large tier
_OFFICIAL_SUITE, _EXTENDED_SUITE = ("c432", "s382", "s641"), ("c880", "c1355", "c1908")
LARGE_SUITE_ENTRIES = ("c499", "c2670", "c3540", "c5315", "c7552", "s420", "s713", "s1238", "s1423", "s1488")


def large_phase1_correctness_cases(repo_root: Optional[str] = None) -> list:
    """The remaining suite entries of up to 6 000 transistors (``--include-large``), as ``<name>_auto`` cases."""
    del repo_root
    return [_suite_case(name) for name in LARGE_SUITE_ENTRIES]


HUGE_SUITE_ENTRIES = ("c6288", "s5378", "s9234", "s13207", "s15850", "s35932", "s38417", "s38584")


def huge_phase1_correctness_cases(repo_root: Optional[str] = None) -> list:
    """The long-running suite entries (``--include-huge``): the 16 x 16 array multiplier, which needs a step of 0.125 ps
    (24 000 steps), and the seven largest sequential entries, 12 000 to 150 000 transistors. Half a minute to several
    minutes each with the half-step oracle, so a report runs them on request only (several at a time with ``--jobs``)."""
    import dataclasses

    del repo_root
    return [dataclasses.replace(_suite_case(name), tier="huge") for name in HUGE_SUITE_ENTRIES]


def blocked_official_correctness_cases(repo_root: Optional[str] = None) -> list:
    """Suite entries that no report runs, with the reason. Every entry of the suite has a case, so the list is empty
    unless ``benchcircuits.SUITE`` gains an entry that no tier names yet."""
    from . import benchcircuits as bc

    del repo_root
    covered = set(_OFFICIAL_SUITE + _EXTENDED_SUITE + LARGE_SUITE_ENTRIES + HUGE_SUITE_ENTRIES) | {"c17", "s27"}
    return [BlockedCorrectnessCase(name, "no case written yet") for name in bc.SUITE if name not in covered]


def _is_ground(node: str) -> bool:
    return node.lower() in ("0", "gnd")


def collect_flattened_nodes(netlist_path: str) -> list:
    """Names of all nets of a deck after sub-circuit expansion, ground excluded (reference: correctness.py:220-230)."""
    from .parser import parse_netlist

    return sorted({n.lower() for dev in parse_netlist(netlist_path).flatten().devices for n in dev.nodes if not _is_ground(n)})


def collect_observable_nodes(netlist_path: str, *, exclude_zero_volt_alias_sinks: bool = False) -> list:
    """Top-level nets of a deck; optionally without nets that a 0 V source merely ties to another net
    (reference: correctness.py:233-261)."""
    from .parser import parse_netlist

    nodes, aliases = set(), set()
    for dev in parse_netlist(netlist_path).devices:
        nodes.update(n.lower() for n in dev.nodes if not _is_ground(n))
        if exclude_zero_volt_alias_sinks and dev.dev_type.upper() == "V" and len(dev.nodes) >= 2 and not _is_ground(dev.nodes[1]):
            value = " ".join(str(x) for x in (dev.value, dev.params.get("dc")) if x is not None).strip().lower()
            if value in ("0", "0.0", "dc 0", "dc 0.0"):
                aliases.add(dev.nodes[1].lower())
    return sorted(nodes - aliases)
