"""Waveform comparison and the accuracy contract, plus runners for the two tools being compared.

API counterpart: ``nangila-spice/src/nangila_spice/correctness.py:26-799`` of the reference. The
oracle there is ``ngspice``; where it is not installed ``run_ngspice_waveform`` raises and callers
fall back to the dense-solver run of this simulator (``run_nangila_waveform(solver="dense")``) or to
closed-form solutions.
"""
from __future__ import annotations

import json
import os
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
    for node in shared:
        rv, cv = np.asarray(reference.traces[node], float), np.asarray(candidate.traces[node], float)
        err = np.abs(np.interp(rt, ct, cv) - rv)
        max_abs = max(max_abs, float(err.max()))
        sum_sq += float((err * err).sum())
        count += err.size
        final_abs = max(final_abs, abs(float(np.interp(t_final, ct, cv)) - float(np.interp(t_final, rt, rv))))
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
                         record_every: int = 1) -> WaveformData:
    """Runs this simulator on a deck: through the ``nangila-node`` process (default) or in-process."""
    if in_process:
        from . import _native

        text = Path(netlist_path).read_text()
        js, _ = _native.parse_spice(text, Path(netlist_path).name, process, vdd, temp)
        r = _native.simulate(js, tstop, dt, reltol, solver, record_every)
        vals = np.asarray(r["values"], float)
        return WaveformData("nangila", netlist_path, list(r["node_names"]), list(r["time"]),
                            {n: vals[:, j].tolist() for j, n in enumerate(r["node_names"]) if j < vals.shape[1]})
    exe = binary or find_nangila_binary()
    if exe is None:
        raise FileNotFoundError("nangila-node is not built: run `python -m nangila._build --spice`")
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "wave.json")
        cmd = [exe, "--partition", netlist_path, "--tstop", repr(tstop), "--dt", repr(dt), "--reltol", repr(reltol), "--process", process,
               "--vdd", repr(vdd), "--temp", repr(temp), "--solver", solver, "--record-every", str(record_every), "--waveform-json", out]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode not in (0, 3) or not os.path.exists(out):
            raise RuntimeError(f"nangila-node failed ({proc.returncode}): {proc.stderr[-500:]}")
        with open(out) as f:
            d = json.load(f)
    names = d["node_names"]
    pts = d["waveform"]
    return WaveformData("nangila", netlist_path, names, [p["time"] for p in pts], {n: [p["voltages"].get(n, 0.0) for p in pts] for n in names})


def run_ngspice_waveform(netlist_path: str, nodes: list[str], *, tstop: float, dt: float, binary: Optional[str] = None) -> WaveformData:
    """Runs ``ngspice -b`` with a ``.control`` block that writes the listed nets; needs ngspice on PATH."""
    exe = binary or find_ngspice_binary()
    if exe is None:
        raise FileNotFoundError("ngspice is not installed")
    text = Path(netlist_path).read_text()
    with tempfile.TemporaryDirectory() as tmp:
        data = os.path.join(tmp, "out.data")
        vec = " ".join(f"v({n})" for n in nodes)
        control = f".control\nset wr_singlescale\ntran {dt!r} {tstop!r}\nwrdata {data} {vec}\nquit\n.endc\n"
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
    return WaveformData(tool, netlist, waveform.node_names, waveform.times.tolist(), {n: v.tolist() for n, v in waveform.traces.items()})
