"""Correctness-first benchmark report: runs a fixed list of cases through the solver, compares every
case with its oracle and writes a JSON record plus a Markdown summary.

Counterpart of ``nangila-spice/src/nangila_spice/phase1_report.py`` (which needs ``ngspice`` for
every case). Oracles here, in order of preference: ``ngspice`` when it is installed, a closed-form
solution where one exists, else the same deck solved with the dense direct solver at half the time
step.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import platform
import tempfile
import time
from pathlib import Path
from typing import Iterable, Optional

import numpy as np

from .benchmark import generate_cim_netlist, generate_rc_ladder_netlist
from .correctness import (WaveformData, compare_waveforms, find_ngspice_binary, run_nangila_waveform, run_ngspice_waveform,
                          within_v1_contract)
from .synth import C17_BENCH, bench_to_spice

_INVERTER = """* CMOS inverter
VDD vdd 0 DC 1.8
VIN in 0 PULSE(0 1.8 100p 50p 50p 400p 1n)
M1 out in vdd vdd pch w=2u l=180n
M2 out in 0 0 nch w=1u l=180n
CL out 0 5f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
.end
"""
_RC_STEP = "* RC step\nV1 vdd 0 DC 1.8\nR1 vdd out 1k\nC1 out 0 10f\n.ic V(out)=0\n.end\n"
_DIODE = "* diode clamp\nV1 in 0 PULSE(0 1.8 0 100p 100p 500p 2n)\nR1 in out 1k\nD1 out 0 dm\nC1 out 0 5f\n.model dm D (is=1e-14 n=1)\n.end\n"


def _cases() -> list[dict]:
    return [
        {"name": "rc_step", "tier": "passive", "deck": _RC_STEP, "tstop": 100e-12, "dt": 0.25e-12, "nonlinear": False, "nodes": ["out"],
         "analytic": lambda t: {"out": 1.8 * (1.0 - np.exp(-t / 10e-12))}},
        {"name": "rc_ladder_50", "tier": "passive", "deck": generate_rc_ladder_netlist(50, 1e3, 10e-15), "tstop": 500e-12, "dt": 0.25e-12,
         "nonlinear": False, "nodes": ["n1", "n25", "n50"]},
        {"name": "cim_8x8", "tier": "passive", "deck": generate_cim_netlist(8, 8), "tstop": 2e-9, "dt": 5e-12, "nonlinear": False,
         "nodes": ["bl0", "bl3", "bl7"]},
        {"name": "diode_clamp", "tier": "nonlinear", "deck": _DIODE, "tstop": 1e-9, "dt": 1e-12, "nonlinear": True, "nodes": ["out"]},
        {"name": "cmos_inverter", "tier": "nonlinear", "deck": _INVERTER, "tstop": 1e-9, "dt": 1e-12, "nonlinear": True, "nodes": ["out"]},
        {"name": "c17_transistor_level", "tier": "nonlinear", "deck": bench_to_spice(C17_BENCH, "c17"), "tstop": 4e-9, "dt": 0.5e-12,
         "nonlinear": True, "nodes": ["n22", "n23"]},
    ]


def _run_case(case: dict, ngspice_bin: Optional[str]) -> dict:
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, case["name"] + ".sp")
        Path(path).write_text(case["deck"])
        t0 = time.perf_counter()
        cand = run_nangila_waveform(path, tstop=case["tstop"], dt=case["dt"], in_process=True)
        wall = time.perf_counter() - t0
        if ngspice_bin:
            ref, oracle = run_ngspice_waveform(path, case["nodes"], tstop=case["tstop"], dt=case["dt"], binary=ngspice_bin), "ngspice"
        elif "analytic" in case:
            t = np.asarray(cand.times)
            tr = case["analytic"](t)
            ref, oracle = WaveformData("analytic", path, list(tr), t.tolist(), {k: v.tolist() for k, v in tr.items()}), "closed form"
        else:
            ref = run_nangila_waveform(path, tstop=case["tstop"], dt=case["dt"] / 2, in_process=True, solver="dense")
            oracle = "dense solver, dt / 2"
        keep = [n for n in case["nodes"] if n in cand.traces and n in ref.traces]
        ref = WaveformData(ref.tool, ref.netlist, keep, ref.times, {n: ref.traces[n] for n in keep})
        cmp_ = compare_waveforms(ref, cand)
        ok, profile = within_v1_contract(cmp_, nonlinear=case["nonlinear"])
    return {"name": case["name"], "tier": case["tier"], "oracle": oracle, "nodes": keep, "samples": cmp_.sample_count,
            "max_abs_error_v": cmp_.max_abs_error, "rms_error_v": cmp_.rms_error, "final_abs_error_v": cmp_.final_abs_error,
            "edge_timing_error_s": cmp_.max_edge_timing_error, "max_abs_tol_v": profile.max_abs_tol, "passed": bool(ok), "wall_time_secs": wall}


def _tier_summary(cases: list[dict]) -> dict:
    return {"cases": len(cases), "passed": sum(1 for c in cases if c["passed"]),
            "worst_max_abs_error_v": max((c["max_abs_error_v"] for c in cases), default=0.0),
            "total_wall_time_secs": sum(c["wall_time_secs"] for c in cases)}


def generate_phase1_benchmark_report(include_extended: bool = False) -> dict:
    ngspice = find_ngspice_binary()
    cases = _cases()
    if include_extended:
        cases.append({"name": "rc_ladder_400", "tier": "passive", "deck": generate_rc_ladder_netlist(400, 1e3, 10e-15), "tstop": 500e-12,
                      "dt": 1e-12, "nonlinear": False, "nodes": ["n1", "n200", "n400"]})
    rows = [_run_case(c, ngspice) for c in cases]
    tiers = sorted({r["tier"] for r in rows})
    return {"generated": time.strftime("%Y-%m-%d %H:%M:%S"), "platform": f"{platform.system()} {platform.machine()}",
            "oracle_tool": "ngspice" if ngspice else "built-in oracles (ngspice not installed)", "cases": rows,
            "tiers": {t: _tier_summary([r for r in rows if r["tier"] == t]) for t in tiers},
            "all_passed": all(r["passed"] for r in rows)}


def _iter_tier_rows(report: dict, tier: str) -> Iterable[str]:
    for c in report["cases"]:
        if c["tier"] == tier:
            edge = "-" if c["edge_timing_error_s"] is None else f"{c['edge_timing_error_s'] * 1e12:.2f} ps"
            yield (f"| {c['name']} | {c['oracle']} | {c['max_abs_error_v'] * 1e3:.3f} mV | {c['rms_error_v'] * 1e3:.3f} mV | {edge} | "
                   f"{'pass' if c['passed'] else 'FAIL'} | {c['wall_time_secs'] * 1e3:.1f} ms |")


def render_markdown_report(report: dict) -> str:
    out = ["# Correctness-first benchmark report", "", f"Generated {report['generated']} on {report['platform']}; oracle: {report['oracle_tool']}.", ""]
    for tier, s in report["tiers"].items():
        out += [f"## {tier}: {s['passed']}/{s['cases']} within contract", "", "| case | oracle | max error | rms error | edge timing | verdict | time |",
                "|---|---|---|---|---|---|---|", *_iter_tier_rows(report, tier), ""]
    return "\n".join(out)


def main(argv: Optional[list[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="correctness-first benchmark report")
    ap.add_argument("--include-extended", action="store_true")
    ap.add_argument("--output-json", default="artifacts/phase1_benchmark_report.json")
    ap.add_argument("--output-md", default="artifacts/phase1_benchmark_report.md")
    args = ap.parse_args(argv)
    report = generate_phase1_benchmark_report(args.include_extended)
    for path, text in ((args.output_json, json.dumps(report, indent=2)), (args.output_md, render_markdown_report(report))):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        Path(path).write_text(text)
    print(render_markdown_report(report))
    return 0 if report["all_passed"] else 1
