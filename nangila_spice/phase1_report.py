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
import os
import platform
import tempfile
import time
from pathlib import Path
from typing import Iterable, Optional

import numpy as np

from .correctness import (CorrectnessCase, WaveformData, blocked_official_correctness_cases, check_logic_levels, compare_waveforms,
                          extended_phase1_correctness_cases, find_ngspice_binary, huge_phase1_correctness_cases, large_phase1_correctness_cases, phase1_automated_correctness_cases, run_nangila_waveform,
                          run_ngspice_waveform, within_v1_contract)

# Closed-form solutions, by case name.
_ANALYTIC = {"rc_step": lambda t: {"out": 1.8 * (1.0 - np.exp(-t / 10e-12))}}


def _run_case(case: CorrectnessCase, ngspice_bin: Optional[str]) -> dict:
    with tempfile.TemporaryDirectory() as tmp:
        path = case.materialize(tmp)
        t0 = time.perf_counter()
        big = case.tier in ("large", "huge")   # thousands of nets: keep the observed ones only
        cand = run_nangila_waveform(path, tstop=case.tstop, dt=case.dt, in_process=True, nodes=list(case.nodes) if big else None)
        wall = time.perf_counter() - t0
        if ngspice_bin:
            ref, oracle = run_ngspice_waveform(path, list(case.nodes), tstop=case.tstop, dt=case.dt, binary=ngspice_bin,
                                                       use_initial_conditions=case.use_initial_conditions), "ngspice"
        elif case.name in _ANALYTIC:
            t = np.asarray(cand.times)
            tr = _ANALYTIC[case.name](t)
            ref, oracle = WaveformData("analytic", path, list(tr), t.tolist(), {k: v.tolist() for k, v in tr.items()}), "closed form"
        else:
            # the dense solver is cubic in the circuit size
            ref = run_nangila_waveform(path, tstop=case.tstop, dt=case.dt / 2, in_process=True, solver="lu" if big else "dense",
                                       nodes=list(case.nodes) if big else None)
            oracle = "sparse solver, dt / 2" if big else "dense solver, dt / 2"
        lower = {n.lower(): n for n in cand.traces}
        cand_l = WaveformData(cand.tool, cand.netlist, list(lower), cand.times, {k: cand.traces[v] for k, v in lower.items()})
        ref_l = {n.lower(): v for n, v in ref.traces.items()}
        keep = [n.lower() for n in case.nodes if n.lower() in cand_l.traces and n.lower() in ref_l]
        ref = WaveformData(ref.tool, ref.netlist, keep, ref.times, {n: ref_l[n] for n in keep})
        cmp_ = compare_waveforms(ref, cand_l)
        ok, profile = within_v1_contract(cmp_, nonlinear=case.nonlinear)
        wrong = check_logic_levels(CorrectnessCase(**{**case.__dict__, "expected_levels": tuple((n.lower(), b) for n, b in case.expected_levels)}), cand_l)
        if case.expected_levels:
            oracle += " + gate-level logic"
    return {"name": case.name, "tier": case.tier, "oracle": oracle, "nodes": keep, "samples": cmp_.sample_count,
            "max_abs_error_v": cmp_.max_abs_error, "rms_error_v": cmp_.rms_error, "final_abs_error_v": cmp_.final_abs_error,
            "edge_timing_error_s": cmp_.max_edge_timing_error, "max_abs_tol_v": profile.max_abs_tol,
            "logic_levels_checked": len(case.expected_levels), "logic_levels_wrong": [list(w) for w in wrong],
            "passed": bool(ok) and not wrong and len(keep) == len(case.nodes), "wall_time_secs": wall}


def _run_partitioned(case: CorrectnessCase, partitions: int, mode: str) -> dict:
    """The case split into ``partitions`` (threads of one process or one process each) against its own single-matrix run."""
    from .correctness import within_v1_contract as contract
    from .orchestrator import SimulationConfig, run_simulation

    with tempfile.TemporaryDirectory() as tmp:
        path = case.materialize(tmp)
        res = run_simulation(SimulationConfig(netlist_path=path, partitions=partitions, tstop=case.tstop, dt=case.dt, mode=mode,
                                              output_dir=os.path.join(tmp, "run")))
    cmp_ = res.reference_comparison
    ok, profile = contract(cmp_, nonlinear=case.nonlinear) if cmp_ is not None else (False, None)
    stats = res.solver_stats.get("stats", {})
    return {"name": f"{case.name} / {len(res.partition_result.partitions)} {'processes' if mode == 'processes' else 'threads'}", "tier": "partitioned",
            "oracle": "single matrix, same step", "nodes": list(cmp_.shared_nodes) if cmp_ else [], "samples": cmp_.sample_count if cmp_ else 0,
            "max_abs_error_v": cmp_.max_abs_error if cmp_ else float("inf"), "rms_error_v": cmp_.rms_error if cmp_ else float("inf"),
            "final_abs_error_v": cmp_.final_abs_error if cmp_ else float("inf"), "edge_timing_error_s": cmp_.max_edge_timing_error if cmp_ else None,
            "max_abs_tol_v": profile.max_abs_tol if profile else 0.0, "logic_levels_checked": 0, "logic_levels_wrong": [],
            "passed": bool(res.success and ok and res.validation_status == "partitioned_validated"),
            "wall_time_secs": float(stats.get("wall_time_secs", res.wall_time_secs)),
            "rollbacks": stats.get("rollbacks"), "relaxation_solves": stats.get("resolves")}


def _tier_summary(cases: list[dict]) -> dict:
    return {"cases": len(cases), "passed": sum(1 for c in cases if c["passed"]),
            "worst_max_abs_error_v": max((c["max_abs_error_v"] for c in cases), default=0.0),
            "total_wall_time_secs": sum(c["wall_time_secs"] for c in cases)}


def generate_phase1_benchmark_report(include_extended: bool = False, include_large: bool = False, include_partitioned: bool = False,
                                     include_huge: bool = False, jobs: int = 1) -> dict:
    """Runs the chosen tiers. ``jobs`` > 1 runs that many cases at a time in worker processes (the cases are independent;
    per-case times then include whatever the cases cost one another in memory bandwidth)."""
    ngspice = find_ngspice_binary()
    cases = phase1_automated_correctness_cases()
    if include_extended:
        cases += extended_phase1_correctness_cases()
    if include_large:
        cases += large_phase1_correctness_cases()
    if include_huge:
        cases += huge_phase1_correctness_cases()
    if jobs > 1:
        from concurrent.futures import ProcessPoolExecutor

        # the longest cases first, so that the last worker does not start the ten-minute case when the others are done
        order = sorted(range(len(cases)), key=lambda i: -len(cases[i].deck or ""))
        with ProcessPoolExecutor(max_workers=jobs) as pool:
            done = dict(zip(order, pool.map(_run_case, [cases[i] for i in order], [ngspice] * len(order))))
        rows = [done[i] for i in range(len(cases))]
    else:
        rows = [_run_case(c, ngspice) for c in cases]
    if include_partitioned:
        by_name = {c.name: c for c in phase1_automated_correctness_cases() + extended_phase1_correctness_cases()}
        for name, k, mode in (("rc_ladder_400", 4, "in_process"), ("alu2", 4, "in_process"), ("adder8", 4, "in_process"),
                              ("comparator_adder4", 3, "processes"), ("rc_ladder_50", 3, "processes")):
            rows.append(_run_partitioned(by_name[name], k, mode))
    tiers = sorted({r["tier"] for r in rows})
    return {"generated": time.strftime("%Y-%m-%d %H:%M:%S"), "platform": f"{platform.system()} {platform.machine()}",
            "oracle_tool": "ngspice" if ngspice else "built-in oracles (ngspice not installed)", "jobs": jobs, "cases": rows,
            "tiers": {t: _tier_summary([r for r in rows if r["tier"] == t]) for t in tiers},
            "blocked": [{"name": b.name, "reason": b.reason} for b in blocked_official_correctness_cases()],
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
        out += [f"## {tier}: {s['passed']}/{s['cases']} within contract", "", "| case | oracle | max error | rms error | edge timing | result | time |",
                "|---|---|---|---|---|---|---|", *_iter_tier_rows(report, tier), ""]
    if report.get("blocked"):
        reasons = {}
        for b in report["blocked"]:
            reasons.setdefault(b["reason"], []).append(b["name"])
        out += ["## not run", "", *(f"- {', '.join(names)}: {why}" for why, names in reasons.items()), ""]
    return "\n".join(out)


def main(argv: Optional[list[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="correctness-first benchmark report")
    ap.add_argument("--include-extended", action="store_true")
    ap.add_argument("--include-large", action="store_true", help="the suite entries of up to 6 000 transistors, against the gate-level logic")
    ap.add_argument("--include-partitioned", action="store_true", help="five cases split into partitions (threads and processes) against the single matrix")
    ap.add_argument("--include-huge", action="store_true", help="the seven largest suite entries (12 000 to 150 000 transistors; up to ten minutes each)")
    ap.add_argument("--jobs", type=int, default=1, help="cases run at a time (worker processes)")
    ap.add_argument("--output-json", default="artifacts/phase1_benchmark_report.json")
    ap.add_argument("--output-md", default="artifacts/phase1_benchmark_report.md")
    args = ap.parse_args(argv)
    report = generate_phase1_benchmark_report(args.include_extended, args.include_large, args.include_partitioned, args.include_huge, max(1, args.jobs))
    for path, text in ((args.output_json, json.dumps(report, indent=2)), (args.output_md, render_markdown_report(report))):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        Path(path).write_text(text)
    print(render_markdown_report(report))
    return 0 if report["all_passed"] else 1
