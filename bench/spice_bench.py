#!/usr/bin/env python
"""Host benchmarks of the circuit simulator, one JSON line each, and the partition scaling report.

    python bench/spice_bench.py [--report docs/spice/scaling-report.md] [--quick]

* ``solver``: transient steps per second of the single-matrix solver on generated decks (a line, a mesh, logic blocks).
* ``scaling``: the same deck at 1, 2, 4 and 8 partitions (threads of one process), errors against the single-matrix run;
  written as Markdown when ``--report`` is given.
* ``processes``: four solver processes over TCP against four threads, with and without windows of speculative steps.
* ``pvt``: a 1001-corner sweep of a 2-bit ALU.

Everything runs on the CPU; times are this machine's.
"""
import argparse
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import nangila_spice as ns  # noqa: E402
from nangila_spice import _native as N  # noqa: E402
from nangila_spice import benchcircuits as bc  # noqa: E402
from nangila_spice import correctness as cx  # noqa: E402
from nangila_spice.benchmark import generate_performance_report, generate_rc_ladder_netlist, run_scaling_study  # noqa: E402


def emit(**row) -> None:
    print(json.dumps(row), flush=True)


def solver_rows(quick: bool) -> None:
    decks = [("rc_ladder_4000", generate_rc_ladder_netlist(4000, 1e3, 10e-15), 200), ("c432_counterpart", bc.deck("c432", cload="20f"), 400),
             ("c6288_counterpart", bc.deck("c6288", cload="20f"), 400)]
    if not quick:
        decks.append(("s13207_counterpart", bc.deck("s13207", cload="20f"), 200))
    for name, text, steps in decks:
        js, _ = N.parse_spice(text)
        for adaptive in (False, True):
            r = N.simulate(js, steps * 1e-12, 1e-12, adaptive=adaptive)
            st, nr = r["stats"], r["newton"]
            emit(bench="solver", deck=name, unknowns=len(r["node_names"]), adaptive=adaptive, steps=st["total_steps"],
                 solver_steps=st["solver_steps"] or st["total_steps"], seconds=st["wall_time_secs"],
                 steps_per_s=st["total_steps"] / max(st["wall_time_secs"], 1e-12), newton_iterations=nr["total_iterations"],
                 lu_refactors=nr["lu_refactors"], lu_reuses=nr["lu_reuses"], lu_factor_nnz=nr["lu_factor_nnz"], completed=st["completed"])


def scaling_rows(quick: bool, report: str) -> None:
    decks = [("rc_ladder_4000", generate_rc_ladder_netlist(4000, 1e3, 10e-15), 200), ("c6288_counterpart", bc.deck("c6288", cload="20f"), 400)]
    if not quick:
        decks.append(("s13207_counterpart", bc.deck("s13207", cload="20f"), 200))
    parts = []
    with tempfile.TemporaryDirectory() as tmp:
        for name, text, steps in decks:
            suite = run_scaling_study(text, name, [1, 2, 4, 8], tstop=steps * 1e-12, dt=1e-12, method="auto")
            for r in suite.results:
                emit(bench="scaling", deck=name, partitions=r.partition_count, seconds=r.wall_time_secs, speedup=r.speedup,
                     max_abs_error_v=r.max_abs_error_vs_single, relaxation_solves=r.rollbacks)
            parts.append(open(generate_performance_report(suite, tmp)).read())
    if report:
        head = ("# Partition scaling on this machine\n\nOne run each of `nangila_spice.benchmark.run_scaling_study` (threads of one process, one thread per "
                "partition, solver time only; errors against the single-matrix run), written by `python bench/spice_bench.py --report " + report +
                "`. The decks are generated: a 4000-stage RC line, the 16 x 16 multiplier that stands in for c6288 and the counter / shift-register "
                "block that stands in for s13207, 20 fF per gate, 1 ps steps. On a shared machine single figures move by 10-20 % between runs.\n\n")
        os.makedirs(os.path.dirname(report) or ".", exist_ok=True)
        with open(report, "w") as f:
            f.write(head + "\n\n".join(parts))


def process_rows() -> None:
    case = next(c for c in cx.extended_phase1_correctness_cases() if c.name == "rc_ladder_400")
    with tempfile.TemporaryDirectory() as tmp:
        path = case.materialize(tmp)
        for mode in ("in_process", "processes"):
            for speculate in (True, False):
                t0 = time.perf_counter()
                res = ns.simulate(path, partitions=4, tstop=case.tstop, dt=1e-12, mode=mode, speculate=speculate, output_dir=os.path.join(tmp, mode + str(speculate)))
                st = res.solver_stats["stats"]
                emit(bench="processes", deck=case.name, mode=mode, speculate=speculate, validated=res.validation_status,
                     max_abs_error_v=res.reference_comparison.max_abs_error, seconds_total=time.perf_counter() - t0,
                     solver_seconds=st.get("wall_time_secs"), log=(st.get("log_tail") or [""])[0][16:])


def pvt_rows() -> None:
    from nangila_spice.pvt_orchestrator import PvtOrchestrator, SweepConfig, generate_1000_corner_grid

    case = next(c for c in cx.extended_phase1_correctness_cases() if c.name == "alu2")
    with tempfile.TemporaryDirectory() as tmp:
        path = case.materialize(tmp)
        res = PvtOrchestrator(SweepConfig(tstop=1e-9, dt=1e-12, output_dir=tmp)).run_sweep(generate_1000_corner_grid(), path)
        emit(bench="pvt", deck="alu2", corners=res.total_corners, completed=res.completed, seconds=res.total_wall_time,
             delta_mode=res.delta_mode_used, simulated=res.full_sim_used, speedup_vs_simulating_every_corner=res.speedup_vs_full)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--report", default="", help="write the scaling tables as Markdown to this path")
    ap.add_argument("--quick", action="store_true", help="leave out the 34 000-unknown deck")
    ap.add_argument("--only", choices=("solver", "scaling", "processes", "pvt"), default=None)
    args = ap.parse_args()
    if args.only in (None, "solver"):
        solver_rows(args.quick)
    if args.only in (None, "scaling"):
        scaling_rows(args.quick, args.report)
    if args.only in (None, "processes"):
        process_rows()
    if args.only in (None, "pvt"):
        pvt_rows()
    return 0


if __name__ == "__main__":
    sys.exit(main())
