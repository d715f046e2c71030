"""``python -m nangila_spice.cli {build,run,synth,sweep,phase1-report,view}``; command set of the
reference's ``nangila`` CLI (``nangila-spice/src/nangila_spice/cli.py:106-180``) plus ``view``."""
from __future__ import annotations

import argparse
import os
import sys


def get_project_root() -> str:
    """The directory that holds ``nangila_spice`` and the native sources (``csrc/spice``)."""
    return os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def invoke_build(args) -> int:
    from nangila import _build

    _build.build_spice(force=args.force)
    if args.gpu:
        _build.build_kernels(force=args.force)
    print("build finished")
    return 0


def invoke_run(args) -> int:
    from .orchestrator import SimulationConfig, run_simulation

    if not os.path.exists(args.netlist):
        print(f"Error: netlist not found at {args.netlist}", file=sys.stderr)
        return 1
    if args.tstop is None or args.dt is None:
        # the deck's own `.tran <step> <stop>` card, then the reference's defaults (1 us in 1 ps steps)
        from .parser import parse_netlist

        step, stop = parse_netlist(args.netlist).tran() or (1e-12, 1e-6)
        args.tstop = stop if args.tstop is None else args.tstop
        args.dt = step if args.dt is None else args.dt
    result = run_simulation(SimulationConfig(netlist_path=args.netlist, partitions=args.partitions, method=args.method, reltol=args.reltol,
                                             tstop=args.tstop, dt=args.dt, predict_depth=args.predict_depth, output_dir=args.output_dir,
                                             output_format=args.output_format,
                                             validate_partitioned_against_reference=not args.skip_reference_validation,
                                             reference_vdd=args.vdd, vdd=args.vdd, verbose=args.verbose, mode=args.mode, adaptive=args.adaptive))
    print(result.summary())
    return 0 if result.success else 1


def invoke_synth(args) -> int:
    from .synth import C17_BENCH, bench_to_spice

    if args.suite:
        # the generated benchmark suite: one deck per ISCAS-class circuit plus the small reference circuits
        from .benchcircuits import SUITE, write_suite

        names = [n for n in (args.only.split(",") if args.only else SUITE)]
        paths = write_suite(args.suite, names=names)
        print(f"wrote {len(paths)} decks under {args.suite}")
        return 0
    if args.circuit:
        from .benchcircuits import deck as suite_deck

        sys.stdout.write(suite_deck(args.circuit))
        return 0
    text = open(args.bench).read() if args.bench else C17_BENCH
    deck = bench_to_spice(text, title=os.path.basename(args.bench) if args.bench else "c17")
    if args.output:
        with open(args.output, "w") as f:
            f.write(deck)
        print(f"wrote {args.output}")
    else:
        sys.stdout.write(deck)
    return 0


def invoke_sweep(args) -> int:
    from .pvt_orchestrator import PvtOrchestrator, SweepConfig, generate_1000_corner_grid

    if not os.path.exists(args.netlist):
        print(f"Error: netlist not found at {args.netlist}", file=sys.stderr)
        return 1
    grid = generate_1000_corner_grid()[:args.corners]
    res = PvtOrchestrator(SweepConfig(max_workers=args.workers, delta_mode=not args.full_sim, tstop=args.tstop, dt=args.dt)).run_sweep(grid, args.netlist)
    print(res.summary())
    return 0 if res.failed == 0 else 1


def invoke_phase1_report(args) -> int:
    from .phase1_report import main as report_main

    argv = ["--output-json", args.output_json, "--output-md", args.output_md]
    if args.include_extended:
        argv.append("--include-extended")
    if args.include_large:
        argv.append("--include-large")
    if args.include_partitioned:
        argv.append("--include-partitioned")
    if args.include_huge:
        argv.append("--include-huge")
    argv += ["--jobs", str(args.jobs)]
    return report_main(argv)


def invoke_view(args) -> int:
    from .nz_viewer import plot_nz

    try:
        print(plot_nz(args.file, args.nodes or None, args.output))
    except (OSError, ValueError) as exc:  # unreadable, truncated or not a .nz file
        print(f"Error: {args.file}: {exc}", file=sys.stderr)
        return 1
    return 0


def invoke_dc(args) -> int:
    from .merger import export_csv
    from .orchestrator import dc_sweep

    if not os.path.exists(args.netlist):
        print(f"Error: netlist not found at {args.netlist}", file=sys.stderr)
        return 1
    try:
        curve = dc_sweep(args.netlist, args.source, args.start, args.stop, args.step, process=args.process, vdd=args.vdd, temp=args.temp)
    except (ValueError, RuntimeError) as exc:
        print(f"Error: {exc}", file=sys.stderr)
        return 1
    if args.output:
        export_csv(curve, args.output)   # first column: the swept voltage
        print(f"wrote {args.output}")
    print(curve.summary())
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="nangila", description="Nangila SPICE command line")
    sub = ap.add_subparsers(dest="command", required=True)
    b = sub.add_parser("build", help="compile the native solver (and, with --gpu, the device kernels)")
    b.add_argument("--gpu", action="store_true")
    b.add_argument("--force", action="store_true")
    r = sub.add_parser("run", help="run one transient simulation")
    r.add_argument("netlist")
    r.add_argument("--partitions", type=int, default=None)
    r.add_argument("--method", default="auto")
    r.add_argument("--reltol", type=float, default=1e-3)
    r.add_argument("--tstop", type=float, default=None, help="end time in seconds (default: the deck's .tran card, else 1e-6)")
    r.add_argument("--dt", type=float, default=None, help="time step in seconds (default: the deck's .tran card, else 1e-12)")
    r.add_argument("--predict-depth", type=int, default=5)
    r.add_argument("--output-dir", default=None)
    r.add_argument("--output-format", choices=("csv", "json"), default="csv")
    r.add_argument("--vdd", type=float, default=1.8)
    r.add_argument("--mode", choices=("auto", "in_process", "processes"), default="auto")
    r.add_argument("--adaptive", action="store_true", help="single-partition runs: the solver chooses its own steps between the points of the --dt grid")
    r.add_argument("--verbose", action="store_true")
    r.add_argument("--skip-reference-validation", action="store_true")
    s = sub.add_parser("synth", help="translate an ISCAS .bench gate list into a transistor-level deck")
    s.add_argument("bench", nargs="?", default=None)
    s.add_argument("-o", "--output", default=None)
    s.add_argument("--suite", default=None, metavar="DIR", help="write the generated benchmark suite (auto_synth/, reference_circuits/) to DIR")
    s.add_argument("--only", default=None, help="with --suite: comma list of circuit names (default: all 26)")
    s.add_argument("--circuit", default=None, help="print the deck of one generated benchmark circuit (e.g. c6288, s1238)")
    w = sub.add_parser("sweep", help="PVT sweep over a deck")
    w.add_argument("netlist")
    w.add_argument("--corners", type=int, default=1000)
    w.add_argument("--full-sim", action="store_true")
    w.add_argument("--workers", type=int, default=8)
    w.add_argument("--tstop", type=float, default=200e-12)
    w.add_argument("--dt", type=float, default=1e-12)
    p = sub.add_parser("phase1-report", help="correctness-first benchmark report")
    p.add_argument("--include-extended", action="store_true")
    p.add_argument("--include-large", action="store_true", help="also the suite entries of up to 6 000 transistors (about a minute)")
    p.add_argument("--include-partitioned", action="store_true", help="also five cases run in partitions, as threads and as processes")
    p.add_argument("--include-huge", action="store_true", help="also the seven largest suite entries (12 000 to 150 000 transistors, up to ten minutes each)")
    p.add_argument("--jobs", type=int, default=1, help="cases run at a time")
    p.add_argument("--output-json", default="artifacts/phase1_benchmark_report.json")
    p.add_argument("--output-md", default="artifacts/phase1_benchmark_report.md")
    d = sub.add_parser("dc", help="DC transfer curves: sweep the voltage source on one net")
    d.add_argument("netlist")
    d.add_argument("--source", required=True, help="net held by the source to sweep (against ground)")
    d.add_argument("--start", type=float, default=0.0)
    d.add_argument("--stop", type=float, default=1.8)
    d.add_argument("--step", type=float, default=0.05)
    d.add_argument("--process", default="TT")
    d.add_argument("--vdd", type=float, default=1.8)
    d.add_argument("--temp", type=float, default=27.0)
    d.add_argument("--output", default=None, help="CSV file (first column: the swept voltage)")
    v = sub.add_parser("view", help="show a .nz waveform file")
    v.add_argument("file")
    v.add_argument("--nodes", nargs="*")
    v.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    return {"build": invoke_build, "run": invoke_run, "synth": invoke_synth, "sweep": invoke_sweep, "phase1-report": invoke_phase1_report,
            "view": invoke_view, "dc": invoke_dc}[args.command](args)


if __name__ == "__main__":
    sys.exit(main())
