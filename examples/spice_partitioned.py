#!/usr/bin/env python
"""Partitioned transient simulation of a generated RC ladder, checked against the single-matrix solve,
then the same waveform written as a `.nz` file and read back. With ``--logic`` the deck is a generated 8-bit adder at
transistor level instead, and ``--processes`` runs one solver process per partition (boundary voltages over TCP).

    python examples/spice_partitioned.py [--stages 200] [--partitions 4] [--logic] [--processes]
"""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import nangila_spice as ns  # noqa: E402
from nangila_spice import _native  # noqa: E402
from nangila_spice.benchmark import generate_rc_ladder_netlist  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--stages", type=int, default=200)
    ap.add_argument("--partitions", type=int, default=4)
    ap.add_argument("--tstop", type=float, default=500e-12)
    ap.add_argument("--logic", action="store_true", help="an 8-bit adder at transistor level instead of the ladder")
    ap.add_argument("--processes", action="store_true", help="one nangila-node process per partition")
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        deck = os.path.join(tmp, "ladder.sp")
        with open(deck, "w") as f:
            if args.logic:
                from nangila_spice import benchcircuits
                from nangila_spice.synth import bench_to_spice

                f.write(bench_to_spice(benchcircuits.adder(8), "8-bit adder", cload="20f", period=0.4e-9))
            else:
                f.write(generate_rc_ladder_netlist(args.stages, 1e3, 10e-15))
        res = ns.simulate(deck, partitions=args.partitions, tstop=args.tstop, dt=1e-12, mode="processes" if args.processes else "auto",
                          output_dir=os.path.join(tmp, "run"))
        print(res.summary())
        st = res.solver_stats.get("stats", {})
        if "windows" in st:
            print(f"windows of speculative steps: {st['windows']} ({st['speculated_steps']} steps ahead, {st['discarded_steps']} discarded in "
                  f"{st['rollbacks']} rollbacks), {st['resolves']} relaxation solves, final depth {st['final_depth']}")
        for line in st.get("log_tail", []):
            print("  " + line)
        if not res.success:
            return 1
        w = res.waveform
        names = w.node_names[:8]
        data, stats = _native.nz_compress(names, w.times.tolist(), [w.traces[n].tolist() for n in names], 1e-6)
        path = os.path.join(tmp, "ladder.nz")
        with open(path, "wb") as f:
            f.write(data)
        print(ns.read_nz(path).summary())
    return 0


if __name__ == "__main__":
    sys.exit(main())
