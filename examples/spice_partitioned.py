#!/usr/bin/env python
"""Partitioned transient simulation of a generated RC ladder, checked against the single-matrix solve,
then the same waveform written as a `.nz` file and read back.

    python examples/spice_partitioned.py [--stages 200] [--partitions 4]
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
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        deck = os.path.join(tmp, "ladder.sp")
        with open(deck, "w") as f:
            f.write(generate_rc_ladder_netlist(args.stages, 1e3, 10e-15))
        res = ns.simulate(deck, partitions=args.partitions, tstop=args.tstop, dt=1e-12)
        print(res.summary())
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
