"""Gate-level to transistor-level translation: an ISCAS ``.bench`` description (``INPUT(a)``,
``OUTPUT(y)``, ``y = NAND(a, b)``) becomes a static-CMOS SPICE deck the simulator can run.

The reference produces such decks with an external Yosys flow (``nangila {synth}``,
``benchmarks/synthesize_all.py``) and ships the results as data; this module is the in-tree
generator. Supported gates: NOT, BUFF, NAND, NOR, AND, OR, XOR, XNOR (any fan-in for the first
six); DFF is cut into a pseudo input / output pair, as combinational test decks do.
"""
from __future__ import annotations

import re
from typing import Iterable

C17_BENCH = """# c17: six NAND gates
INPUT(1)
INPUT(2)
INPUT(3)
INPUT(6)
INPUT(7)
OUTPUT(22)
OUTPUT(23)
10 = NAND(1, 3)
11 = NAND(3, 6)
16 = NAND(2, 11)
19 = NAND(11, 7)
22 = NAND(10, 16)
23 = NAND(16, 19)
"""

_MODELS = """.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
"""


def _net(name: str) -> str:
    return "n" + re.sub(r"[^A-Za-z0-9_]", "_", name)


class _Deck:
    def __init__(self, wn: str, wp: str, length: str, cload: str, cint: str = "0.1f"):
        self.lines: list[str] = []
        self.count = 0      # transistors
        self.internal = 0   # nets inside series stacks
        self.wn, self.wp, self.length, self.cload, self.cint = wn, wp, length, cload, cint

    def mos(self, d: str, g: str, s: str, pmos: bool) -> None:
        self.count += 1
        bulk, model, w = ("vdd", "pch", self.wp) if pmos else ("0", "nch", self.wn)
        self.lines.append(f"M{self.count} {d} {g} {s} {bulk} {model} w={w} l={self.length}")

    def tmp(self) -> str:
        """A net between two transistors of a series stack. It gets the diffusion capacitance ``cint``: with none at all
        its voltage is the quotient of two leakage conductances whenever both neighbours are off, which no comparison of
        two runs can pin down."""
        self.internal += 1
        name = f"t{self.internal}"
        if self.cint not in ("", "0"):
            self.lines.append(f"CT{self.internal} {name} 0 {self.cint}")
        return name

    def nand(self, out: str, ins: list[str]) -> None:
        for a in ins:
            self.mos(out, a, "vdd", True)
        prev = out
        for i, a in enumerate(ins):
            nxt = "0" if i == len(ins) - 1 else self.tmp()
            self.mos(prev, a, nxt, False)
            prev = nxt

    def nor(self, out: str, ins: list[str]) -> None:
        for a in ins:
            self.mos(out, a, "0", False)
        prev = "vdd"
        for i, a in enumerate(ins):
            nxt = out if i == len(ins) - 1 else self.tmp()
            self.mos(nxt, a, prev, True)
            prev = nxt

    def inv(self, out: str, a: str) -> None:
        self.mos(out, a, "vdd", True)
        self.mos(out, a, "0", False)

    def gate(self, kind: str, out: str, ins: list[str]) -> None:
        kind = kind.upper()
        if kind in ("NOT", "INV"):
            self.inv(out, ins[0])
        elif kind in ("BUFF", "BUF"):
            t = self.tmp()
            self.inv(t, ins[0])
            self.inv(out, t)
        elif kind == "NAND":
            self.nand(out, ins)
        elif kind == "NOR":
            self.nor(out, ins)
        elif kind == "AND":
            t = self.tmp()
            self.nand(t, ins)
            self.inv(out, t)
        elif kind == "OR":
            t = self.tmp()
            self.nor(t, ins)
            self.inv(out, t)
        elif kind in ("XOR", "XNOR"):
            acc = ins[0]
            for k, b in enumerate(ins[1:]):
                last = k == len(ins) - 2
                t1, t2, t3 = self.tmp(), self.tmp(), self.tmp()
                self.nand(t1, [acc, b])
                self.nand(t2, [acc, t1])
                self.nand(t3, [b, t1])
                x = self.tmp() if (not last or kind == "XNOR") else out
                self.nand(x, [t2, t3])
                acc = x
            if kind == "XNOR":
                self.inv(out, acc)
        else:
            raise ValueError(f"unsupported gate {kind}")
        self.lines.append(f"C{out} {out} 0 {self.cload}")


def bench_to_spice(bench_text: str, title: str = "synthesised", vdd: float = 1.8, period: float = 2e-9, wn: str = "1u", wp: str = "2u",
                   length: str = "180n", cload: str = "2f", stimulus: Iterable[str] = (), cint: str = "0.1f") -> str:
    """Returns the deck. Primary inputs get pulse sources whose periods double from input to input
    (a binary counter over the input vector) unless listed in ``stimulus`` lines. ``cload`` loads every gate output,
    ``cint`` every net inside a series stack ("0": none)."""
    inputs: list[str] = []
    outputs: list[str] = []
    gates: list[tuple[str, str, list[str]]] = []
    for raw in bench_text.splitlines():
        line = raw.split("#")[0].strip()
        if not line:
            continue
        m = re.match(r"(INPUT|OUTPUT)\s*\(\s*([^)]+?)\s*\)$", line, re.I)
        if m:
            (inputs if m.group(1).upper() == "INPUT" else outputs).append(_net(m.group(2)))
            continue
        m = re.match(r"([^=\s]+)\s*=\s*([A-Za-z]+)\s*\(([^)]*)\)$", line)
        if not m:
            raise ValueError(f"cannot parse bench line: {raw!r}")
        out, kind, args = _net(m.group(1)), m.group(2), [_net(a.strip()) for a in m.group(3).split(",") if a.strip()]
        if kind.upper() == "DFF":
            inputs.append(out)
            outputs.append(args[0])
            continue
        gates.append((kind, out, args))
    deck = _Deck(wn, wp, length, cload, cint)
    for kind, out, args in gates:
        deck.gate(kind, out, args)
    lines = [f"* {title}: {len(gates)} gates, {deck.count} transistors", f"VDD vdd 0 DC {vdd}"]
    given = {s.split()[1].lower() for s in stimulus if len(s.split()) > 1}
    for i, name in enumerate(inputs):
        if name.lower() in given:
            continue
        per = period * (2 ** min(i, 24))  # beyond 2^24 periods an input never toggles within any run; also keeps the float finite
        lines.append(f"VIN{i} {name} 0 PULSE(0 {vdd} {per / 4!r} 20p 20p {per / 2!r} {per!r})")
    lines += list(stimulus) + deck.lines + [_MODELS.rstrip(), f"* outputs: {' '.join(outputs)}", ".end"]
    return "\n".join(lines) + "\n"
