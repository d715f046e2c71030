"""Benchmark circuits generated in-tree: gate-level descriptions (ISCAS ``.bench`` syntax) of the kinds of
logic the ISCAS-85 / ISCAS-89 suites are made of, the static-CMOS decks synthesised from them, and three
small transistor-level reference circuits.

The reference ships 27 pre-synthesised ISCAS decks (``benchmarks/auto_synth/*.sp``) and four hand-written
circuits (``benchmarks/reference_circuits/*.sp``) as data files made with an external Yosys flow. Here the
decks are *generated*: every entry of :data:`SUITE` names the ISCAS circuit whose function and size class it
stands in for and builds its own netlist of that function (an n x n array multiplier for c6288, a
single-error-correcting parity network for c499 / c1355, a priority encoder for c432, and so on; counters,
shift registers and LFSRs with combinational clouds for the sequential ones). They are not the ISCAS
netlists themselves, whose gate-for-gate text is not reproduced; c17 and s27, a dozen gates each, are.
``write_suite(dir)`` writes all decks (``python -m nangila_spice.cli synth --suite DIR``).
"""
from __future__ import annotations

import os
import re
from typing import Callable, Dict, List, Tuple

from .synth import C17_BENCH, bench_to_spice

S27_BENCH = """# s27: four inputs, three flip-flops, ten gates
INPUT(G0)
INPUT(G1)
INPUT(G2)
INPUT(G3)
OUTPUT(G17)
G5 = DFF(G10)
G6 = DFF(G11)
G7 = DFF(G13)
G14 = NOT(G0)
G17 = NOT(G11)
G8 = AND(G14, G6)
G15 = OR(G12, G8)
G16 = OR(G3, G8)
G9 = NAND(G16, G15)
G10 = NOR(G14, G11)
G11 = NOR(G5, G9)
G12 = NOR(G1, G7)
G13 = NOR(G2, G12)
"""


class _Bench:
    """Accumulates ``.bench`` lines; every helper returns the name of the net it drives."""

    def __init__(self, title: str):
        self.lines: List[str] = [f"# {title}"]
        self.n = 0
        self.gates = 0

    def inp(self, name: str) -> str:
        self.lines.append(f"INPUT({name})")
        return name

    def out(self, name: str) -> str:
        self.lines.append(f"OUTPUT({name})")
        return name

    def g(self, kind: str, *ins: str, name: str = "") -> str:
        self.n += 1
        self.gates += 1
        name = name or f"w{self.n}"
        self.lines.append(f"{name} = {kind}({', '.join(ins)})")
        return name

    def dff(self, d: str, name: str) -> str:
        self.lines.append(f"{name} = DFF({d})")
        return name

    def xor(self, a: str, b: str, name: str = "") -> str:
        return self.g("XOR", a, b, name=name)

    def full_adder(self, a: str, b: str, c: str) -> Tuple[str, str]:
        p = self.xor(a, b)
        s = self.xor(p, c)
        carry = self.g("NAND", self.g("NAND", a, b), self.g("NAND", p, c))
        return s, carry

    def half_adder(self, a: str, b: str) -> Tuple[str, str]:
        return self.xor(a, b), self.g("AND", a, b)

    def text(self) -> str:
        return "\n".join(self.lines) + "\n"


def adder(n: int) -> str:
    """n-bit ripple-carry adder with carry in: outputs s0..s(n-1), cout."""
    b = _Bench(f"{n}-bit ripple-carry adder")
    a = [b.inp(f"a{i}") for i in range(n)]
    x = [b.inp(f"b{i}") for i in range(n)]
    c = b.inp("cin")
    for i in range(n):
        s, c = b.full_adder(a[i], x[i], c)
        b.g("BUFF", s, name=f"s{i}")
        b.out(f"s{i}")
    b.g("BUFF", c, name="cout")
    b.out("cout")
    return b.text()


def multiplier(n: int) -> str:
    """n x n unsigned array multiplier (rows of adder cells added one partial product at a time, the structure of
    c6288): outputs p0..p(2n-1)."""
    b = _Bench(f"{n} x {n} array multiplier")
    a = [b.inp(f"a{i}") for i in range(n)]
    x = [b.inp(f"b{i}") for i in range(n)]
    pp = [[b.g("AND", a[i], x[j]) for i in range(n)] for j in range(n)]  # pp[j][i] has weight i + j
    outs: List[str] = [pp[0][0]]
    acc: List[str] = pp[0][1:] + [""]          # acc[i] has weight j + i while row j is added; "" = no bit yet
    for j in range(1, n):
        row: List[str] = []
        c = ""
        for i in range(n):
            terms = [t for t in (pp[j][i], acc[i], c) if t]
            if len(terms) == 1:
                s, c = terms[0], ""
            elif len(terms) == 2:
                s, c = b.half_adder(*terms)
            else:
                s, c = b.full_adder(*terms)
            row.append(s)
        outs.append(row[0])
        acc = row[1:] + [c]
    outs += [t for t in acc if t]
    for k, w in enumerate(outs):
        b.g("BUFF", w, name=f"p{k}")
        b.out(f"p{k}")
    return b.text()


def parity_sec(n: int, nand_only: bool = False) -> str:
    """Single-error-correcting network over n data bits (c499; with two-input NANDs only, c1355): check bits
    over Hamming groups, syndrome against the received check bits, corrected data out."""
    b = _Bench(f"{n}-bit single-error-correcting network" + (" (NAND only)" if nand_only else ""))
    k = 1
    while (1 << k) < n + k + 1:
        k += 1
    d = [b.inp(f"d{i}") for i in range(n)]
    r = [b.inp(f"r{j}") for j in range(k)]
    enable = b.inp("en")

    def x2(p: str, q: str) -> str:
        if not nand_only:
            return b.xor(p, q)
        t = b.g("NAND", p, q)
        return b.g("NAND", b.g("NAND", p, t), b.g("NAND", q, t))

    # data bit i sits at Hamming position pos[i] (positions that are not powers of two)
    pos, p = [], 1
    while len(pos) < n:
        if p & (p - 1):
            pos.append(p)
        p += 1
    syn = []
    for j in range(k):
        members = [d[i] for i in range(n) if pos[i] >> j & 1]
        acc = members[0]
        for m in members[1:]:
            acc = x2(acc, m)
        syn.append(x2(acc, r[j]))
    nsyn = [b.g("NOT", s) for s in syn]
    for i in range(n):
        lits = [syn[j] if pos[i] >> j & 1 else nsyn[j] for j in range(k)] + [enable]
        hit = b.g("AND", *lits)
        b.g("BUFF", x2(d[i], hit), name=f"q{i}")
        b.out(f"q{i}")
    return b.text()


def priority(n: int) -> str:
    """n-channel priority encoder with enables (the function class of c432's interrupt controller)."""
    b = _Bench(f"{n}-channel priority encoder")
    req = [b.inp(f"req{i}") for i in range(n)]
    en = [b.inp(f"en{i}") for i in range(n)]
    act = [b.g("AND", req[i], en[i]) for i in range(n)]
    blocked = ""
    grant = []
    for i in range(n):
        grant.append(act[i] if not blocked else b.g("AND", act[i], b.g("NOT", blocked)))
        blocked = act[i] if not blocked else b.g("OR", blocked, act[i])
    bits = max(1, (n - 1).bit_length())
    for j in range(bits):
        members = [grant[i] for i in range(n) if i >> j & 1]
        while len(members) > 1:
            members = [b.g("OR", *members[t:t + 4]) if len(members[t:t + 4]) > 1 else members[t] for t in range(0, len(members), 4)]
        b.g("BUFF", members[0], name=f"idx{j}")
        b.out(f"idx{j}")
    b.g("BUFF", blocked, name="any")
    b.out("any")
    return b.text()


def alu(n: int) -> str:
    """n-bit ALU: op1 op0 select AND / OR / XOR / ADD, plus zero and carry flags (c880 / c3540 / c5315 class)."""
    b = _Bench(f"{n}-bit ALU")
    a = [b.inp(f"a{i}") for i in range(n)]
    x = [b.inp(f"b{i}") for i in range(n)]
    op0, op1, cin = b.inp("op0"), b.inp("op1"), b.inp("cin")
    n0, n1 = b.g("NOT", op0), b.g("NOT", op1)
    sel = [b.g("AND", n1, n0), b.g("AND", n1, op0), b.g("AND", op1, n0), b.g("AND", op1, op0)]
    c = cin
    ys = []
    for i in range(n):
        s, c = b.full_adder(a[i], x[i], c)
        cand = [b.g("AND", a[i], x[i]), b.g("OR", a[i], x[i]), b.xor(a[i], x[i]), s]
        y = b.g("OR", *[b.g("AND", cand[t], sel[t]) for t in range(4)])
        ys.append(b.g("BUFF", y, name=f"y{i}"))
        b.out(f"y{i}")
    z = ys
    while len(z) > 1:
        z = [b.g("OR", *z[t:t + 4]) if len(z[t:t + 4]) > 1 else z[t] for t in range(0, len(z), 4)]
    b.g("NOT", z[0], name="zero")
    b.out("zero")
    b.g("AND", c, sel[3], name="carry")
    b.out("carry")
    return b.text()


def comparator_adder(n: int) -> str:
    """n-bit adder plus magnitude comparator and parity of the sum (c2670 / c7552 class)."""
    b = _Bench(f"{n}-bit adder and comparator")
    a = [b.inp(f"a{i}") for i in range(n)]
    x = [b.inp(f"b{i}") for i in range(n)]
    c = b.inp("cin")
    par = ""
    gt, eq = "", ""
    for i in range(n):
        s, c = b.full_adder(a[i], x[i], c)
        b.g("BUFF", s, name=f"s{i}")
        b.out(f"s{i}")
        par = s if not par else b.xor(par, s)
    for i in reversed(range(n)):
        e = b.g("XNOR", a[i], x[i])
        g = b.g("AND", a[i], b.g("NOT", x[i]))
        gt = g if not gt else b.g("OR", gt, b.g("AND", eq, g))
        eq = e if not eq else b.g("AND", eq, e)
    for src, name in ((c, "cout"), (par, "parity"), (gt, "a_gt_b"), (eq, "a_eq_b")):
        b.g("BUFF", src, name=name)
        b.out(name)
    return b.text()


def sequential(n_ff: int, cloud: int, kind: str = "counter") -> str:
    """A sequential circuit in the ISCAS-89 manner: ``n_ff`` flip-flops (counter, shift register or LFSR next-state
    logic) and a combinational cloud of about ``cloud`` gates mixing state and inputs into a few outputs."""
    b = _Bench(f"{kind} with {n_ff} flip-flops and a {cloud}-gate cloud")
    ins = [b.inp(f"i{t}") for t in range(max(2, min(16, n_ff // 2)))]
    q = [f"q{t}" for t in range(n_ff)]
    if kind == "counter":
        carry = ins[0]
        for t in range(n_ff):
            b.dff(b.xor(q[t], carry), q[t])
            carry = b.g("AND", carry, q[t])
    elif kind == "lfsr":
        fb = b.xor(b.xor(q[-1], q[n_ff // 2]), ins[0])
        b.dff(fb, q[0])
        for t in range(1, n_ff):
            b.dff(q[t - 1], q[t])
    else:  # shift register with parallel load
        for t in range(n_ff):
            src = q[t - 1] if t else ins[1 % len(ins)]
            load = ins[t % len(ins)]
            b.dff(b.g("OR", b.g("AND", src, b.g("NOT", ins[0])), b.g("AND", load, ins[0])), q[t])
    pool = q + ins
    made = 0
    k = 0
    kinds = ("NAND", "NOR", "AND", "OR", "XOR")
    while made < cloud:
        x1, x2, x3 = pool[(7 * k + 1) % len(pool)], pool[(11 * k + 3) % len(pool)], pool[(13 * k + 5) % len(pool)]
        args = (x1, x2) if x1 != x2 else (x1, x3 if x3 != x1 else pool[(k + 1) % len(pool)])
        if args[0] == args[1]:
            k += 1
            continue
        pool.append(b.g(kinds[k % len(kinds)], *args))
        made += 1
        k += 1
    for t in range(min(8, len(pool))):
        b.g("BUFF", pool[-1 - t], name=f"o{t}")
        b.out(f"o{t}")
    return b.text()


# name -> (generator, arguments, what it stands in for)
SUITE: Dict[str, Tuple[Callable[..., str], tuple, str]] = {
    "c17": (lambda: C17_BENCH, (), "c17 itself: six NAND gates"),
    "c432": (priority, (27,), "c432: 27-channel interrupt controller (priority encoder)"),
    "c499": (parity_sec, (32,), "c499: 32-bit single-error-correcting circuit"),
    "c880": (alu, (8,), "c880: 8-bit ALU"),
    "c1355": (parity_sec, (32, True), "c1355: c499 with the XORs expanded into NANDs"),
    "c1908": (parity_sec, (16,), "c1908: 16-bit error detector / corrector"),
    "c2670": (comparator_adder, (12,), "c2670: 12-bit ALU and comparator"),
    "c3540": (alu, (8,), "c3540: 8-bit ALU with BCD logic (ALU only here)"),
    "c5315": (alu, (9,), "c5315: 9-bit ALU"),
    "c6288": (multiplier, (16,), "c6288: 16 x 16 array multiplier"),
    "c7552": (comparator_adder, (32,), "c7552: 32-bit adder / comparator"),
    "s27": (lambda: S27_BENCH, (), "s27 itself: three flip-flops, ten gates"),
    "s382": (sequential, (21, 140, "counter"), "s382: traffic-light controller, 21 flip-flops"),
    "s420": (sequential, (16, 200, "counter"), "s420: 16-bit fractional multiplier control"),
    "s641": (sequential, (19, 350, "shift"), "s641: 19 flip-flops, 379 gates"),
    "s713": (sequential, (19, 380, "shift"), "s713: 19 flip-flops, 393 gates"),
    "s1238": (sequential, (18, 500, "lfsr"), "s1238: 18 flip-flops, 508 gates"),
    "s1423": (sequential, (74, 600, "counter"), "s1423: 74 flip-flops, 657 gates"),
    "s1488": (sequential, (6, 650, "counter"), "s1488: controller, 6 flip-flops, 653 gates"),
    "s5378": (sequential, (179, 2600, "shift"), "s5378: 179 flip-flops, 2779 gates"),
    "s9234": (sequential, (211, 5400, "lfsr"), "s9234: 211 flip-flops, 5597 gates"),
    "s13207": (sequential, (638, 7400, "shift"), "s13207: 638 flip-flops, 7951 gates"),
    "s15850": (sequential, (534, 9300, "lfsr"), "s15850: 534 flip-flops, 9772 gates"),
    "s35932": (sequential, (1728, 15000, "shift"), "s35932: 1728 flip-flops, 16065 gates"),
    "s38417": (sequential, (1636, 21000, "counter"), "s38417: 1636 flip-flops, 22179 gates"),
    "s38584": (sequential, (1426, 18500, "lfsr"), "s38584: 1426 flip-flops, 19253 gates"),
}

INVERTER_SP = """* CMOS inverter driven by a pulse, 10 fF load
VDD vdd 0 DC 1.8
VSS vss 0 DC 0
VIN in 0 PULSE(0 1.8 100p 20p 20p 400p 1n)
MP out in vdd vdd pch w=2u l=180n
MN out in vss vss nch w=1u l=180n
CL out 0 10f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
.tran 1p 2n
.end
"""

SRAM_6T_SP = """* six-transistor SRAM cell: write a 0 then a 1 through the access transistors
VDD vdd 0 DC 1.8
VWL wl 0 PULSE(0 1.8 200p 20p 20p 300p 1n)
VBL bl 0 PULSE(0 1.8 900p 20p 20p 900p 2n)
VBLB blb 0 PULSE(1.8 0 900p 20p 20p 900p 2n)
* cross-coupled inverters
MP1 q qb vdd vdd pch w=0.6u l=180n
MN1 q qb 0 0 nch w=1.2u l=180n
MP2 qb q vdd vdd pch w=0.6u l=180n
MN2 qb q 0 0 nch w=1.2u l=180n
* access transistors
MA1 bl wl q 0 nch w=0.8u l=180n
MA2 blb wl qb 0 nch w=0.8u l=180n
CQ q 0 1f
CQB qb 0 1f
.ic v(q)=1.8 v(qb)=0
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
.tran 1p 2n
.end
"""


def reference_circuits() -> Dict[str, str]:
    """The small hand-written circuits: an inverter, a 6T SRAM cell, c17 at transistor level with pulsed inputs
    (``c17_full``) and with DC inputs (``c17_synth``)."""
    dc = [f"VIN{k} n{name} 0 DC 1.8" for k, name in enumerate(("1", "2", "3", "6", "7"))]
    return {"inverter": INVERTER_SP, "sram_6t": SRAM_6T_SP,
            "c17_full": bench_to_spice(C17_BENCH, "c17, pulsed inputs", period=1e-9) .replace(".end\n", ".tran 2p 16n\n.end\n"),
            "c17_synth": bench_to_spice(C17_BENCH, "c17, all inputs high", stimulus=dc)}


_LOGIC = {"AND": lambda v: int(all(v)), "NAND": lambda v: 1 - int(all(v)), "OR": lambda v: int(any(v)), "NOR": lambda v: 1 - int(any(v)),
          "NOT": lambda v: 1 - v[0], "BUFF": lambda v: v[0], "BUF": lambda v: v[0], "XOR": lambda v: sum(v) & 1, "XNOR": lambda v: 1 - (sum(v) & 1)}


def evaluate_bench(bench: str, values: Dict[str, int]) -> Dict[str, int]:
    """Logic value of every net of a ``.bench`` description for the given primary-input values. Flip-flop outputs
    are inputs of the combinational cloud and are read from ``values`` as well. The logic-level oracle of the
    transistor-level correctness cases."""
    nets = dict(values)
    pending = []
    for line in bench.splitlines():
        m = re.match(r"([^=\s]+)\s*=\s*([A-Za-z]+)\s*\(([^)]*)\)", line.split("#")[0].strip())
        if m and m.group(2).upper() != "DFF":
            pending.append((m.group(1), m.group(2).upper(), [a.strip() for a in m.group(3).split(",") if a.strip()]))
    while pending:
        rest = []
        for out, kind, ins in pending:
            if all(i in nets for i in ins):
                nets[out] = _LOGIC[kind]([nets[i] for i in ins])
            else:
                rest.append((out, kind, ins))
        if len(rest) == len(pending):
            raise ValueError("combinational loop or undriven net: " + ", ".join(o for o, _, _ in rest[:5]))
        pending = rest
    return nets


def bench_text(name: str) -> str:
    gen, args, _ = SUITE[name]
    return gen(*args)


def deck(name: str, **kw) -> str:
    """The static-CMOS deck of one suite entry."""
    return bench_to_spice(bench_text(name), f"{name} ({SUITE[name][2]})", **kw)


def write_suite(directory: str, names=None, with_reference: bool = True) -> List[str]:
    """Writes ``auto_synth/<name>.sp`` for the chosen entries (default: all) and ``reference_circuits/*.sp``."""
    written: List[str] = []
    syn = os.path.join(directory, "auto_synth")
    os.makedirs(syn, exist_ok=True)
    for name in (names or SUITE):
        path = os.path.join(syn, f"{name}.sp")
        with open(path, "w") as fh:
            fh.write(deck(name))
        written.append(path)
    if with_reference:
        ref = os.path.join(directory, "reference_circuits")
        os.makedirs(ref, exist_ok=True)
        for name, text in reference_circuits().items():
            path = os.path.join(ref, f"{name}.sp")
            with open(path, "w") as fh:
                fh.write(text)
            written.append(path)
    return written
