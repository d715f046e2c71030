"""The generated benchmark circuits: every gate-level description computes the function it is named for (checked with a
plain Python evaluation of the .bench text), the decks synthesised from them parse, and the transistor-level solution of a
small one agrees with the logic."""
import json
import os
import random
import re

import pytest

from nangila_spice import benchcircuits as bc
from nangila_spice.synth import bench_to_spice

N = pytest.importorskip("nangila_spice._native")


def evaluate(bench: str, values: dict) -> dict:
    """Logic values of every net of a combinational .bench description (flip-flop outputs are read from ``values``)."""
    ops = {"AND": lambda v: int(all(v)), "NAND": lambda v: 1 - int(all(v)), "OR": lambda v: int(any(v)), "NOR": lambda v: 1 - int(any(v)),
           "NOT": lambda v: 1 - v[0], "BUFF": lambda v: v[0], "XOR": lambda v: sum(v) & 1, "XNOR": lambda v: 1 - (sum(v) & 1)}
    nets = dict(values)
    gates = []
    for line in bench.splitlines():
        m = re.match(r"(\w+) = (\w+)\((.*)\)", line.strip())
        if m and m.group(2) != "DFF":
            gates.append((m.group(1), m.group(2), [a.strip() for a in m.group(3).split(",")]))
    pending = gates
    while pending:
        rest = []
        for out, kind, ins in pending:
            if all(i in nets for i in ins):
                nets[out] = ops[kind]([nets[i] for i in ins])
            else:
                rest.append((out, kind, ins))
        assert len(rest) < len(pending), "combinational loop or undriven net"
        pending = rest
    return nets


def bits(x, n):
    return [(x >> i) & 1 for i in range(n)]


def test_adder_multiplier_alu_compute_arithmetic():
    rng = random.Random(1)
    n = 6
    text = bc.adder(n)
    for _ in range(40):
        a, b, c = rng.randrange(1 << n), rng.randrange(1 << n), rng.randrange(2)
        v = evaluate(text, {**{f"a{i}": x for i, x in enumerate(bits(a, n))}, **{f"b{i}": x for i, x in enumerate(bits(b, n))}, "cin": c})
        got = sum(v[f"s{i}"] << i for i in range(n)) + (v["cout"] << n)
        assert got == a + b + c
    n = 5
    text = bc.multiplier(n)
    for _ in range(60):
        a, b = rng.randrange(1 << n), rng.randrange(1 << n)
        v = evaluate(text, {**{f"a{i}": x for i, x in enumerate(bits(a, n))}, **{f"b{i}": x for i, x in enumerate(bits(b, n))}})
        assert sum(v[f"p{i}"] << i for i in range(2 * n)) == a * b
    n = 4
    text = bc.alu(n)
    for _ in range(60):
        a, b, op, c = rng.randrange(1 << n), rng.randrange(1 << n), rng.randrange(4), rng.randrange(2)
        v = evaluate(text, {**{f"a{i}": x for i, x in enumerate(bits(a, n))}, **{f"b{i}": x for i, x in enumerate(bits(b, n))},
                            "op0": op & 1, "op1": op >> 1, "cin": c})
        want = [a & b, a | b, a ^ b, (a + b + c) & ((1 << n) - 1)][op]
        assert sum(v[f"y{i}"] << i for i in range(n)) == want
        assert v["zero"] == int(want == 0)
        assert v["carry"] == (int(a + b + c >= (1 << n)) if op == 3 else 0)


def test_error_corrector_priority_and_comparator():
    rng = random.Random(2)
    n = 11
    for nand_only in (False, True):
        text = bc.parity_sec(n, nand_only)
        k = len(re.findall(r"INPUT\(r\d+\)", text))
        pos = [p for p in range(1, 64) if p & (p - 1)][:n]
        for _ in range(30):
            data = rng.randrange(1 << n)
            d = bits(data, n)
            check = [sum(d[i] for i in range(n) if pos[i] >> j & 1) & 1 for j in range(k)]
            flip = rng.randrange(-1, n)
            recv = list(d)
            if flip >= 0:
                recv[flip] ^= 1                      # one data bit corrupted in transit
            v = evaluate(text, {**{f"d{i}": x for i, x in enumerate(recv)}, **{f"r{j}": x for j, x in enumerate(check)}, "en": 1})
            assert [v[f"q{i}"] for i in range(n)] == d
    n = 9
    text = bc.priority(n)
    for _ in range(40):
        req, en = rng.randrange(1 << n), rng.randrange(1 << n)
        v = evaluate(text, {**{f"req{i}": x for i, x in enumerate(bits(req, n))}, **{f"en{i}": x for i, x in enumerate(bits(en, n))}})
        act = req & en
        assert v["any"] == int(act != 0)
        if act:
            first = (act & -act).bit_length() - 1
            assert sum(v[f"idx{j}"] << j for j in range((n - 1).bit_length())) == first
    n = 7
    text = bc.comparator_adder(n)
    for _ in range(40):
        a, b, c = rng.randrange(1 << n), rng.randrange(1 << n), rng.randrange(2)
        v = evaluate(text, {**{f"a{i}": x for i, x in enumerate(bits(a, n))}, **{f"b{i}": x for i, x in enumerate(bits(b, n))}, "cin": c})
        s = a + b + c
        assert sum(v[f"s{i}"] << i for i in range(n)) + (v["cout"] << n) == s
        assert (v["a_gt_b"], v["a_eq_b"]) == (int(a > b), int(a == b))
        assert v["parity"] == bin(s & ((1 << n) - 1)).count("1") & 1


def test_s27_next_state_and_sequential_generators():
    # s27 with state (G5, G6, G7) = (0, 1, 0) and inputs (G0..G3) = (1, 0, 1, 0), by hand from the netlist
    v = evaluate(bc.S27_BENCH, {"G0": 1, "G1": 0, "G2": 1, "G3": 0, "G5": 0, "G6": 1, "G7": 0})
    g14 = 0; g8 = g14 & 1; g12 = 1 - (0 | 0); g15 = g12 | g8; g16 = 0 | g8; g9 = 1 - (g16 & g15); g11 = 1 - (0 | g9)  # noqa: E702
    assert (v["G9"], v["G11"], v["G17"], v["G10"], v["G13"]) == (g9, g11, 1 - g11, 1 - (g14 | g11), 1 - (1 | g12))
    for kind in ("counter", "lfsr", "shift"):
        text = bc.sequential(8, 40, kind)
        assert text.count("= DFF(") == 8
        state = {f"q{t}": (t * 3 + 1) & 1 for t in range(8)}
        ins = {m: 1 for m in re.findall(r"INPUT\((\w+)\)", text)}
        v = evaluate(text, {**state, **ins})
        nxt = {m.group(1): v[m.group(2)] for m in re.finditer(r"(\w+) = DFF\((\w+)\)", text)}
        if kind == "counter":   # enabled by i0 = 1: the state increments
            cur = sum(state[f"q{t}"] << t for t in range(8))
            assert sum(nxt[f"q{t}"] << t for t in range(8)) == (cur + 1) & 255


def test_suite_decks_and_reference_circuits(tmp_path):
    assert len(bc.SUITE) == 26
    small = ["c17", "c432", "c880", "s27", "s382"]
    paths = bc.write_suite(str(tmp_path), names=small)
    assert len(paths) == len(small) + 4
    for name in small:
        text = (tmp_path / "auto_synth" / f"{name}.sp").read_text()
        js, warnings = N.parse_spice(text, name)
        parsed = json.loads(js)
        assert warnings == [] and len(parsed["node_names"]) > 5, name
    # the large entries are generated too (text only: their decks have up to ~10^5 devices)
    big = bc.bench_text("c6288")
    assert big.count("= AND(") >= 256 and "p31" in big
    assert bc.bench_text("s38417").count("= DFF(") == 1636
    # transistor level agrees with the logic: a 2-bit adder at its DC operating point
    text = bc.adder(2)
    for a, b, c in ((3, 1, 0), (2, 2, 1), (0, 0, 0), (3, 3, 1)):
        vals = {**{f"a{i}": x for i, x in enumerate(bits(a, 2))}, **{f"b{i}": x for i, x in enumerate(bits(b, 2))}, "cin": c}
        stim = [f"V{k} n{net} 0 DC {1.8 * bit}" for k, (net, bit) in enumerate(vals.items())]
        js, _ = N.parse_spice(bench_to_spice(text, "adder2", stimulus=stim), "adder2")
        ok, volt = N.dc_operating_point(js)
        names = json.loads(js)["node_names"]
        total = a + b + c
        assert ok
        for net, bit in (("ns0", total & 1), ("ns1", total >> 1 & 1), ("ncout", total >> 2 & 1)):
            assert abs(volt[names.index(net)] - 1.8 * bit) < 0.06, (a, b, c, net)
    # reference circuits run: the inverter inverts, the SRAM cell flips when written
    ref = bc.reference_circuits()
    assert set(ref) == {"inverter", "sram_6t", "c17_full", "c17_synth"}
    for name in ("inverter", "sram_6t"):
        js, warnings = N.parse_spice(ref[name], name)
        assert warnings == []


def test_evaluate_bench_matches_the_local_evaluator():
    rng = random.Random(3)
    text = bc.alu(3)
    ins = re.findall(r"INPUT\((.*?)\)", text)
    for _ in range(10):
        vals = {i: rng.randint(0, 1) for i in ins}
        assert bc.evaluate_bench(text, vals) == evaluate(text, vals)
    with pytest.raises(ValueError):
        bc.evaluate_bench("INPUT(a)\nx = AND(a, y)\ny = OR(x, a)\n", {"a": 1})


def test_mosfet_model_is_continuous_and_symmetric():
    beta, vth, lam = 1e-3, 0.45, 0.05
    for pmos in (False, True):
        sg = -1.0 if pmos else 1.0
        # no jump of the current at the linear / saturation boundary, derivatives agree with finite differences
        vgs = sg * 1.2
        for vds in (0.2, 0.7499, 0.7501, 1.5, -0.3, -0.9):
            i0, gm, gds, _ = N.mosfet_eval(vgs, sg * vds, pmos, vth, beta, lam)
            h = 1e-6
            ip, _, _, _ = N.mosfet_eval(vgs, sg * vds + h, pmos, vth, beta, lam)
            ig, _, _, _ = N.mosfet_eval(vgs + h, sg * vds, pmos, vth, beta, lam)
            assert abs((ip - i0) / h - gds) < 1e-6 + 1e-4 * abs(gds), (pmos, vds)
            assert abs((ig - i0) / h - gm) < 1e-6 + 1e-4 * abs(gm), (pmos, vds)
        lo, _, _, _ = N.mosfet_eval(vgs, sg * (0.75 - 1e-9), pmos, vth, beta, lam)
        hi, _, _, _ = N.mosfet_eval(vgs, sg * (0.75 + 1e-9), pmos, vth, beta, lam)
        assert abs(lo - hi) < 1e-11
        # drain and source trade places: I(vg - vs, vd - vs) = -I(vg - vd, vs - vd)
        fwd, _, _, _ = N.mosfet_eval(sg * 1.0, sg * 0.4, pmos, vth, beta, lam)
        rev, _, _, _ = N.mosfet_eval(sg * 0.6, sg * -0.4, pmos, vth, beta, lam)
        assert abs(fwd + rev) < 1e-15 and (fwd > 0) == (not pmos)


def test_correctness_registry_and_logic_oracle(tmp_path):
    from nangila_spice import correctness as cx

    official = cx.official_correctness_cases()
    assert len(official) == 13 and len({c.name for c in official}) == 13
    assert [c.name for c in cx.phase1_automated_correctness_cases()] == [c.name for c in official]
    assert {c.tier for c in official} == {"passive", "nonlinear", "logic", "large"}
    assert len(cx.extended_phase1_correctness_cases()) == 13
    blocked = cx.blocked_official_correctness_cases()
    assert blocked == []   # every suite entry has a case in some tier
    huge = cx.huge_phase1_correctness_cases()
    assert [c.name for c in huge] == [n + "_auto" for n in ("c6288", "s5378", "s9234", "s13207", "s15850", "s35932", "s38417", "s38584")]
    assert huge[0].dt == 0.125e-12   # the multiplier's hazards need the fine step
    assert {c.tier for c in huge} == {"huge"} and all(1 <= len(c.expected_levels) <= 16 for c in huge)
    large = cx.large_phase1_correctness_cases()
    assert len(large) == 10 and {c.tier for c in large} == {"large"}
    from nangila_spice import benchcircuits as bc

    named = {c.name[:-5] for c in official + cx.extended_phase1_correctness_cases() + large + huge if c.name.endswith("_auto")}
    assert set(bc.SUITE) - named == {"c17"}   # c17 is there as c17_full / c17_synth
    # the reference's names and signatures: cases of the suite are called <name>_auto, the lists take a repository root
    assert {"c432_auto", "c17_full", "c17_synth", "s27_auto", "s382_auto", "s641_auto"} <= {c.name for c in cx.phase1_automated_correctness_cases("/anywhere")}
    assert {"c880_auto", "c1355_auto", "c1908_auto"} <= {c.name for c in cx.extended_phase1_correctness_cases("/anywhere")}
    assert os.path.exists(cx.BlockedCorrectnessCase("c17", "an example").netlist_path)
    assert os.path.exists(official[0].netlist_path) and open(official[0].netlist_path).read() == official[0].deck
    assert all(1 <= len(c.expected_levels) <= 16 for c in large)
    assert [c.deck for c in cx.large_phase1_correctness_cases()] == [c.deck for c in large]   # the random vectors are seeded
    case = next(c for c in cx.extended_phase1_correctness_cases() if c.name == "priority4")
    path = case.materialize(str(tmp_path))
    # this deck used to stop at 68 ps (Newton oscillating across the jump of the old model); now it completes without a single retry
    js, _ = N.parse_spice(case.deck)
    r = N.simulate(js, case.tstop, 1e-12)
    assert r["stats"]["completed"] and r["newton"]["failed"] == 0 and r["newton"]["step_cuts"] == 0
    wave = cx.run_nangila_waveform(path, tstop=case.tstop, dt=case.dt, in_process=True)
    lower = cx.WaveformData(wave.tool, wave.netlist, [n.lower() for n in wave.node_names], wave.times, {k.lower(): v for k, v in wave.traces.items()})
    assert cx.check_logic_levels(case, lower) == []
    wrong = cx.CorrectnessCase(**{**case.__dict__, "expected_levels": (("nany", 0),)})
    assert [w[0] for w in cx.check_logic_levels(wrong, lower)] == ["nany"]
    flat = cx.collect_flattened_nodes(path)
    assert "nany" in flat and "0" not in flat and "vdd" in flat
    alias = tmp_path / "alias.sp"
    alias.write_text("* alias\nV1 in 0 DC 1\nVA in out 0\nR1 out 0 1k\n.end\n")
    assert cx.collect_observable_nodes(str(alias)) == ["in", "out"]
    assert cx.collect_observable_nodes(str(alias), exclude_zero_volt_alias_sinks=True) == ["in"]


def test_partial_run_raises_unless_allowed(tmp_path):
    from nangila_spice import correctness as cx

    # 1e30 A into a diode: the junction voltage that carries it is out of reach of the limited Newton steps, at any step size
    deck = tmp_path / "hard.sp"
    deck.write_text("* unreachable\nI1 0 a DC 1e30\nD1 a 0 dm\n.model dm D (is=1e-14 n=1)\n.ic V(a)=0\n.end\n")
    with pytest.raises(RuntimeError, match="did not converge"):
        cx.run_nangila_waveform(str(deck), tstop=5e-12, dt=1e-12, in_process=True)
    w = cx.run_nangila_waveform(str(deck), tstop=5e-12, dt=1e-12, in_process=True, allow_partial=True)
    assert len(w.times) == 1 and w.times[0] == 0.0


def test_partitions_keep_transistor_channels_whole_and_logic_runs_partitioned(tmp_path):
    import nangila_spice as ns
    from nangila_spice import correctness as cx
    from nangila_spice.partitioner import partition_flat

    case = next(c for c in cx.extended_phase1_correctness_cases() if c.name == "alu2")
    path = case.materialize(str(tmp_path))
    flat = ns.parse_netlist(path).to_native()
    flat.pop("warnings", None)
    names = flat["node_names"]
    held = {names.index("vdd") + 1}
    for keep, want_cut in ((True, False), (False, True)):
        pr = partition_flat(flat, 4, "spectral", keep_channels=keep)
        assert len(pr.partitions) == 4
        cut = 0
        for el in flat["elements"]:
            if "Mosfet" in el:
                d, s = el["Mosfet"]["d"], el["Mosfet"]["s"]
                if d > 0 and s > 0 and d not in held and s not in held:
                    cut += pr.net_assignment[names[d - 1]] != pr.net_assignment[names[s - 1]]
        assert (cut > 0) == want_cut, (keep, cut)
    res = ns.simulate(path, partitions=4, tstop=1e-9, dt=1e-12)
    assert res.success and res.validation_status == "partitioned_validated", res.warnings
    assert res.solver_stats["stats"]["completed"] and res.solver_stats["stats"]["unconverged_steps"] == 0
    assert res.reference_comparison.max_abs_error < 5e-3


def test_a_large_suite_entry_settles_to_its_gate_level_outputs():
    """One of the ``--include-large`` cases end to end (the 27-channel priority encoder, 740 transistors)."""
    from nangila_spice import correctness as cx
    from nangila_spice.phase1_report import _run_case

    case = next(c for c in cx.official_correctness_cases() if c.name == "c432_auto")
    row = _run_case(case, None)
    assert row["passed"] and row["logic_levels_checked"] == len(case.expected_levels) and row["logic_levels_wrong"] == []
    assert row["oracle"] == "sparse solver, dt / 2 + gate-level logic" and row["max_abs_error_v"] < 0.036


def test_committed_decks_match_the_generators(tmp_path):
    """The decks under ``benchmarks/`` are the generators' output, byte for byte (a sample of the suite, every
    reference circuit), and the smallest example runs."""
    import os

    from nangila_spice import benchcircuits as bc
    from nangila_spice.correctness import run_nangila_waveform

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks")
    for name, text in bc.reference_circuits().items():
        assert open(os.path.join(root, "reference_circuits", name + ".sp")).read() == text, name
    for name in ("c17", "c432", "c1908", "s27", "s382"):
        assert open(os.path.join(root, "auto_synth", name + ".sp")).read() == bc.deck(name), name
    carried = {f[:-3] for f in os.listdir(os.path.join(root, "auto_synth"))}
    assert carried <= set(bc.SUITE) and len(carried) == 19
    wf = run_nangila_waveform(os.path.join(root, "spice_examples", "simple_rc.sp"), tstop=1e-11, dt=1e-12)
    assert abs(wf.traces["vdd"][-1] - 1.8) < 1e-9 and wf.traces["n1"][-1] > 1.7
