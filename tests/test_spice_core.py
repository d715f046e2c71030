"""CPU tests of the circuit simulator's native core (nangila_spice._native): devices, sources, MNA,
linear solvers, Newton, transient accuracy against closed forms, parser, predictors, codec, fabric,
.nz container, PVT, balancer, generators. Test plan modelled on the unit tests beside each module of
the reference's nangila-node crate."""
import json
import math

import numpy as np
import pytest

N = pytest.importorskip("nangila_spice._native")


def _rc(ic=True):
    nl = {"name": "rc", "num_nodes": 2, "elements": [
        {"VoltageSource": {"pos": 1, "neg": 0, "source": {"Dc": 1.8}}},
        {"Resistor": {"a": 1, "b": 2, "r": 1000.0}},
        {"Capacitor": {"a": 2, "b": 0, "c": 1e-14}}],
        "ghost_map": [], "node_names": ["vdd", "out"], "initial_conditions": [[1, 1.8], [2, 0.0]] if ic else []}
    return json.dumps(nl)


def test_scale_suffixes():
    assert N.parse_scaled("10k") == 1e4
    assert N.parse_scaled("2.5meg") == 2.5e6
    assert math.isclose(N.parse_scaled("10pF"), 1e-11)
    assert math.isclose(N.parse_scaled("1e-9"), 1e-9)
    assert math.isclose(N.parse_scaled("100f"), 1e-13)
    assert N.parse_scaled("abc") is None


def test_pulse_source_shape():
    src = json.dumps({"Pulse": {"v1": 0.0, "v2": 1.8, "td": 1e-9, "tr": 1e-10, "tf": 2e-10, "pw": 5e-10, "per": 2e-9}})
    assert N.source_value(src, 0.5e-9) == 0.0
    assert math.isclose(N.source_value(src, 1.05e-9), 0.9)
    assert N.source_value(src, 1.3e-9) == 1.8
    assert math.isclose(N.source_value(src, 1.7e-9), 0.9)
    assert N.source_value(src, 1.9e-9) == 0.0
    assert N.source_value(src, 3.3e-9) == 1.8  # second period
    assert N.source_value(json.dumps({"Dc": 0.7}), 123.0) == 0.7


def test_diode_and_mosfet_models():
    i_f, g_f = N.diode_eval(0.7)
    i_l, _ = N.diode_eval(0.1)
    i_r, g_r = N.diode_eval(-1.0)
    assert i_f > 100 * i_l > 0 and g_f > 0
    assert -2e-14 < i_r < 0 and g_r >= 1e-12
    assert N.mosfet_eval(0.2, 1.0)[3] == "Cutoff" and N.mosfet_eval(0.2, 1.0)[0] == 0.0
    id_sat, gm, gds, reg = N.mosfet_eval(1.0, 1.5)
    assert reg == "Saturation" and id_sat > 0 and gm > 0 and gds > 0
    assert math.isclose(id_sat, 0.5 * 1e-3 * 0.25 * (1 + 0.1 * 1.5))
    id_lin, _, _, reg = N.mosfet_eval(1.0, 0.2)
    assert reg == "Linear" and 0 < id_lin < id_sat
    # derivatives match finite differences
    h = 1e-6
    for vgs, vds in ((1.0, 1.5), (1.0, 0.2), (1.2, 0.45)):
        _, gm, gds, _ = N.mosfet_eval(vgs, vds)
        assert math.isclose(gm, (N.mosfet_eval(vgs + h, vds)[0] - N.mosfet_eval(vgs - h, vds)[0]) / (2 * h), rel_tol=1e-4)
        assert math.isclose(gds, (N.mosfet_eval(vgs, vds + h)[0] - N.mosfet_eval(vgs, vds - h)[0]) / (2 * h), rel_tol=1e-4)
    # a PMOS mirrors the NMOS
    idp = N.mosfet_eval(-1.0, -1.5, pmos=True)[0]
    assert math.isclose(idp, -id_sat)


def test_netlist_json_roundtrip_keeps_every_element_kind():
    nl = {"name": "all", "num_nodes": 5, "elements": [
        {"Resistor": {"a": 1, "b": 2, "r": 50.0}}, {"Capacitor": {"a": 2, "b": 0, "c": 1e-12}}, {"Inductor": {"a": 2, "b": 3, "l": 1e-9}},
        {"VoltageSource": {"pos": 1, "neg": 0, "source": {"Pulse": {"v1": 0, "v2": 1, "td": 0, "tr": 1e-12, "tf": 1e-12, "pw": 1e-9, "per": 2e-9}}}},
        {"CurrentSource": {"pos": 0, "neg": 3, "source": {"Dc": 1e-3}}}, {"GhostSource": {"node": 4, "voltage": 0.5}},
        {"Diode": {"p": 3, "n": 0, "model": {"is": 2e-14, "vt": 0.02585, "n": 1.1, "node_p": 3, "node_n": 0}}},
        {"Mosfet": {"d": 5, "g": 3, "s": 0, "b": 0, "model": {"kind": "Pmos", "vth": 0.4, "beta": 2e-3, "lambda": 0.02, "node_g": 3, "node_d": 5, "node_s": 0}}}],
        "ghost_map": [[12345, 4, 1]], "node_names": ["a", "b", "c", "d", "e"], "initial_conditions": [[2, 0.25]]}
    back = json.loads(N.netlist_roundtrip(json.dumps(nl)))
    assert back == nl


@pytest.mark.parametrize("solver", ["lu", "dense", "krylov"])
def test_rc_charging_matches_closed_form(solver):
    r = N.simulate(_rc(), 100e-12, 0.25e-12, solver=solver)
    assert r["stats"]["completed"] and r["stats"]["total_steps"] == 400
    t = np.array(r["time"])
    v = np.array(r["values"])[:, 1]
    assert np.abs(v - 1.8 * (1 - np.exp(-t / 10e-12))).max() < 1e-3
    assert np.allclose(np.array(r["values"])[:, 0], 1.8)


def test_dc_operating_point_is_the_start_without_ic():
    ok, v = N.dc_operating_point(_rc(ic=False))
    assert ok and math.isclose(v[0], 1.8) and math.isclose(v[1], 1.8, rel_tol=1e-6)
    r = N.simulate(_rc(ic=False), 10e-12, 1e-12)
    assert np.allclose(np.array(r["values"])[:, 1], 1.8, atol=1e-6)


def test_rlc_ringing_matches_closed_form():
    # series RLC driven by a step: underdamped response of the capacitor voltage
    R, L, C = 10.0, 1e-9, 1e-12
    nl = {"name": "rlc", "num_nodes": 3, "elements": [
        {"VoltageSource": {"pos": 1, "neg": 0, "source": {"Dc": 1.0}}}, {"Resistor": {"a": 1, "b": 2, "r": R}},
        {"Inductor": {"a": 2, "b": 3, "l": L}}, {"Capacitor": {"a": 3, "b": 0, "c": C}}],
        "ghost_map": [], "node_names": ["in", "m", "out"], "initial_conditions": [[1, 1.0], [2, 1.0], [3, 0.0]]}
    r = N.simulate(json.dumps(nl), 400e-12, 0.05e-12)
    t = np.array(r["time"])
    v = np.array(r["values"])[:, 2]
    alpha, w0 = R / (2 * L), 1 / math.sqrt(L * C)
    wd = math.sqrt(w0 * w0 - alpha * alpha)
    exact = 1 - np.exp(-alpha * t) * (np.cos(wd * t) + alpha / wd * np.sin(wd * t))
    assert np.abs(v - exact).max() < 0.02 and v.max() > 1.5  # it rings above the supply


def test_diode_clamp_and_inverter_converge():
    deck = "* clamp\nV1 in 0 DC 1.8\nR1 in out 1k\nD1 out 0 dm\n.model dm D (is=1e-14 n=1)\n.end\n"
    js, warnings = N.parse_spice(deck)
    ok, v = N.dc_operating_point(js)
    nl = json.loads(js)
    out = v[nl["node_names"].index("out")]
    assert ok and 0.55 < out < 0.8
    i_d, _ = N.diode_eval(out, vt=8.617333e-5 * 300.15)
    assert math.isclose(i_d, (1.8 - out) / 1e3, rel_tol=1e-3)  # KCL at the junction
    inv = ("* inv\nVDD vdd 0 DC 1.8\nVIN in 0 DC {vin}\nM1 out in vdd vdd pch w=2u l=180n\nM2 out in 0 0 nch w=1u l=180n\n"
           ".model nch NMOS (vto=0.45 kp=200u lambda=0.05)\n.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)\n.end\n")
    outs = []
    for vin in (0.0, 0.9, 1.8):
        js, _ = N.parse_spice(inv.format(vin=vin))
        ok, v = N.dc_operating_point(js)
        assert ok
        outs.append(v[json.loads(js)["node_names"].index("out")])
    assert outs[0] > 1.79 and outs[2] < 0.01 and outs[0] > outs[1] > outs[2]


def test_parser_subcircuits_params_continuations_and_ic():
    deck = """my title line
.param rval=2k cval=5f
.subckt stage a b
R1 a b rval
C1 b 0 cval
.ends
V1 in 0 PULSE(0 1.8 0 10p
+ 10p 100p 300p)
X1 in n1 stage
X2 n1 n2 stage
.ic V(n1)=0.3 V(n2)=0.1
.ghost n2 3 1
.end
"""
    js, warnings = N.parse_spice(deck, "t.sp")
    nl = json.loads(js)
    assert warnings == []
    assert nl["node_names"] == ["in", "n1", "n2"] and nl["num_nodes"] == 3
    kinds = [next(iter(e)) for e in nl["elements"]]
    assert kinds == ["VoltageSource", "Resistor", "Capacitor", "Resistor", "Capacitor"]
    assert nl["elements"][1]["Resistor"] == {"a": 1, "b": 2, "r": 2000.0}
    assert math.isclose(nl["elements"][4]["Capacitor"]["c"], 5e-15)
    assert nl["elements"][0]["VoltageSource"]["source"]["Pulse"]["per"] == 300e-12
    assert sorted(map(tuple, nl["initial_conditions"])) == [(2, 0.3), (3, 0.1)]
    assert nl["ghost_map"] == [[N.net_name_hash("N2"), 3, 1]]


def test_parser_pvt_scaling():
    deck = "* m\nVDD vdd 0 DC 1.8\nM1 d g 0 0 nch w=1u l=100n\n.model nch NMOS (vto=0.5 kp=100u)\n.end\n"
    tt = json.loads(N.parse_spice(deck, "m", "TT", 1.8, 27.0)[0])["elements"]
    ff = json.loads(N.parse_spice(deck, "m", "FF", 1.98, 27.0)[0])["elements"]
    hot = json.loads(N.parse_spice(deck, "m", "TT", 1.8, 125.0)[0])["elements"]
    m = lambda els: els[1]["Mosfet"]["model"]  # noqa: E731
    assert math.isclose(m(tt)["vth"], 0.5) and math.isclose(m(tt)["beta"], 100e-6 * 10)
    assert math.isclose(m(ff)["vth"], 0.4) and math.isclose(m(ff)["beta"], 1.15 * m(tt)["beta"])
    assert math.isclose(ff[0]["VoltageSource"]["source"]["Dc"], 1.98)
    assert m(hot)["vth"] < m(tt)["vth"] and m(hot)["beta"] < m(tt)["beta"]


def test_sparse_solvers_agree_and_refine_bad_scaling():
    import scipy.sparse as sp

    rng = np.random.default_rng(0)
    n = 120
    a = (sp.random(n, n, density=0.05, random_state=1, format="csr") + sp.diags(rng.uniform(1, 2, n) * 10.0 ** rng.integers(-6, 12, n))).tocsr()
    a.sort_indices()
    b = rng.standard_normal(n)
    for solver in ("lu", "dense", "krylov"):
        ok, x, _ = N.solve_csr(n, a.indptr.tolist(), a.indices.tolist(), a.data.tolist(), b.tolist(), solver)
        x = np.array(x)
        assert ok
        assert (np.abs(a @ x - b) / (abs(a) @ np.abs(x) + np.abs(b))).max() < (1e-9 if solver == "lu" else 1e-6)
    ok, _, _ = N.solve_csr(2, [0, 1, 2], [0, 0], [1.0, 1.0], [1.0, 1.0], "lu")  # singular
    assert not ok
    y = N.csr_spmv(n, a.indptr.tolist(), a.indices.tolist(), a.data.tolist(), b.tolist())
    assert np.allclose(y, a @ b)


def test_ghost_pin_and_corrections_and_rollback():
    nl = json.loads(_rc())
    nl["elements"] = nl["elements"][1:]  # no source: node 1 becomes a ghost driven from outside
    nl["ghost_map"] = [[777, 1, 1]]
    nl["initial_conditions"] = [[2, 0.0]]
    inject = [(1, 0.0, [(777, 1.0)])]
    r = N.simulate(json.dumps(nl), 60e-12, 1e-12, inject=inject)
    v = np.array(r["values"])
    assert np.allclose(v[1:, 0], 1.0, atol=1e-6)  # pinned to the corrected value (first prediction is flat)
    assert 0.99 < v[-1, 1] < 1.0
    assert r["stats"]["prediction_hits"] + r["stats"]["prediction_misses"] == 1
    # a rollback request before any checkpoint exists is ignored; the run still completes
    r = N.simulate(json.dumps(nl), 10e-12, 1e-12, inject=inject, rollbacks=[0.0])
    assert r["stats"]["completed"]


def test_predictors_classifier_and_confidence():
    g = N.GhostNode(1, 0)
    for k in range(8):  # a ramp is predicted exactly by the linear predictor
        g.apply_correction(0.1 * k, k * 1e-12, 1e-3)
    assert g.signal_class() == "Smooth"
    v, name = g.predict_named(10e-12)
    assert name == "Linear" and math.isclose(v, 1.0, rel_tol=1e-9)
    d = N.GhostNode(2, 0)
    for k in range(10):  # decaying exponential
        d.apply_correction(math.exp(-k / 3.0), k * 1e-12, 1e-3)
    assert d.signal_class() == "Decaying" and d.predict_named(10e-12)[1] == "Exponential"
    assert abs(d.predict(10e-12) - math.exp(-10 / 3.0)) < 0.01
    s = N.GhostNode(3, 0)
    for k in range(10):  # alternating signal
        s.apply_correction((-1) ** k * 0.5, k * 1e-12, 1e-3)
    assert s.signal_class() == "Stiff" and s.predict_named(10e-12)[1] == "RungeKutta"
    c = N.AdaptiveConfidence(6)
    assert c.effective_depth() == 6 and c.confidence_for(9) == 0.5
    for _ in range(40):
        c.update(1, True)
    deep = c.effective_depth()
    c.update(2, False)
    assert deep > 6 and c.effective_depth() < deep and c.effective_depth() >= 1
    ctl = N.SpeculativeDepthController(8, 1, 16)
    for _ in range(64):
        ctl.record_prediction(True)
    assert ctl.depth() == 16
    ctl.record_rollback()
    assert ctl.depth() == 12
    for _ in range(32):
        ctl.record_prediction(False)
    assert ctl.depth() == 1


def test_codec_roundtrip_and_fabric():
    updates = [(1, 1.2345), (2, -0.5), (3, 0.70000000001)]
    predicted = [(1, 1.2), (2, -0.45), (3, 0.7)]
    r = N.codec_roundtrip(updates, predicted)
    got = dict(r["updates"])
    assert r["ok"] and json.loads(r["bytes"])["scale"] > 0
    for k, v in updates:
        assert abs(got[k] - v) <= 0.05 / 32767 + 1e-15  # one quantization step of the largest delta
    assert r["ratio"] > 1.3
    r = N.codec_roundtrip([(1, 1.0)], [(1, 1.0)])
    assert r["skipped"] == 1 and r["updates"] == []
    residuals, done, total = N.fabric_selftest(4, 10)
    assert residuals == 4 * 3 * 10 and done == 4 * 3
    assert math.isclose(total, sum((r + 0.5) * 12 for r in range(10)), rel_tol=1e-4)


def test_nz_container_bound_and_raw_fallback():
    t = np.linspace(0, 1e-9, 1000)
    smooth = 0.9 * (1 - np.exp(-t / 2e-10))
    spiky = np.where((np.arange(1000) % 97) == 0, 50.0, 0.0) * np.sign(np.sin(np.arange(1000)))
    data, st = N.nz_compress(["smooth", "spiky"], t.tolist(), [smooth.tolist(), spiky.tolist()], 1e-5)
    names, time, sig, hdr = N.nz_decompress(data)
    assert names == ["smooth", "spiky"] and hdr["version"] == 2 and np.array_equal(time, t)
    assert np.abs(np.array(sig[0]) - smooth).max() <= 1e-5 * (1 + 1e-9)
    assert np.abs(np.array(sig[1]) - spiky).max() <= 1e-5 * (1 + 1e-9)
    assert st["raw_blocks"] >= 1 and st["predicted_blocks"] >= 4 and st["compression_ratio"] > 1.4
    _, st_smooth = N.nz_compress(["smooth"], t.tolist(), [smooth.tolist()], 1e-5)
    assert st_smooth["raw_blocks"] == 0 and st_smooth["compression_ratio"] > 3.5
    with pytest.raises(RuntimeError):
        N.nz_decompress(b"XXXX" + data[4:])
    with pytest.raises(RuntimeError):
        N.nz_decompress(data[: len(data) // 2])


def test_pvt_delta_cache_and_balancer():
    t = [k * 1e-12 for k in range(5)]
    golden = [[1.8, 0.1 * k] for k in range(5)]
    near = N.pvt_delta(t, golden, "FF", 1.89, 40.0)
    assert near["used_delta_mode"] and near["bytes_roundtrip"]
    scale = 1.89 / 1.8 * math.sqrt(1.15)
    assert math.isclose(near["waveform"][4][1], 0.4 * scale - 0.5e-3 * 13.0)
    far = N.pvt_delta(t, golden, "SS", 1.2, 125.0)
    assert not far["used_delta_mode"] and far["peak_delta_v"] == 0.0
    found, size, hits, misses, evictions = N.pvt_cache_selftest(2, ["a", "b", "c"], ["a", "b", "c"])
    assert found == [False, True, True] and size == 2 and hits == 2 and misses == 1 and evictions == 1
    fast = [1e-3] * 20
    st, plans, score = N.balance_plan([(0, 1000, fast), (1, 1000, fast), (2, 1000, fast), (3, 1000, [4e-3] * 20)])
    assert [s[0] for s in st] == [3] and math.isclose(st[0][1], 4.0)
    assert plans and plans[0][0] == 3 and plans[0][1] in (0, 1, 2) and plans[0][2] == int(1000 * 0.25 * 0.75)
    assert math.isclose(score, 0.75)
    assert N.balance_plan([(0, 10, fast), (1, 10, fast)])[0] == []


def test_generators_and_benchmark_suite():
    lad = json.loads(N.generate_circuit("rc_ladder", 10))
    assert lad["num_nodes"] == 11 and len(lad["elements"]) == 21
    cim = json.loads(N.generate_circuit("cim_array", 4, 5))
    assert cim["num_nodes"] == 9 and len(cim["elements"]) == 4 + 20 + 5
    mesh = N.generate_circuit("resistor_mesh", 6)
    ok, v = N.dc_operating_point(mesh)
    assert ok and math.isclose(v[0], 1.8) and min(v[:36]) == v[35] < 1.8  # the sink corner is the lowest node
    rows = N.run_benchmark_suite()
    assert len(rows) == 4 and all(r["completed"] and r["steps"] == 100 for r in rows)


def test_spmv_row_block_table():
    """Host part of the device SpMV: rows are packed into blocks of at most 2048 non-zeros; a longer
    row stands alone."""
    from nangila_spice.gpu import build_row_blocks, kernels_library, tridiagonal

    try:
        kernels_library()
    except (RuntimeError, OSError):
        pytest.skip("kernel library not built (needs nvcc)")
    rp, col, val = tridiagonal(5000)
    b = build_row_blocks(rp)
    assert b[0] == 0 and b[-1] == 5000 and np.all(np.diff(b) > 0)
    assert np.diff(rp[b]).max() <= 2048 and np.diff(rp[b])[:-1].min() > 2048 - 4
    rp = np.array([0, 3, 5000, 5001, 5001, 9000], dtype=np.int32)
    assert build_row_blocks(rp).tolist() == [0, 1, 2, 4, 5]
    assert build_row_blocks(np.array([0, 0, 0], dtype=np.int32)).tolist() == [0, 2]
    assert col.size == val.size == rp.size * 0 + 3 * 5000 - 2


def _csr(a):
    rp, col, val = [0], [], []
    for row in a:
        nz = np.nonzero(row)[0]
        col += nz.tolist()
        val += row[nz].tolist()
        rp.append(len(col))
    return rp, col, val


def test_factored_lu_matches_numpy_and_reuses_its_analysis():
    rng = np.random.default_rng(7)
    n = 120
    a = np.zeros((n, n))
    for i in range(n):
        a[i, i] = rng.uniform(0.5, 2.0) if rng.random() > 0.25 else 0.0  # zero diagonals need a row exchange
        for j in rng.integers(0, n, 3):
            a[i, j] += rng.normal()
            a[j, i] += rng.normal()
    rp, col, val = _csr(a)
    lu = N.FactoredLU()
    for trial in range(6):
        scale = 1.0 + 0.05 * trial * rng.normal(size=len(val))      # same pattern, drifting values
        v = (np.array(val) * scale).tolist()
        m = np.zeros((n, n))
        for r in range(n):
            for k in range(rp[r], rp[r + 1]):
                m[r, col[k]] = v[k]
        b = rng.normal(size=n)
        ok, x = lu.solve(n, rp, col, v, b.tolist())
        want = np.linalg.solve(m, b)
        assert ok and np.abs(np.array(x) - want).max() <= 1e-9 * np.abs(want).max()
    st = lu.stats()
    assert st["orderings"] == 1 and st["refactors"] >= 6 and st["analyses"] < 6 and st["factor_nnz"] >= len(val)
    # a singular matrix is reported, not solved
    z = np.array([[1.0, 2.0], [2.0, 4.0]])
    rp2, col2, val2 = _csr(z)
    ok, _ = N.FactoredLU().solve(2, rp2, col2, val2, [1.0, 1.0])
    assert not ok
    # a new pattern on the same object starts over
    ok, x = lu.solve(2, [0, 1, 2], [0, 1], [2.0, 4.0], [2.0, 4.0])
    assert ok and x == [1.0, 1.0] and lu.stats()["orderings"] == 2


def test_singleton_pivots_take_out_sources_and_order_is_a_permutation():
    # v1 -- R -- v2 -- R -- ground, source on v1: unknowns (v1, v2, i_src); the source rows are free pivots
    g = 1e-3
    a = np.array([[g, -g, 1.0], [-g, 2 * g, 0.0], [1.0, 0.0, 0.0]])
    rp, col, val = _csr(a)
    piv = N.singleton_pivots(3, rp, col)
    assert (0, 2) in piv or (2, 0) in piv          # column i_src only appears in row v1; row i_src only has column v1
    assert len(piv) == 3                            # everything cascades here
    ok, x = N.FactoredLU().solve(3, rp, col, val, [0.0, 0.0, 1.8])
    assert ok and abs(x[0] - 1.8) < 1e-12 and abs(x[1] - 0.9) < 1e-12
    # a 2-D grid Laplacian: nothing is a singleton, and the order must be a permutation with less fill than the natural one
    k = 12
    n = k * k
    lap = np.zeros((n, n))
    for i in range(k):
        for j in range(k):
            v = i * k + j
            lap[v, v] = 4.1
            for di, dj in ((1, 0), (-1, 0), (0, 1), (0, -1)):
                if 0 <= i + di < k and 0 <= j + dj < k:
                    lap[v, (i + di) * k + j + dj] = -1.0
    rp, col, val = _csr(lap)
    assert N.singleton_pivots(n, rp, col) == []
    order = N.minimum_degree_order(n, rp, col)
    assert sorted(order) == list(range(n))
    lu = N.FactoredLU()
    ok, x = lu.solve(n, rp, col, val, np.ones(n).tolist())
    assert ok and np.abs(lap @ np.array(x) - 1.0).max() < 1e-10
    natural = np.linalg.cholesky(lap)
    assert lu.stats()["factor_nnz"] < 2 * np.count_nonzero(np.abs(natural) > 1e-14)


def test_large_logic_deck_runs_on_the_refactoring_path():
    from nangila_spice import benchcircuits as bc

    js, _ = N.parse_spice(bc.deck("c1355", cload="20f"))
    r = N.simulate(js, 50e-12, 1e-12)
    nr = r["newton"]
    assert r["stats"]["completed"] and nr["lu_fallbacks"] == 0 and nr["lu_singletons"] > 40
    assert nr["lu_analyses"] < nr["lu_refactors"] / 5


def test_long_line_with_underflowing_far_end_stays_on_the_direct_path():
    # 400 RC stages, 100 ps: the far nodes hold voltages that underflow. The backward-error test of the LU must not take
    # that for a bad solve (it once did: the run fell back to cut Backward-Euler steps and was 3.7 mV off).
    from nangila_spice.benchmark import generate_rc_ladder_netlist

    js, _ = N.parse_spice(generate_rc_ladder_netlist(400, 1e3, 10e-15))
    lu = N.simulate(js, 100e-12, 1e-12, 1e-3, "lu")
    dense = N.simulate(js, 100e-12, 1e-12, 1e-3, "dense")
    nr = lu["newton"]
    assert np.abs(np.asarray(lu["values"]) - np.asarray(dense["values"])).max() < 1e-12
    assert nr["step_cuts"] == 0 and nr["be_fallbacks"] == 0 and nr["lu_fallbacks"] == 0 and nr["lu_repivots"] == 0
    assert nr["lu_analyses"] <= 3 and nr["lu_refactors"] <= 4 and nr["lu_reuses"] >= 90   # DC, first (BE) step, trapezoidal steps


def test_partition_files_with_bad_indices_are_rejected():
    good = {"name": "rc", "num_nodes": 2, "node_names": ["a", "b"], "initial_conditions": [],
            "elements": [{"VoltageSource": {"pos": 1, "neg": 0, "source": {"Dc": 1.0}}}, {"Resistor": {"a": 1, "b": 2, "r": 1e3}},
                         {"Capacitor": {"a": 2, "b": 0, "c": 1e-14}}], "ghost_map": []}
    assert N.simulate(json.dumps(good), 5e-12, 1e-12)["stats"]["completed"]
    for mutate, what in ((lambda d: d["elements"][1]["Resistor"].update(b=7), "node outside"),
                         (lambda d: d["elements"][1]["Resistor"].update(a=9e9), "node outside"),
                         (lambda d: d["elements"][1]["Resistor"].update(a=-3), "node outside"),
                         (lambda d: d["elements"][1]["Resistor"].update(r=0.0), "unusable value"),
                         (lambda d: d.update(ghost_map=[[12345, 5, 1]]), "ghost link"),
                         (lambda d: d.update(ghost_map=[[-1.0, 1, 1]]), "out of range"),
                         (lambda d: d.update(initial_conditions=[[3, 1.0]]), "initial condition"),
                         (lambda d: d.update(num_nodes=-4), "num_nodes"),
                         (lambda d: d.update(node_names=["a"]), "fewer node names")):
        bad = json.loads(json.dumps(good))
        mutate(bad)
        with pytest.raises(Exception, match=what):
            N.simulate(json.dumps(bad), 5e-12, 1e-12)


def test_mosfet_overlap_and_junction_capacitances_from_the_model_card():
    deck = """* inverter behind a source resistance
VDD vdd 0 DC 1.8
VIN src 0 PULSE(0 1.8 100p 20p 20p 400p 1n)
RIN src in 5k
M1 out in vdd vdd pch w=2u l=180n
M2 out in 0 0 nch w=1u l=180n
CL out 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05 {caps})
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05 {caps})
.end
"""
    got = {}
    for caps in ("", "cgso=3e-10 cgdo=3e-10 cbd=1f cbs=1f"):
        js, _ = N.parse_spice(deck.format(caps=caps))
        parts = json.loads(js)["elements"]
        r = N.simulate(js, 0.4e-9, 0.5e-12)
        v, names, t = np.asarray(r["values"]), r["node_names"], np.asarray(r["time"])
        out = v[:, names.index("out")]
        got[caps] = (sum("Capacitor" in e for e in parts), out.max(), t[np.argmax(out < 0.9)])
    # cgso, cgdo and cbd per device (cbs would sit between a net and itself here and is left out)
    assert got[""][0] == 1 and got["cgso=3e-10 cgdo=3e-10 cbd=1f cbs=1f"][0] == 7
    caps_run = got["cgso=3e-10 cgdo=3e-10 cbd=1f cbs=1f"]
    widths = [c["Capacitor"]["c"] for c in json.loads(N.parse_spice(deck.format(caps="cgso=3e-10 cgdo=3e-10"))[0])["elements"] if "Capacitor" in c]
    assert sorted(widths)[:4] == pytest.approx([3e-16, 3e-16, 6e-16, 6e-16])   # F/m times the width of each device
    # the gate-drain capacitance couples the rising input into the output (above the rail) and slows the edge
    assert got[""][1] <= 1.8 + 1e-9 and caps_run[1] > 1.82 and caps_run[2] > got[""][2] + 5e-12


def test_type_stub_lists_every_public_name():
    import ast
    import os

    stub = os.path.join(os.path.dirname(N.__file__), "_native.pyi")
    tree = ast.parse(open(stub).read())
    declared = {n.name for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef))} | \
               {n.target.id for n in tree.body if isinstance(n, ast.AnnAssign)}
    public = {n for n in dir(N) if not n.startswith("_")}
    assert public <= declared, sorted(public - declared)
    classes = {n.name: {m.name for m in n.body if isinstance(m, ast.FunctionDef)} for n in tree.body if isinstance(n, ast.ClassDef)}
    assert {"solve", "stats"} <= classes["FactoredLU"] and {"solve", "stats"} <= classes["PvtDeltaSolver"]


def test_adaptive_steps_keep_the_grid_and_the_accuracy():
    # RC step against its closed form: same accuracy as the fixed step, a fraction of the solves
    rc = "* rc\nV1 vdd 0 DC 1.8\nR1 vdd out 1k\nC1 out 0 10f\n.ic V(out)=0\n.end\n"
    js, _ = N.parse_spice(rc)
    fixed = N.simulate(js, 200e-12, 0.25e-12)
    adapt = N.simulate(js, 200e-12, 0.25e-12, adaptive=True)
    t = np.asarray(adapt["time"])
    assert np.array_equal(t, np.asarray(fixed["time"])) and adapt["stats"]["completed"]
    exact = 1.8 * (1.0 - np.exp(-t / 10e-12))
    out = adapt["node_names"].index("out")
    assert np.abs(np.asarray(adapt["values"])[:, out] - exact).max() < 2e-3
    assert adapt["stats"]["solver_steps"] < fixed["stats"]["total_steps"] / 4
    # a pulse train: every corner of the source is a step boundary, so no edge is smeared over a long step
    deck = "* pulse into RC\nV1 in 0 PULSE(0 1.8 1n 20p 20p 2n 6n)\nR1 in out 1k\nC1 out 0 20f\n.end\n"
    js, _ = N.parse_spice(deck)
    fixed = N.simulate(js, 20e-9, 5e-12)
    adapt = N.simulate(js, 20e-9, 5e-12, adaptive=True)
    vf, va = np.asarray(fixed["values"]), np.asarray(adapt["values"])
    assert np.abs(vf - va).max() < 5e-3
    assert adapt["stats"]["solver_steps"] < fixed["stats"]["total_steps"] / 5 and adapt["stats"]["total_steps"] == 4000


def test_adaptive_steps_on_logic_with_long_idle_periods():
    from nangila_spice import benchcircuits as bc
    from nangila_spice.synth import bench_to_spice

    # a 2-bit adder whose inputs toggle every few nanoseconds: almost all of the run is quiet
    deck = bench_to_spice(bc.adder(2), "adder2", cload="20f", period=8e-9)
    js, _ = N.parse_spice(deck)
    names = json.loads(js)["node_names"]
    fixed = N.simulate(js, 40e-9, 2e-12)
    adapt = N.simulate(js, 40e-9, 2e-12, adaptive=True)
    assert adapt["stats"]["completed"] and adapt["stats"]["solver_steps"] < fixed["stats"]["total_steps"] / 2
    obs = [names.index(n) for n in ("ns0", "ns1", "ncout")]
    vf, va = np.asarray(fixed["values"])[:, obs], np.asarray(adapt["values"])[:, obs]
    # same logic levels at every sample away from the edges, and edges within a couple of grid points of each other
    settled = np.abs(vf - 0.9) > 0.8
    assert np.abs(vf - va)[settled].max() < 0.05
    assert np.mean(np.abs(vf - va) > 0.2) < 0.01


def test_sin_exp_and_pwl_sources():
    # value_at of each kind against its definition, and the JSON round trip through a netlist
    sin = {"Sin": {"offset": 0.9, "amplitude": 0.5, "freq": 1e9, "delay": 1e-10, "damping": 2e9, "phase": 30.0}}
    for t in (0.0, 5e-11, 1e-10, 3.3e-10, 1.7e-9):
        want = 0.9 + 0.5 * math.sin(math.radians(30.0)) if t < 1e-10 else \
            0.9 + 0.5 * math.sin(2 * math.pi * 1e9 * (t - 1e-10) + math.radians(30.0)) * math.exp(-(t - 1e-10) * 2e9)
        assert math.isclose(N.source_value(json.dumps(sin), t), want, rel_tol=1e-12, abs_tol=1e-15)
    exp = {"Exp": {"v1": 0.2, "v2": 1.2, "td1": 1e-10, "tau1": 5e-11, "td2": 5e-10, "tau2": 1e-10}}
    for t in (0.0, 1e-10, 2e-10, 5e-10, 9e-10):
        want = 0.2 + (1.0 * (1 - math.exp(-(t - 1e-10) / 5e-11)) if t > 1e-10 else 0.0) - (1.0 * (1 - math.exp(-(t - 5e-10) / 1e-10)) if t > 5e-10 else 0.0)
        assert math.isclose(N.source_value(json.dumps(exp), t), want, rel_tol=1e-12)
    pwl = {"Pwl": {"points": [1e-10, 0.0, 2e-10, 1.8, 2e-10, 5.0, 6e-10, 1.8, 7e-10, 0.6]}}  # the repeated time is dropped
    for t, want in ((0.0, 0.0), (1e-10, 0.0), (1.5e-10, 0.9), (2e-10, 1.8), (4e-10, 1.8), (6.5e-10, 1.2), (7e-10, 0.6), (1.0, 0.6)):
        assert math.isclose(N.source_value(json.dumps(pwl), t), want, abs_tol=1e-12)
    nl = {"name": "s", "num_nodes": 3, "elements": [{"VoltageSource": {"pos": 1, "neg": 0, "source": sin}},
                                                     {"VoltageSource": {"pos": 2, "neg": 0, "source": exp}},
                                                     {"CurrentSource": {"pos": 0, "neg": 3, "source": pwl}},
                                                     {"Resistor": {"a": 3, "b": 0, "r": 1000.0}}],
          "ghost_map": [], "node_names": ["a", "b", "c"], "initial_conditions": []}
    back = json.loads(N.netlist_roundtrip(json.dumps(nl)))
    assert back["elements"][0]["VoltageSource"]["source"] == sin and back["elements"][1]["VoltageSource"]["source"] == exp
    assert back["elements"][2]["CurrentSource"]["source"]["Pwl"]["points"] == [1e-10, 0.0, 2e-10, 1.8, 6e-10, 1.8, 7e-10, 0.6]
    # a transient run follows them: the voltage sources exactly, the current source through its resistor
    res = N.simulate(json.dumps(nl), 1e-9, 1e-12)
    t, v = np.asarray(res["time"]), np.asarray(res["values"])
    assert np.abs(v[:, 0] - [N.source_value(json.dumps(sin), x) for x in t]).max() < 1e-12
    assert np.allclose(v[:, 2], 1000.0 * np.asarray([N.source_value(json.dumps(pwl), x) for x in t]), rtol=1e-8, atol=1e-9)  # gmin to ground
    # the adaptive loop lands on the corners of a PWL source: same waveform as the fixed step
    deck = "* pwl into RC\nV1 in 0 PWL(0 0 1n 0 1.02n 1.8 4n 1.8 4.5n 0.3)\nR1 in out 1k\nC1 out 0 20f\n.end\n"
    js, _ = N.parse_spice(deck)
    fixed, adapt = N.simulate(js, 8e-9, 5e-12), N.simulate(js, 8e-9, 5e-12, adaptive=True)
    assert np.abs(np.asarray(fixed["values"]) - np.asarray(adapt["values"])).max() < 5e-3
    assert adapt["stats"]["solver_steps"] < fixed["stats"]["total_steps"] / 4


def test_parser_reads_sin_exp_pwl_cards():
    deck = ("* sources\n.param amp=0.5\nVS s 0 SIN(0.9 amp 1g 100p)\nIE 0 e EXP(0 1m 100p 50p)\nVP p 0 PWL(0 0, 100p 0, 150p 1.8)\n"
            "VD d 0 DC 1.2 AC 1\nRS s 0 1k\nRE e 0 1k\nRP p 0 1k\nRD d 0 1k\n.end\n")
    js, warnings = N.parse_spice(deck)
    src = {next(iter(e.values()))["pos"] or -next(iter(e.values()))["neg"]: next(iter(e.values()))["source"]
           for e in json.loads(js)["elements"] if "Source" in next(iter(e))}
    names = json.loads(js)["node_names"]
    by_name = {names[abs(k) - 1]: v for k, v in src.items()}
    assert by_name["s"] == {"Sin": {"offset": 0.9, "amplitude": 0.5, "freq": 1e9, "delay": 1e-10, "damping": 0, "phase": 0}}
    assert by_name["e"] == {"Exp": {"v1": 0, "v2": 1e-3, "td1": 1e-10, "tau1": 5e-11, "td2": 1.5e-10, "tau2": 5e-11}}  # SPICE defaults for the fall
    assert by_name["p"] == {"Pwl": {"points": [0, 0, 1e-10, 0, 1.5e-10, 1.8]}}
    assert by_name["d"] == {"Dc": 1.2} and not warnings


def test_first_line_title_rule_and_includes(tmp_path):
    from nangila_spice.parser import parse_netlist, parse_netlist_text

    # a first line that reads like prose is the title even when it starts with an element letter
    for text, title, devices in (("inverter with a 10 fF load\nR1 a 0 1k\nV1 a 0 1\n", "inverter with a 10 fF load", 2),
                                 ("ring oscillator 3 stages\nR1 a 0 1\nV1 a 0 1\n", "ring oscillator 3 stages", 2),
                                 ("I1 0 n1 1m\nR1 n1 0 1k\n", "", 2), ("V1 a 0 DC 1\nR1 a 0 1\n", "", 2),
                                 ("C1 a 0 {cval} ic=0\n.param cval=1p\nV1 a 0 1\n", "", 2), ("VIN in 0 PULSE(0 1.8 100p 20p 20p 400p 1n)\nR1 in 0 1k\n", "", 2)):
        nl = parse_netlist_text(text)
        assert (nl.title or "") == title and nl.num_devices == devices and len(nl.to_native()["elements"]) == devices, text
    # a diode, MOSFET or sub-circuit line has to name something the deck defines; prose with the same field count does not
    cards = ".model dm D (is=1e-14)\n.model nch NMOS (vto=0.45 kp=200u)\n.subckt inv a y\nR1 a y 1k\n.ends\n"
    for text, title, devices in (("Diode bridge rectifier circuit\nR1 a 0 1k\nV1 a 0 1\n", "Diode bridge rectifier circuit", 2),
                                 ("Mixer with two local oscillator inputs\nR1 a 0 1k\nV1 a 0 1\n", "Mixer with two local oscillator inputs", 2),
                                 ("XOR gate test\nR1 a 0 1k\nV1 a 0 1\n", "XOR gate test", 2), ("D1 a 0 dm\nV1 a 0 1\n" + cards, "", 2),
                                 ("M1 d g 0 0 nch w=1u l=180n\nV1 d 0 1\nV2 g 0 1\n" + cards, "", 3), ("X1 a b inv\nV1 a 0 1\nR2 b 0 1k\n" + cards, "", 3)):
        nl = parse_netlist_text(text)
        assert (nl.title or "") == title and nl.num_devices == devices and len(nl.to_native()["elements"]) == devices, text
    # model cards in a library section, a sub-circuit in an included file, both relative to the deck
    (tmp_path / "models").mkdir()
    (tmp_path / "models" / "cmos.lib").write_text(
        "* corners\n.lib tt\n.model nch NMOS (vto=0.45 kp=200u)\n.model pch PMOS (vto=-0.45 kp=100u)\n.endl\n"
        ".lib ss\n.model nch NMOS (vto=0.60 kp=150u)\n.model pch PMOS (vto=-0.60 kp=75u)\n.endl\n")
    (tmp_path / "models" / "inv.sub").write_text(".subckt inv a y vdd\nMP y a vdd vdd pch w=2u l=180n\nMN y a 0 0 nch w=1u l=180n\n.ends\n")
    top = tmp_path / "top.sp"
    top.write_text("inverter with its models in a library\n.lib 'models/cmos.lib' ss\n.include \"models/inv.sub\"\nVDD vdd 0 DC 1.8\n"
                   "VIN in 0 PWL(0 0 100p 0 150p 1.8)\nX1 in out vdd inv\nCL out 0 10f\n.include missing.inc\n.end\n")
    nl = parse_netlist(str(top))
    assert nl.title.startswith("inverter with") and "INV" in nl.subcircuits and nl.num_devices == 4
    native = nl.to_native()
    mos = [e["Mosfet"] for e in native["elements"] if "Mosfet" in e]
    assert len(mos) == 2 and sorted(round(abs(m["model"]["vth"]), 2) for m in mos) == [0.6, 0.6]  # the ss section, not tt
    assert any("missing.inc" in w for w in native["warnings"])
    res = N.simulate(json.dumps({k: v for k, v in native.items() if k != "warnings"}), 6e-10, 1e-12)
    out = np.asarray(res["values"])[:, res["node_names"].index("out")]
    assert out[50] > 1.7 and out[-1] < 0.05
    # the solver process follows the same includes
    import os
    import subprocess

    from nangila_spice.correctness import find_nangila_binary

    proc = subprocess.run([find_nangila_binary(), "--partition", str(top), "--tstop", "6e-10", "--dt", "1e-12", "--waveform-json", str(tmp_path / "w.json")],
                          capture_output=True, text=True, timeout=60)
    assert proc.returncode == 0 and os.path.exists(tmp_path / "w.json"), proc.stderr[-400:]


def test_a_deck_that_includes_itself_ends(tmp_path):
    from nangila_spice.parser import parse_netlist

    deck = tmp_path / "loop.sp"
    (tmp_path / "part.inc").write_text("* a part with its own end card\nR2 a 0 2k\n.include loop.sp\n.end\n")
    deck.write_text("* loop\n.include part.inc\n.include loop.sp\nR1 a 0 1k\nV1 a 0 1\n.end\n")
    nl = parse_netlist(str(deck))  # the cycle is cut, and the `.end` of the included file does not end the deck
    assert sorted(d.name for d in nl.devices) == ["R1", "R2", "V1"]


def test_tran_card_gives_the_default_run_length(tmp_path):
    import subprocess
    import sys

    from nangila_spice.correctness import find_nangila_binary
    from nangila_spice.parser import parse_netlist

    deck = tmp_path / "rc.sp"
    deck.write_text("* rc\nV1 vdd 0 DC 1.8\nR1 vdd out 1k\nC1 out 0 10f\n.ic v(out)=0\n.tran 2p 40p\n.end\n")
    assert parse_netlist(str(deck)).tran() == (2e-12, 40e-12)
    out = tmp_path / "w.json"
    proc = subprocess.run([find_nangila_binary(), "--partition", str(deck), "--waveform-json", str(out)], capture_output=True, text=True, timeout=60)
    assert proc.returncode == 0, proc.stderr[-300:]
    wave = json.loads(out.read_text())["waveform"]
    assert len(wave) == 21 and math.isclose(wave[-1]["time"], 40e-12)
    # flags win over the card, each on its own
    proc = subprocess.run([find_nangila_binary(), "--partition", str(deck), "--dt", "1e-12", "--waveform-json", str(out)], capture_output=True, text=True, timeout=60)
    assert proc.returncode == 0 and len(json.loads(out.read_text())["waveform"]) == 41
    run = subprocess.run([sys.executable, "-m", "nangila_spice.cli", "run", str(deck), "--output-dir", str(tmp_path / "o")], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "21 points" in run.stdout, run.stdout + run.stderr


def test_record_nodes_keeps_the_named_columns_only():
    deck = "* ladder\nV1 a 0 PULSE(0 1.8 10p 5p 5p 40p 100p)\nR1 a b 1k\nC1 b 0 5f\nR2 b c 1k\nC2 c 0 5f\n.end\n"
    js, _ = N.parse_spice(deck)
    full = N.simulate(js, 100e-12, 1e-12)
    for adaptive in (False, True):
        part = N.simulate(js, 100e-12, 1e-12, adaptive=adaptive, record_nodes=["C", "a", "nosuch", "c"])
        assert part["node_names"] == ["c", "a"] and np.asarray(part["values"]).shape == (101, 2)
        ref = N.simulate(js, 100e-12, 1e-12, adaptive=adaptive)
        cols = [ref["node_names"].index(n) for n in ("c", "a")]
        assert np.array_equal(np.asarray(part["values"]), np.asarray(ref["values"])[:, cols])
        assert len(part["final"]) == len(full["final"])  # the final state is whole


def test_solver_process_records_the_named_nets_only(tmp_path):
    import subprocess

    from nangila_spice.correctness import find_nangila_binary, run_nangila_waveform

    deck = tmp_path / "ladder.sp"
    deck.write_text("* ladder\nV1 a 0 PULSE(0 1.8 10p 5p 5p 40p 100p)\nR1 a b 1k\nC1 b 0 5f\nR2 b c 1k\nC2 c 0 5f\n.tran 1p 60p\n.end\n")
    out = tmp_path / "w.json"
    proc = subprocess.run([find_nangila_binary(), "--partition", str(deck), "--record-nodes", "C,a,nosuch", "--waveform-json", str(out),
                           "--waveform-nz", str(tmp_path / "w.nz")], capture_output=True, text=True, timeout=60)
    assert proc.returncode == 0, proc.stderr[-300:]
    d = json.loads(out.read_text())
    assert d["node_names"] == ["c", "a"] and set(d["waveform"][-1]["voltages"]) == {"c", "a"} and len(d["waveform"]) == 61
    assert "V(b)" in proc.stderr   # the final values printed are still those of every net
    from nangila_spice.nz_reader import read_nz

    assert read_nz(str(tmp_path / "w.nz")).node_names == ["c", "a"]
    full = run_nangila_waveform(str(deck), tstop=60e-12, dt=1e-12)
    part = run_nangila_waveform(str(deck), tstop=60e-12, dt=1e-12, nodes=["c"])
    assert part.node_names == ["c"] and np.allclose(part.traces["c"], full.traces["c"], atol=1e-12)


def test_parameter_expressions():
    deck = ("expressions in parameter values\n.param w=1u half='w/2' cl={2*(5f + 5f)} vhi=1.8 neg='-w+3u' tiny='1e-9*2'\nVDD vdd 0 vhi\n"
            "VIN in 0 PULSE(0 vhi 100p 20p 20p 400p 1n)\nM1 out in vdd vdd pch W='2*w' L=180n\nM2 out in 0 0 nch W=half L='0.18u'\n"
            "C1 out 0 cl\nC2 out 0 tiny\nR1 out 0 {1meg * (1 + 1)}\nR2 out 0 'nosuch*2'\nR3 out 0 neg\n"
            ".model nch NMOS (VTO=0.45 KP='100u*2' LAMBDA=0.05)\n.model pch PMOS (VTO=-0.45 KP=100u LAMBDA=0.05)\n.end\n")
    js, warnings = N.parse_spice(deck)
    el = json.loads(js)["elements"]
    beta = [e["Mosfet"]["model"]["beta"] for e in el if "Mosfet" in e]
    assert np.allclose(beta, [100e-6 * 2e-6 / 180e-9, 200e-6 * 0.5e-6 / 0.18e-6])
    caps = [e["Capacitor"]["c"] for e in el if "Capacitor" in e]
    res = [e["Resistor"]["r"] for e in el if "Resistor" in e]
    assert np.allclose(caps, [20e-15, 2e-9]) and np.allclose([res[0], res[2]], [2e6, 2e-6])
    assert len(warnings) == 1 and "nosuch*2" in warnings[0]   # what cannot be evaluated is said, not silently zero
    # powers (right to left, tighter than a leading sign) and the usual functions; what is undefined is refused
    def dc(expr):
        text, notes = N.parse_spice(f"* e\n.param p=3.5 q=0.25\nV1 a 0 DC '{expr}'\nR1 a 0 1k\n.end\n")
        return json.loads(text)["elements"][0]["VoltageSource"]["source"]["Dc"], notes

    for expr, want in (("2**3", 8), ("2^3^2", 512), ("-2**2", -4), ("2*3**2", 18), ("sqrt(16)+abs(-3)", 7), ("max(1, p, q) * min(4, 8)", 14),
                       ("pow(p, 2)", 12.25), ("exp(ln(5))", 5), ("log10(1000)", 3), ("sqrt(2*(p+q))", math.sqrt(7.5)), ("10k/4", 2500)):
        got, notes = dc(expr)
        assert math.isclose(got, want, rel_tol=1e-12) and not notes, expr
    for expr in ("nosuch(3)", "sqrt(-1)", "min()", "pow(2)", "2**", "(1,2)"):
        got, notes = dc(expr)
        assert got == 0 and notes, expr
    # plain numbers with unit text still read as before, and a keyword is not arithmetic
    js, warnings = N.parse_spice("* units\nV1 a 0 DC 1.8V\nR1 a b 10kOhm\nC1 b 0 10pF\n.end\n")
    el = json.loads(js)["elements"]
    assert el[1]["Resistor"]["r"] == 1e4 and math.isclose(el[2]["Capacitor"]["c"], 1e-11) and not warnings


def test_global_nets_reach_into_nested_subcircuits():
    deck = ("* globals\n.global vdd\n.subckt inv a y\nMP y a vdd vdd pch w=2u l=180n\nMN y a 0 0 nch w=1u l=180n\n.ends\n"
            ".subckt buf a y\nX1 a m inv\nX2 m y inv\n.ends\nVDD vdd 0 1.8\nVIN in 0 0\nX1 in out inv\nX2 in out2 buf\n"
            ".model nch NMOS (vto=0.45 kp=200u)\n.model pch PMOS (vto=-0.45 kp=100u)\n.end\n")
    js, warnings = N.parse_spice(deck)
    names = json.loads(js)["node_names"]
    assert names == ["vdd", "in", "out", "out2", "x2.m"] and not warnings   # no private copy of the supply inside an instance
    ok, v = N.dc_operating_point(js)
    assert ok and np.allclose(v[:5], [1.8, 0.0, 1.8, 0.0, 1.8], atol=1e-6)
    from nangila_spice.parser import parse_netlist_text

    flat = parse_netlist_text(deck).flatten()   # the text-level view agrees
    assert sorted({n.lower() for d in flat.devices for n in d.nodes}) == ["0", "in", "out", "out2", "vdd", "x2.m"]


def test_subcircuit_parameters_and_device_multiplier():
    deck = ("* parameters of sub-circuits\n.param r1=10k\n.subckt rdiv top mid r1=1k r2=1k\nR1 top mid r1\nR2 mid 0 'r2*2'\n.ends\n"
            ".subckt two top mid PARAMS: scale=1\nX1 top mid rdiv r1='1k*scale' r2='500*scale'\n.ends\n"
            "V1 a 0 4\nX1 a m1 rdiv\nX2 a m2 rdiv r1=3k r2=500\nX3 a m3 two scale=2\nR9 a 0 r1\n"
            "M1 d g 0 0 nch w=1u l=180n m=4\nVD d 0 1\nVG g 0 1\n.model nch NMOS (vto=0.45 kp=200u)\n.end\n")
    js, warnings = N.parse_spice(deck)
    nl = json.loads(js)
    res = [e["Resistor"]["r"] for e in nl["elements"] if "Resistor" in e]
    # defaults, overrides on the X line, a parameter handed down two levels, and the outer r1 intact afterwards
    assert res == [1e3, 2e3, 3e3, 1e3, 2e3, 2e3, 1e4] and not warnings
    beta = [e["Mosfet"]["model"]["beta"] for e in nl["elements"] if "Mosfet" in e][0]
    assert math.isclose(beta, 4 * 200e-6 * 1e-6 / 180e-9)   # m = 4: four devices in parallel
    ok, v = N.dc_operating_point(js)
    by = dict(zip(nl["node_names"], v))
    assert ok and np.allclose([by["m1"], by["m2"], by["m3"]], [4 * 2 / 3, 1.0, 2.0], atol=1e-6)
    # a sub-circuit that calls itself ends with a warning instead of a stack overflow
    js, warnings = N.parse_spice("* loop\n.subckt a x\nX1 x a\nR1 x 0 1k\n.ends\nV1 n 0 1\nX0 n a\n.end\n")
    assert any("nested more than" in w for w in warnings)
