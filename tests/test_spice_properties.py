"""Property tests of the circuit simulator's native core (hypothesis). Derandomised by default;
``NANGILA_PROPERTY_EXAMPLES=2000`` explores with fresh random examples."""
import os

import numpy as np
import pytest

hypothesis = pytest.importorskip("hypothesis")
N = pytest.importorskip("nangila_spice._native")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from nangila_spice.nz_reader import read_nz_bytes  # noqa: E402

RUN = settings(max_examples=int(os.environ.get("NANGILA_PROPERTY_EXAMPLES", "50")), deadline=None,
               derandomize="NANGILA_PROPERTY_EXAMPLES" not in os.environ)


def _entries(tiny):
    """Matrix entries; with ``tiny`` also values down to the subnormal range, which no circuit produces but a solver
    has to survive (answer correctly or refuse)."""
    plain = st.floats(-2.0, 2.0).map(lambda v: 0.0 if abs(v) < 1e-6 else v)
    return st.one_of(plain, st.sampled_from([5e-324, 2.2e-308, 1e-300, -1e-250, 1e-200])) if tiny else plain


@st.composite
def sparse_systems(draw, tiny=False):
    n = draw(st.integers(1, 28))
    entry = _entries(tiny)
    a = np.zeros((n, n))
    for i in range(n):
        if draw(st.integers(0, 4)) > 0:   # one diagonal in five is structurally absent: the solver has to exchange rows
            a[i, i] = draw(st.floats(0.5, 4.0)) * draw(st.sampled_from([1.0, -1.0, 1e3, 1e-3]))
        for _ in range(draw(st.integers(0, 3))):
            j = draw(st.integers(0, n - 1))
            a[i, j] += draw(entry)
            if draw(st.booleans()):
                a[j, i] += draw(entry)
    b = np.array([draw(entry) * 2.5 for _ in range(n)])
    return a, b


def _backward_error(a, x, b, componentwise, normwise):
    """Largest over the rows of the better of the two usual measures, each divided by its bound."""
    with np.errstate(over="ignore"):   # an answer of 1e300 is allowed to make these products infinite
        resid = np.abs(a @ x - b)
        comp = resid / (np.abs(a) @ np.abs(x) + np.abs(b) + 1e-300)
        norm = resid / (np.abs(a).sum(axis=1) * np.abs(x).max() + np.abs(b) + 1e-300)
        return float(np.minimum(comp / componentwise, norm / normwise).max())


def _csr(a):
    rp, col, val = [0], [], []
    for row in a:
        nz = np.nonzero(row)[0]
        col += nz.tolist()
        val += row[nz].tolist()
        rp.append(len(col))
    return rp, col, val


@RUN
@given(sparse_systems())
def test_factored_lu_solves_what_is_solvable_and_refuses_the_rest(system):
    a, b = system
    n = len(b)
    rp, col, val = _csr(a)
    lu = N.FactoredLU()
    ok, x = lu.solve(n, rp, col, val, b.tolist())
    sv = np.linalg.svd(a, compute_uv=False)
    cond = sv[0] / sv[-1] if sv[-1] > 0 else np.inf
    if cond < 1e9:
        assert ok
        x = np.asarray(x)
        # backward error: the answer solves a nearby system exactly (every row either componentwise or relative to its norm)
        assert _backward_error(a, x, b, 1e-8, 1e-12) <= 1.0
        # the same object solves the pattern again with other values without a new ordering
        ok2, x2 = lu.solve(n, rp, col, [v * 1.25 for v in val], b.tolist())
        assert ok2 and np.allclose(np.asarray(x2) * 1.25, x, rtol=1e-7, atol=1e-9 * (1 + np.abs(x).max()))
        assert lu.stats()["orderings"] == 1
    elif ok:
        # an ill-conditioned or singular system may be answered, but only with finite numbers that do solve it
        x = np.asarray(x)
        assert np.all(np.isfinite(x)) and _backward_error(a, x, b, 1e-5, 1e-9) <= 1.0


@RUN
@given(sparse_systems(tiny=True))
def test_factored_lu_survives_entries_down_to_the_subnormal_range(system):
    a, b = system
    rp, col, val = _csr(a)
    ok, x = N.FactoredLU().solve(len(b), rp, col, val, b.tolist())
    if ok:   # whatever is answered is finite and solves the system; overflowing or singular ones are refused
        x = np.asarray(x)
        assert np.all(np.isfinite(x)) and _backward_error(a, x, b, 1e-5, 1e-9) <= 1.0


@RUN
@given(st.integers(1, 60), st.data())
def test_minimum_degree_order_is_a_permutation_and_singletons_are_pivots(n, data):
    a = np.zeros((n, n), dtype=bool)
    for i in range(n):
        a[i, i] = data.draw(st.booleans())
        for _ in range(data.draw(st.integers(0, 3))):
            a[i, data.draw(st.integers(0, n - 1))] = True
    rp, col = [0], []
    for row in a:
        col += np.nonzero(row)[0].tolist()
        rp.append(len(col))
    assert sorted(N.minimum_degree_order(n, rp, col)) == list(range(n))
    pivots = N.singleton_pivots(n, rp, col)
    rows, cols = [p[0] for p in pivots], [p[1] for p in pivots]
    assert len(set(rows)) == len(rows) and len(set(cols)) == len(cols) and all(a[r, c] for r, c in pivots)
    # each pivot was alone in its row or in its column among what was left at that moment
    live_r, live_c = np.ones(n, bool), np.ones(n, bool)
    for r, c in pivots:
        assert (a[r] & live_c).sum() == 1 or (a[:, c] & live_r).sum() == 1
        live_r[r] = live_c[c] = False


@RUN
@given(st.integers(1, 4), st.integers(2, 120), st.sampled_from([1e-3, 1e-6, 1e-9]), st.data())
def test_nz_container_keeps_its_error_bound(nets, points, bound, data):
    kind = data.draw(st.sampled_from(["smooth", "steps", "noise"]))
    t = np.linspace(0.0, 1e-9, points)
    rng = np.random.default_rng(data.draw(st.integers(0, 2**31)))
    signals = []
    for k in range(nets):
        if kind == "smooth":
            signals.append(1.8 * (1 - np.exp(-t / (1e-10 * (k + 1)))))
        elif kind == "steps":
            signals.append(1.8 * (rng.random(points) > 0.5).astype(float))
        else:
            signals.append(rng.normal(size=points))
    names = [f"n{k}" for k in range(nets)]
    blob, stats = N.nz_compress(names, t.tolist(), [s.tolist() for s in signals], bound)
    back_names, back_t, back, header = N.nz_decompress(blob)
    assert back_names == names and np.allclose(back_t, t, rtol=0, atol=1e-21)
    for s, r in zip(signals, back):
        assert np.abs(np.asarray(r) - s).max() <= bound * (1 + 1e-9)
    py = read_nz_bytes(blob)   # the Python reader decodes the same bytes to the same values
    for k, name in enumerate(names):
        assert np.allclose(py.signals[name], np.asarray(back[k]), rtol=0, atol=1e-15)


@RUN
@given(st.lists(st.tuples(st.integers(1, 2**53 - 1), st.floats(-5.0, 5.0), st.floats(-5.0, 5.0)), min_size=1, max_size=40, unique_by=lambda x: x[0]),
       st.sampled_from([8, 12, 16, 24]))
def test_boundary_codec_error_is_one_quantisation_step(entries, bits):
    updates = [(i, v) for i, v, _ in entries]
    predicted = [(i, p) for i, _, p in entries]
    out = N.codec_roundtrip(updates, predicted, bits)
    assert out["ok"]
    decoded = dict(out["updates"])
    largest = max(abs(v - p) for _, v, p in entries)
    step = largest / (2 ** (bits - 1) - 1) if largest > 0 else 0.0
    for i, v, p in entries:
        if i in decoded:
            assert abs(decoded[i] - v) <= 0.5 * step * (1 + 1e-9) + 1e-15
        else:   # deltas below the codec's floor are not sent: the receiver keeps its prediction
            assert abs(v - p) < 1e-15


@RUN
@given(st.lists(st.tuples(st.floats(0.0, 1e-8), st.floats(-5.0, 5.0)), min_size=1, max_size=12), st.floats(-1e-9, 2e-8))
def test_pwl_source_is_the_interpolant_of_its_increasing_points(points, t):
    """Whatever the card holds (unsorted, repeated times), the source keeps the points whose time increases, is their
    piecewise-linear interpolant, holds the end values outside, and its next corner is the next kept time."""
    import json

    flat = [x for p in points for x in p]
    kept_t, kept_v = [], []
    for pt, pv in points:
        if not kept_t or pt > kept_t[-1]:
            kept_t.append(pt)
            kept_v.append(pv)
    src = json.dumps({"Pwl": {"points": flat}})
    got = N.source_value(src, t)
    want = float(np.interp(t, kept_t, kept_v))
    assert abs(got - want) <= 1e-9 * max(1.0, max(abs(v) for v in kept_v))
    assert min(kept_v) - 1e-12 <= got <= max(kept_v) + 1e-12
    back = json.loads(N.netlist_roundtrip(json.dumps({"name": "p", "num_nodes": 1, "elements": [
        {"VoltageSource": {"pos": 1, "neg": 0, "source": {"Pwl": {"points": flat}}}}], "ghost_map": [], "node_names": ["a"], "initial_conditions": []})))
    assert back["elements"][0]["VoltageSource"]["source"]["Pwl"]["points"] == [x for p in zip(kept_t, kept_v) for x in p]


def _expressions():
    number = st.one_of(st.integers(0, 999).map(str), st.floats(0.001, 999.0).map(lambda v: f"{v:.4g}"),
                       st.sampled_from(["1e-3", "2.5e2", "1e+2", "p", "q"]))

    def combine(children):
        binary = st.tuples(children, st.sampled_from(["+", "-", "*", "/"]), children).map(lambda t: f"{t[0]}{t[1]}{t[2]}")
        power = st.one_of(st.tuples(children, st.sampled_from(["**2", "**3", "**-1"])).map(lambda t: f"({t[0]}){t[1]}"),
                          children.map(lambda c: f"(abs({c}))**0.5"))   # Python turns a root of a negative number into a complex one
        call = st.one_of(children.map(lambda c: f"sqrt(abs({c}))"), st.tuples(children, children).map(lambda t: f"max({t[0]},{t[1]})"),
                         st.tuples(children, children).map(lambda t: f"min({t[0]},{t[1]})"))
        return st.one_of(binary, children.map(lambda c: f"({c})"), children.map(lambda c: f"-({c})"), power, call)

    return st.recursive(number, combine, max_leaves=12)


@RUN
@given(_expressions(), st.booleans())
def test_parameter_arithmetic_agrees_with_python(expr, spaced):
    """An expression over numbers, two parameters, + - * / **, parentheses, sqrt, abs, min and max has the value Python gives it (blanks inside
    the quotes do not matter); one that divides by zero or overflows is refused with a warning instead of a value."""
    import json

    p, q = 3.5, 0.25
    try:
        want = eval(expr, {"__builtins__": {}}, {"p": p, "q": q, "sqrt": np.sqrt, "abs": abs, "min": min, "max": max})  # noqa: S307 - arithmetic only
    except (ZeroDivisionError, OverflowError):
        want = None
    if want is not None and not isinstance(want, complex):
        try:
            want = float(want)   # integers are exact and unbounded in Python
        except OverflowError:
            want = None
    if want is not None and (isinstance(want, complex) or not np.isfinite(want)):
        want = None   # a root of a negative number, an overflow
    shown = expr.replace("+", " + ").replace("*", " * ") if spaced and "e +" not in expr.replace("+", " + ") else expr
    js, warnings = N.parse_spice(f"* arithmetic\n.param p={p} q={q}\nV1 a 0 DC '{shown}'\nR1 a 0 1k\n.end\n")
    got = json.loads(js)["elements"][0]["VoltageSource"]["source"]["Dc"]
    if want is None:
        assert got == 0 and any("cannot evaluate" in w for w in warnings)
    elif abs(abs(want) - 1.8) < 0.21 or abs(abs(want) - 1.0) < 0.21:
        pass  # supply-like values are rescaled with the corner's supply voltage; not what is under test
    else:
        assert abs(got - want) <= 1e-9 * max(1.0, abs(want)), (expr, got, want)
