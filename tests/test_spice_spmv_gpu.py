"""GPU tests of the circuit simulator's CSR SpMV kernel and device BiCGSTAB against FP64 references
computed on the host (NumPy / SciPy)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _random_csr(n, row_lengths, seed):
    rng = np.random.default_rng(seed)
    row_ptr = np.zeros(n + 1, dtype=np.int32)
    cols, vals = [], []
    for r in range(n):
        k = min(n, int(row_lengths[r]))
        c = np.sort(rng.choice(n, size=k, replace=False)) if k else np.zeros(0, dtype=np.int64)
        cols.append(c.astype(np.int32))
        vals.append(rng.standard_normal(k))
        row_ptr[r + 1] = row_ptr[r] + k
    return row_ptr, np.concatenate(cols) if cols else np.zeros(0, np.int32), np.concatenate(vals) if vals else np.zeros(0)


def _reference(row_ptr, col, val, x):
    y = np.zeros(row_ptr.size - 1)
    prod = val * x[col]
    nz = np.flatnonzero(np.diff(row_ptr))
    y[nz] = np.add.reduceat(prod, row_ptr[:-1][nz]) if prod.size else 0.0
    return y


@pytest.mark.parametrize("plain", [False, True], ids=["bulk", "plain"])
@pytest.mark.parametrize("case", ["short", "mixed", "long", "empty_rows", "dense_ish"])
def test_spmv_matches_host(case, plain):
    from nangila_spice.gpu import DeviceCsr

    rng = np.random.default_rng(1)
    n = 5003
    if case == "short":
        lens = rng.integers(1, 5, n)
    elif case == "mixed":
        lens = rng.integers(0, 70, n)
    elif case == "long":
        lens = rng.integers(1, 6, n)
        lens[[7, 2500, n - 1]] = [3000, 5003, 2049]  # rows longer than one block's capacity
    elif case == "empty_rows":
        lens = np.where(rng.random(n) < 0.7, 0, 3)
    else:
        n = 600
        lens = rng.integers(100, 400, n)
    row_ptr, col, val = _random_csr(n, lens, 2)
    x = rng.standard_normal(n)
    m = DeviceCsr(row_ptr, col, val, plain_loads=plain)
    y = m.matvec(x)
    ref = _reference(row_ptr, col, val, x)
    scale = np.abs(ref).max() + 1.0
    assert np.abs(y - ref).max() / scale < 1e-13
    # device-resident path on torch tensors, and a values-only update
    xd = torch.from_numpy(x).cuda()
    yd = torch.full((n,), float("nan"), dtype=torch.float64, device="cuda")
    m.update_values(val * 2.0)
    m.matvec_device(xd, yd, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    m.check_status()
    assert np.abs(yd.cpu().numpy() - 2.0 * ref).max() / scale < 1e-13
    m.close()


@pytest.mark.parametrize("n", [200_000, 200_001, 7, 2])
def test_tridiagonal_like_reference_benchmark(n):
    """Banded pattern at even, odd and tiny sizes."""
    from nangila_spice.gpu import DeviceCsr, tridiagonal

    row_ptr, col, val = tridiagonal(n)
    m = DeviceCsr(row_ptr, col, val)
    y = m.matvec(np.ones(n))
    assert y[0] == 1.0 and y[-1] == 1.0 and np.all(y[1:-1] == 0.0)
    x = np.random.default_rng(n).standard_normal(n)
    ref = 2.0 * x
    ref[1:] -= x[:-1]
    ref[:-1] -= x[1:]
    assert np.abs(m.matvec(x) - ref).max() < 1e-14
    # an x vector that is only 8-byte aligned
    buf = torch.zeros(n + 1, dtype=torch.float64, device="cuda")
    buf[1:] = torch.from_numpy(x).cuda()
    yd = torch.empty(n, dtype=torch.float64, device="cuda")
    m.matvec_device(buf[1:], yd, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    m.check_status()
    assert np.abs(yd.cpu().numpy() - ref).max() < 1e-14


def test_device_bicgstab_solves_rc_ladder_system():
    from nangila_spice.gpu import DeviceCsr, tridiagonal

    n = 4000
    row_ptr, col, val = tridiagonal(n, diag=2.5, off=-1.0)  # diagonally dominant: G + C/dt of a ladder
    b = np.random.default_rng(3).standard_normal(n)
    m = DeviceCsr(row_ptr, col, val)
    x, iters, rel, ok = m.solve(b, tol=1e-11, max_iter=500)
    assert ok and rel < 1e-11 and iters > 0
    import scipy.sparse as sp
    import scipy.sparse.linalg as spla

    ref = spla.spsolve(sp.csr_matrix((val, col, row_ptr), shape=(n, n)).tocsc(), b)
    assert np.abs(x - ref).max() < 1e-8 * (np.abs(ref).max() + 1.0)
    # the same inputs give the same bits (fixed-order reductions)
    x2, _, _, _ = m.solve(b, tol=1e-11, max_iter=500)
    assert np.array_equal(x, x2)


def test_mna_system_from_the_simulator_on_the_device():
    """The assembled MNA matrix of a generated circuit: device product against the host product."""
    from nangila_spice import _native as N
    from nangila_spice.gpu import DeviceCsr

    size, row_ptr, col, val, rhs = N.mna_matrix(N.generate_circuit("resistor_mesh", 30), 1e-12, 0.0)
    x = np.random.default_rng(4).standard_normal(size)
    m = DeviceCsr(row_ptr, col, val)
    host = np.array(N.csr_spmv(size, row_ptr, col, val, list(x)))
    assert np.abs(m.matvec(x) - host).max() <= 1e-12 * (np.abs(host).max() + 1.0)


def test_transient_simulation_with_the_device_linear_solver():
    """solver="cuda": every Newton iteration's system is solved by the device BiCGSTAB (pattern uploaded
    once, values per iteration); the waveform matches the sparse-LU run."""
    from nangila_spice import _native as N
    from nangila_spice.gpu import enable_device_solver

    enable_device_solver()
    deck = ("* inverter driving a ladder\nVDD vdd 0 DC 1.8\nVIN in 0 PULSE(0 1.8 20p 20p 20p 100p 300p)\n"
            "M1 out in vdd vdd pch w=2u l=180n\nM2 out in 0 0 nch w=1u l=180n\n"
            + "".join(f"R{i} {'out' if i == 0 else 'n%d' % i} n{i + 1} 500\nC{i} n{i + 1} 0 2f\n" for i in range(40))
            + ".model nch NMOS (vto=0.45 kp=200u lambda=0.05)\n.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)\n.end\n")
    js, _ = N.parse_spice(deck)
    ref = N.simulate(js, 150e-12, 1e-12, solver="lu")
    dev = N.simulate(js, 150e-12, 1e-12, solver="cuda")
    assert dev["stats"]["completed"] and not dev["newton"]["cuda_error"]
    assert dev["newton"]["device_solves"] == dev["newton"]["linear_solves"] > 150
    assert dev["newton"]["krylov_fallbacks"] <= dev["newton"]["linear_solves"] // 10
    assert np.abs(np.array(dev["values"]) - np.array(ref["values"])).max() < 1e-6


def test_graph_captured_iteration_agrees_with_the_host_driven_loop(monkeypatch):
    """The CUDA-graph form of the BiCGSTAB iteration (scalars on the device, convergence read every 4th
    iteration) against the loop whose scalars go through the host."""
    from nangila_spice.gpu import DeviceCsr, tridiagonal

    n = 30_001
    row_ptr, col, val = tridiagonal(n, diag=2.2, off=-1.0)
    b = np.random.default_rng(5).standard_normal(n)
    m = DeviceCsr(row_ptr, col, val)
    x_graph, it_graph, rel_graph, ok_graph = m.solve(b, tol=1e-10, max_iter=400)
    monkeypatch.setenv("NANGILA_SPMV_GRAPH", "0")
    x_host, it_host, rel_host, ok_host = m.solve(b, tol=1e-10, max_iter=400)
    assert ok_graph and ok_host and rel_graph < 1e-10 and rel_host < 1e-10
    assert abs(it_graph - it_host) <= 4  # the graph form tests convergence every 4th iteration
    assert np.abs(x_graph - x_host).max() < 1e-8 * (np.abs(x_host).max() + 1.0)
    # a right-hand side of zeros is solved before the first iteration; an unreachable tolerance stops at max_iter
    monkeypatch.delenv("NANGILA_SPMV_GRAPH")
    x0, it0, _, ok0 = m.solve(np.zeros(n))
    assert ok0 and it0 == 0 and not x0.any()
    _, it_cap, _, ok_cap = m.solve(b, tol=1e-30, max_iter=8)
    assert not ok_cap and it_cap <= 8 + 3


def test_solver_process_with_the_device_linear_solver():
    """``nangila-node --solver cuda`` finds the in-tree kernel library by itself and reports where its solves ran."""
    import re
    import subprocess

    from nangila_spice.correctness import find_nangila_binary

    proc = subprocess.run([find_nangila_binary(), "--demo", "--tstop", "3e-11", "--solver", "cuda"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stderr
    m = re.search(r"device linear solver: (\d+) solves on the GPU, (\d+) fell back", proc.stderr)
    assert m and int(m.group(1)) >= 30 and "not usable" not in proc.stderr, proc.stderr
    v = float(re.search(r"V\(cap\) = ([0-9.]+)", proc.stderr).group(1))
    assert abs(v - 1.8 * (1 - 2.718281828 ** -3.0)) < 0.02
