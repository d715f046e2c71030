"""Stress tier for the fused bucket kernel (single-GPU loopback world), after the reference's
tests/test_stress.py:31-234: many iterations on one bucket, a sweep of odd shapes and dtypes, edge values
(zeros, constants, huge, denormal, NaN / Inf), and a sustained-throughput loop."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(world, **kw):
    from nangila.parallel.predres_engine import PredResEngine
    from nangila.parallel.symm import LoopbackArena

    dev = torch.device("cuda", 0)
    kw.setdefault("use_side_stream", False)
    return PredResEngine(LoopbackArena(world, dev), dev, **kw)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_many_iterations_stay_consistent(world):
    """600 calls on one bucket with the gain controller running: replicas identical, values finite, the error
    memory bounded by the gradient scale, no status raised, history equal to the last result when written."""
    n = 4096 * 7 + 123
    eng = _engine(world, stochastic=False, error_feedback=True)
    torch.manual_seed(0)
    base = torch.randn(n, device="cuda") * 0.01
    for step in range(600):
        noise = 0.3 if step % 50 < 25 else 1.0   # alternate between a predictable and a noisy regime
        grads = [(base * (1 + 0.01 * step) + torch.randn(n, device="cuda") * 0.01 * noise).to(torch.bfloat16) for _ in range(world)]
        eng.reduce(0, grads, compressed=step >= 2, step=step)
        eng.end_step()
        if step % 100 == 99:
            eng.check_status()
            for g in grads[1:]:
                assert torch.equal(g, grads[0])
            assert bool(torch.isfinite(grads[0].float()).all())
            st = eng.buckets[0]
            assert st.ef[0].float().abs().max().item() < 0.05
    assert eng.launches == 600


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_shape_sweep(dtype):
    """Odd sizes around every internal boundary (8-element vectors, 64-element blocks, 2048-element iterations,
    chunk size) through the exact and the compressed mode."""
    eng = _engine(2, stochastic=False, error_feedback=True, adaptive_gain=False)
    sizes = [8, 9, 63, 64, 65, 2047, 2048, 2049, 4095, 4096, 4097, 8191, 12288, 12295, 100_003, 262_144, 1_000_001]
    for i, n in enumerate(sizes):
        torch.manual_seed(n)
        grads = [(torch.randn(n, device="cuda") * 0.02).to(dtype) for _ in range(2)]
        exact = torch.stack([g.float() for g in grads]).mean(0)
        eng.reduce(i, grads, compressed=False)
        assert torch.allclose(grads[0].float(), exact, atol=1e-6 if dtype == torch.float32 else 3e-4, rtol=1e-2)
        eng.buckets[i].pred_gain = 0.0
        grads = [(torch.randn(n, device="cuda") * 0.02).to(dtype) for _ in range(2)]
        exact = torch.stack([g.float() for g in grads]).mean(0)
        eng.reduce(i, grads, compressed=True, step=1)
        eng.check_status()
        assert torch.equal(grads[0], grads[1])
        rel = ((grads[0].float() - exact).norm() / exact.norm()).item()
        assert rel < 0.2, (n, dtype, rel)


@pytest.mark.parametrize("world", [1, 2])
def test_edge_values(world):
    n = 4096 * 3
    eng = _engine(world, stochastic=False, error_feedback=True, adaptive_gain=False)
    cases = {
        "zeros": lambda: torch.zeros(n, device="cuda"),
        "constant": lambda: torch.full((n,), 0.125, device="cuda"),
        # the kernels treat |x| > 3.0e38 as non-finite, and the sum over the ranks (taken before the division) must stay finite
        "huge": lambda: torch.full((n,), 2.5e38 / world, device="cuda"),
        "denormal": lambda: torch.full((n,), 1e-41, device="cuda"),
        "one spike": lambda: torch.zeros(n, device="cuda").index_fill_(0, torch.tensor([17], device="cuda"), 1e4),
        "nan and inf": lambda: torch.randn(n, device="cuda").index_fill_(0, torch.tensor([5, 70], device="cuda"), float("nan"))
        .index_fill_(0, torch.tensor([4000], device="cuda"), float("inf")),
    }
    for i, (name, make) in enumerate(cases.items()):
        for dtype in (torch.float32, torch.bfloat16):
            key = 2 * i + (dtype == torch.bfloat16)
            src = make()
            for compressed in (False, True, True):
                grads = [src.to(dtype).clone() for _ in range(world)]
                st = eng.buckets.get(key)
                if st is not None:
                    st.pred_gain = 0.0
                eng.reduce(key, grads, compressed=compressed, step=int(compressed))
                eng.check_status()
                out = grads[0].float()
                assert bool(torch.isfinite(out).all()), (name, dtype, compressed)
                for g in grads[1:]:
                    assert torch.equal(g, grads[0])
                clean = torch.nan_to_num(src.to(dtype).float(), nan=0.0, posinf=0.0, neginf=0.0)
                if name in ("zeros", "denormal"):
                    assert out.abs().max().item() <= 1e-30, (name, dtype)
                elif not compressed:
                    assert torch.allclose(out, clean, rtol=1e-2, atol=1e-30), (name, dtype)
                elif name == "constant":
                    assert torch.allclose(out, clean, rtol=0.08), (name, dtype)


def test_sustained_throughput_loop():
    """200 back-to-back compressed calls on a 64 MB bucket: no status, and the rate stays within 2x of the first
    measurement (the loop of the reference's GB/s test; the number itself belongs to bench/kernel_roofline.py)."""
    eng = _engine(1, stochastic=False, error_feedback=True, adaptive_gain=False)
    n = 32 << 20
    g = (torch.randn(n, device="cuda") * 0.01).to(torch.bfloat16)
    eng.reduce(0, [g], compressed=False)
    eng.buckets[0].pred_gain = 0.0
    times = []
    for rep in range(4):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(50):
            eng.reduce(0, [g], compressed=True, step=rep * 50 + i)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / 50)
    eng.check_status()
    assert max(times) < 2.0 * min(times) + 0.05, times
    gbs = n * 8 / (min(times) * 1e-3) / 1e9
    assert gbs > 1000, gbs
