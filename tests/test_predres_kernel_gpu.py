"""GPU tests of the fused prediction-residual bucket kernel in the single-GPU loopback world
(W emulated ranks inside one cooperative launch), against a plain PyTorch FP32 restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(world, **kw):
    from nangila.parallel.predres_engine import PredResEngine
    from nangila.parallel.symm import LoopbackArena

    dev = torch.device("cuda", 0)
    kw.setdefault("use_side_stream", False)
    kw.setdefault("adaptive_gain", False)
    return PredResEngine(LoopbackArena(world, dev), dev, **kw)


from _refmath import bf16_ceil as _bf16_ceil  # noqa: E402
from _refmath import ref_quantize as _ref_quantize  # noqa: E402


def ref_quantize(e, nearest=True):
    return _ref_quantize(e)


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [4096 * 3 + 17, 100_000, 1 << 20])
def test_uncompressed_is_exact_mean(world, dtype, n):
    eng = _engine(world)
    torch.manual_seed(n + world)
    grads = [torch.randn(n, device="cuda").mul_(0.01).to(dtype) for _ in range(world)]
    want = torch.stack([g.float() for g in grads]).mean(0)
    eng.reduce(0, grads, compressed=False)
    eng.check_status()
    tol = 0 if dtype == torch.float32 and world <= 2 else (1e-7 if dtype == torch.float32 else 2e-4)
    for g in grads:
        assert torch.allclose(g.float(), want, atol=max(tol, 1e-9), rtol=1e-2 if dtype == torch.bfloat16 else 1e-6)
    for g in grads[1:]:
        assert torch.equal(g, grads[0])
    st = eng.buckets[0]
    # history: the newest entry (curr after the swap) is the reduced gradient
    for v in range(world):
        assert torch.equal(st.curr[v].float(), grads[0].to(st.state_dtype).float())


@pytest.mark.parametrize("world,gather_max", [(1, 2), (2, 2), (2, 1), (4, 2), (4, 4), (8, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_compressed_matches_reference_math(world, gather_max, dtype):
    """Round-to-nearest mode, no error feedback: out = g_hat + Q(mean_r Q(g_r - g_hat)) in the three-phase
    form, g_hat + mean_r Q(g_r - g_hat) in the gather form (worlds up to ``gather_max``); for a single rank
    out = g_hat + Q(g - g_hat)."""
    n = 4096 * 8 + 4096 * 3 + 100
    eng = _engine(world, stochastic=False, error_feedback=False, state_dtype=torch.float32)
    eng.gather_max_world = gather_max
    torch.manual_seed(7)
    mu = eng.momentum
    hist = []
    for step in range(2):  # two uncompressed steps build the history
        grads = [(torch.randn(n, device="cuda") * 0.02 + 0.01 * step).to(dtype) for _ in range(world)]
        eng.reduce(0, grads, compressed=False, step=step)
        hist.append(grads[0].float().clone())
    prev, curr = hist
    pred = curr + mu * (curr - prev)
    grads = [(pred + torch.randn(n, device="cuda") * 0.005).to(dtype) for _ in range(world)]
    orig = [g.float().clone() for g in grads]
    eng.reduce(0, grads, compressed=True, step=2)
    eng.check_status()
    acc = torch.zeros(n, device="cuda")
    for g in orig:
        deq, _ = ref_quantize(g - pred)
        acc += deq
    if world == 1:  # a single rank does not exchange anything: one quantization, no re-quantized broadcast
        deq2, scale2 = ref_quantize(orig[0] - pred)
    elif world <= gather_max:  # gather mode: every rank sums the W dequantized residuals itself, no second quantization
        deq2 = acc / world
        scale2 = torch.stack([ref_quantize(g - pred)[1] for g in orig]).amax(0)
    else:
        deq2, scale2 = ref_quantize(acc / world)
        scale2 = scale2 * (1.0 + 1.0 / world)  # a tie on one rank moves the mean by step / W before the second rounding
    want = pred + deq2
    got = grads[0].float()
    step_size = scale2.repeat_interleave(64)[:n]
    err = (got - want).abs()
    tol = step_size * 1.01 + (1e-6 if dtype == torch.float32 else 4e-3 * want.abs() + 1e-5)
    assert bool((err <= tol).all()), f"max err {err.max().item()}"
    # at most a small fraction of elements may land one level away (ties under fused multiply-add)
    exact_tol = 1e-6 if dtype == torch.float32 else 4e-3 * want.abs() + 1e-5
    assert (err > exact_tol).float().mean().item() < 5e-3
    for g in grads[1:]:
        assert torch.equal(g, grads[0])  # every rank reconstructs the same bytes
    # quality: the reconstruction is close to the true mean
    true_mean = torch.stack(orig).mean(0)
    rel = (got - true_mean).norm() / true_mean.norm()
    assert rel < 0.05


def test_error_feedback_identity_and_state():
    world, n = 2, 4096 * 5
    eng = _engine(world, stochastic=True, error_feedback=True, state_dtype=torch.float32)
    torch.manual_seed(3)
    grads = [torch.randn(n, device="cuda") * 0.01 for _ in range(world)]
    orig = [g.clone() for g in grads]
    eng.reduce(0, grads, compressed=True, step=0)  # zero history: g_hat = 0
    eng.check_status()
    st = eng.buckets[0]
    # ef = e - deq(q) with e = g (first step): |ef| <= one quantization step of its block
    for v in range(world):
        ef = st.ef[v]
        amax = orig[v].view(-1, 64).abs().amax(1)
        assert bool((ef.view(-1, 64).abs().amax(1) <= _bf16_ceil(amax * 0.14285715) * 1.001).all())
    # new history entry equals the output
    assert torch.equal(st.curr[0], grads[0])
    # unbiasedness of stochastic rounding: mean error far below a quantization step
    bias = (grads[0] - torch.stack(orig).mean(0)).mean().abs().item()
    assert bias < 2e-5


def test_stochastic_rounding_is_unbiased():
    world, n = 1, 1 << 20
    eng = _engine(world, stochastic=True, error_feedback=False, state_dtype=torch.float32)
    base = torch.full((n,), 0.0123, device="cuda")
    base[::64] = 0.07  # sets every block's scale to 0.01
    acc = torch.zeros(n, device="cuda")
    reps = 16
    for step in range(reps):
        g = [base.clone()]
        eng.buckets.clear()  # fresh zero history each time
        eng.reduce(0, g, compressed=True, step=step)
        acc += g[0]
    eng.check_status()
    mean = acc / reps
    assert abs(mean[1::64].mean().item() - 0.0123) < 2e-4


def test_prediction_gain_mean_and_stats():
    world, n = 2, 4096 * 4
    eng = _engine(world, stochastic=False, error_feedback=False, state_dtype=torch.float32)
    torch.manual_seed(11)
    for step in range(2):
        grads = [torch.randn(n, device="cuda") * 0.02 for _ in range(world)]
        eng.reduce(0, grads, compressed=False, step=step)
    st = eng.buckets[0]
    prev, curr = st.prev[0].clone(), st.curr[0].clone()
    pred = curr + eng.momentum * (curr - prev)
    st.extra["pred_gain_per_rank"] = [1.0, 0.0]
    grads = [torch.randn(n, device="cuda") * 0.02 for _ in range(world)]
    orig = [g.clone() for g in grads]
    eng.reduce(0, grads, compressed=True, step=2)
    eng.check_status()
    d0, _ = ref_quantize(orig[0] - pred)
    d1, _ = ref_quantize(orig[1])
    deq2 = (d0 + d1) / 2  # world 2 runs in gather mode: no re-quantization of the mean
    s2 = torch.maximum(ref_quantize(orig[0] - pred)[1], ref_quantize(orig[1])[1])
    want = 0.5 * pred + deq2
    err = (grads[0] - want).abs()
    assert bool((err <= s2.repeat_interleave(64)[:n] * 1.01 + 1e-6).all())
    assert (err > 1e-6).float().mean().item() < 5e-3
    stats = eng.stats_table[st.slot * world].tolist()  # rank 0: kappa = 1, no error feedback
    assert stats[0] == pytest.approx((orig[0] - pred).pow(2).sum().item(), rel=1e-3)
    assert stats[1] == pytest.approx(orig[0].pow(2).sum().item(), rel=1e-3)
    assert stats[2] == pytest.approx((orig[0] * pred).sum().item(), rel=1e-2, abs=1e-3)
    assert stats[3] == pytest.approx(pred.pow(2).sum().item(), rel=1e-3)


class _OneOfTwo:
    """Arena of a two-rank group in which only rank 0 exists: rank 1's buffer is mapped but nobody
    ever launches rank 1's kernel, so the flags rank 0 waits for are never set."""

    world, rank, provider = 2, 0, "test"

    def __init__(self, dev):
        from nangila.parallel.symm import LoopbackArena

        self._inner = LoopbackArena(2, dev)

    def reserve(self, nbytes):
        return None

    def allocate(self, nbytes):
        return self._inner.allocate(nbytes)


def test_wait_times_out_and_reports_status():
    """The host withholds rank 1: rank 0's bounded wait expires, the kernel records what it was
    waiting for and returns, and the context stays usable."""
    from nangila.parallel.predres_engine import PredResEngine

    dev = torch.device("cuda", 0)
    eng = PredResEngine(_OneOfTwo(dev), dev, use_side_stream=False, timeout_s=0.2, adaptive_gain=False)
    n = 4096 * 4
    grads = [torch.randn(n, device="cuda")]
    before = grads[0].clone()
    eng.reduce(0, grads, compressed=False)
    with pytest.raises(RuntimeError, match="timeout in phase"):
        eng.check_status()
    assert torch.equal(grads[0], before)  # nothing was reconstructed, the bucket is untouched
    assert torch.ones(4, device="cuda").sum().item() == 4.0  # the device is still healthy
    # the status block was cleared by the check: a later launch can be diagnosed again
    assert int(eng.status[0][0].item()) == 0


def test_replay_is_deterministic_and_guards_hold(monkeypatch):
    """Two engines fed the same inputs produce the same bytes (outputs, history, error memory), with
    stochastic rounding on; in checked mode the guard blocks behind every symmetric region stay intact."""
    monkeypatch.setenv("NANGILA_CHECKED", "1")
    world, n = 4, 4096 * 9 + 333
    outs = []
    for _ in range(2):
        eng = _engine(world, stochastic=True, error_feedback=True)
        gen = torch.Generator(device="cuda").manual_seed(5)
        for step in range(4):
            grads = [(torch.randn(n, device="cuda", generator=gen) * 0.01).to(torch.bfloat16) for _ in range(world)]
            eng.reduce(0, grads, compressed=step >= 2, step=step)
        eng.check_status()  # includes the guard check
        st = eng.buckets[0]
        outs.append([grads[0].clone(), st.curr[0].clone(), st.prev[0].clone(), st.ef[0].clone()])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_cpp_hook_matches_python_engine_on_one_gpu(monkeypatch):
    """The C++ hook and the Python engine drive the same kernel: identical results for identical inputs
    (single-rank group, round-to-nearest, fixed prediction gain, so nothing is random or adaptive)."""
    import os

    monkeypatch.setenv("NANGILA_PRED_GAIN", "1")
    import socket

    import torch.distributed as dist

    import nangila
    from nangila.parallel.predres_engine import PredResEngine
    from nangila.parallel.symm import SymmArena

    created = False
    if not dist.is_initialized():
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(s.getsockname()[1])
        s.close()
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        created = True
    try:
        dev = torch.device("cuda", 0)
        n = 4096 * 7 + 40
        cpp = nangila.NangilaCppHook(1, 2, None, stochastic=False)
        cpp._attach(dev)
        eng = PredResEngine(SymmArena(None, dev), dev, stochastic=False, use_side_stream=False, adaptive_gain=False)
        eng.fixed_gain = 1.0
        gen = torch.Generator(device="cuda").manual_seed(9)
        for step in range(5):
            g = (torch.randn(n, device="cuda", generator=gen) * 0.01).to(torch.bfloat16)
            a, b = g.clone(), g.clone()
            cpp.run_tensor(0, a).wait()
            eng.reduce(0, [b], compressed=step >= 2, step=step)
            torch.cuda.synchronize()
            cpp.step()
            eng.end_step()
            assert torch.equal(a, b), f"step {step}"
        cpp.check_status()
        assert cpp.get_stats()["compression_enabled"] and cpp.get_kernel_launches() == 5
    finally:
        if created:
            dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("gain", [0.0, 1.0])
def test_split_phase_launches_give_the_same_bytes(world, gain):
    """The phases of one exchange queued as separate launches (what the C++ DDP hook does to defer the
    waiting phases) must reproduce the fused launch bit for bit: same gradients, history and error memory."""
    n = 4096 * 11 + 300
    results = []
    for split in (False, True):
        eng = _engine(world, stochastic=False, error_feedback=True)
        torch.manual_seed(11)
        for step in range(2):
            grads = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(world)]
            eng.reduce(0, grads, compressed=False, step=step)
        eng.buckets[0].pred_gain = gain
        outs = []
        for step in range(2, 5):
            grads = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(world)]
            eng.reduce(0, grads, compressed=True, step=step, split_phases=split)
            outs.append(grads[0].clone())
        eng.check_status()
        st = eng.buckets[0]
        results.append((outs, st.curr[0].clone(), st.prev[0].clone(), st.ef[0].clone()))
        for g in grads[1:]:
            assert torch.equal(g, grads[0])
    (o0, c0, p0, e0), (o1, c1, p1, e1) = results
    for a, b in zip(o0, o1):
        assert torch.equal(a, b)
    assert torch.equal(c0, c1) and torch.equal(p0, p1) and torch.equal(e0, e1)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_history_is_skipped_only_where_nothing_reads_it(world):
    """With a zero gain the kernel may leave the history unwritten between probes. The gradients it
    returns must not depend on that, and the history must be current again by the time a probe reads it."""
    n = 4096 * 6 + 40
    runs = []
    for skip in (True, False):
        eng = _engine(world, stochastic=False, error_feedback=True, adaptive_gain=True)
        eng.probe_every = 8
        eng.skip_history = skip
        torch.manual_seed(5)
        outs = []
        skipped = 0
        for step in range(20):
            grads = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(world)]
            st = eng.buckets.get(0)
            if st is not None:
                st.pred_gain = 0.0
            eng.reduce(0, grads, compressed=step >= 2, step=step)
            st = eng.buckets[0]
            outs.append(grads[0].clone())
            # curr (after the swap) holds this step's result unless the write was skipped
            skipped += int(not torch.equal(st.curr[0].float(), grads[0].float()))
            if step >= 2 and st.calls + 1 >= st.next_probe:
                # the next call is a probe: both history entries must be the last two results
                assert torch.equal(st.curr[0].float(), outs[-1].float())
                assert torch.equal(st.prev[0].float(), outs[-2].float())
        eng.check_status()
        runs.append((outs, skipped))
    for a, b in zip(runs[0][0], runs[1][0]):
        assert torch.equal(a, b)
    assert runs[1][1] == 0 and runs[0][1] > 0


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_packed_bf16_path_against_fp32_reference(world):
    """bf16 gradients with bf16 state and a zero gain take the packed-bf16 arithmetic. Against the FP32
    restatement: never more than one quantization step away, a few per cent of the codes may fall on the
    other side of a tie (g + ef and x / s are rounded to 8 bits), every rank holds the same bytes, and the
    error memory holds exactly what was not sent."""
    n = 4096 * 10
    eng = _engine(world, stochastic=False, error_feedback=True)
    torch.manual_seed(21)
    for step in range(2):
        grads = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(world)]
        eng.reduce(0, grads, compressed=False, step=step)
    st = eng.buckets[0]
    st.pred_gain = 0.0
    for step in range(2, 5):
        grads = [(torch.randn(n, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(world)]
        if step == 4:
            grads[0][17] = float("nan")      # a warp that meets a NaN drops to the FP32 path and zeroes it
            grads[-1][4096 + 5] = float("inf")
        orig = [g.float().clone() for g in grads]
        ef_old = [e.float().clone() for e in st.ef]
        eng.reduce(0, grads, compressed=True, step=step)
        eng.check_status()
        for g in grads[1:]:
            assert torch.equal(g, grads[0])
        assert bool(torch.isfinite(grads[0].float()).all())
        acc = torch.zeros(n, device="cuda")
        smax = torch.zeros((n + 63) // 64, device="cuda")
        for r in range(world):
            x = torch.nan_to_num(orig[r], nan=0.0, posinf=0.0, neginf=0.0) + ef_old[r]
            deq, sc = ref_quantize(x)
            acc += deq
            smax = torch.maximum(smax, sc)
            # error memory: x - (what this rank sent); half a step plus the 8-bit roundings of x and 1 / s (0.07 at |q| = 7)
            assert bool((st.ef[r].float().abs() <= sc.repeat_interleave(64)[:n] * 0.6 + 1e-6).all())
        if world <= eng.gather_max_world:
            want, step_size = acc / world, smax.repeat_interleave(64)[:n]
        else:
            want, s2 = ref_quantize(acc / world)
            # codes of several ranks may fall on the other side of a tie (each moves the mean by step / W) before the
            # second quantization adds its own level
            step_size = s2.repeat_interleave(64)[:n] * 1.6
        err = (grads[0].float() - want).abs()
        tol = 4e-3 * want.abs() + 1e-5
        assert bool((err <= step_size * 1.02 + tol).all()), err.max().item()
        # a block whose largest element rounds differently gets the neighbouring bf16 scale (0.4-0.8 % apart): all its
        # values then move by up to 7 x 0.8 % of a step; only codes on the other side of a tie are further off
        assert (err > tol + 0.07 * step_size).float().mean().item() < 0.08
        if world == 1 and step < 4:
            # one rank: output + new error memory = gradient + old error memory, to bf16 rounding
            resid = grads[0].float() + st.ef[0].float() - (orig[0] + ef_old[0])
            assert bool((resid.abs() <= 8e-3 * (orig[0] + ef_old[0]).abs() + 1e-6).all())
