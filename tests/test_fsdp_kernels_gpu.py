"""GPU tests of the fully-sharded collectives in the single-GPU loopback world."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _arena(world):
    from nangila.parallel.symm import LoopbackArena

    return LoopbackArena(world, torch.device("cuda", 0))


def _bf16_ceil(x):
    b = x.float().view(torch.int32)
    return (((b + 0xFFFF) >> 16) << 16).view(torch.float32)


def ref_int4_nearest(x):
    n = x.numel()
    pad = (-n) % 64
    v = torch.cat([x.float(), x.new_zeros(pad, dtype=torch.float32)]).view(-1, 64)
    s = _bf16_ceil(v.abs().amax(1, keepdim=True) * 0.14285715)
    inv = torch.where(s > 1e-30, 1.0 / s, torch.zeros_like(s))
    q = torch.floor(v * inv + 0.5).clamp_(-8, 7)
    return (q * s).view(-1)[:n], s.view(-1)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shard", [2048 * 3, 40_000, 1 << 18])
def test_reduce_scatter_round_to_nearest(world, dtype, shard):
    from nangila.parallel.fsdp_collectives import NangilaReduceScatter

    rs = NangilaReduceScatter(_arena(world), stochastic=False)
    torch.manual_seed(shard + world)
    n = shard * world
    inputs = [(torch.randn(n, device="cuda") * 0.01).to(dtype) for _ in range(world)]
    outputs = [torch.empty(shard, device="cuda", dtype=dtype) for _ in range(world)]
    for rep in range(2):  # two launches exercise both slot sets
        rs.reduce(outputs, inputs, 1.0 / world)
        rs.check_status()
        for r in range(world):
            acc = torch.zeros(shard, device="cuda")
            step = torch.zeros(shard, device="cuda")
            for src in range(world):
                deq, s = ref_int4_nearest(inputs[src][r * shard:(r + 1) * shard])
                acc += deq
                step += s.repeat_interleave(64)[:shard]
            want = acc / world
            got = outputs[r].float()
            tol = 1e-6 if dtype == torch.float32 else 4e-3 * want.abs() + 1e-6
            err = (got - want).abs()
            assert bool((err <= step / world * 1.01 + tol).all())
            # bf16 buckets use packed-bf16 arithmetic: a few per cent of the codes may fall on the other side of a tie
            # (and a block whose largest element rounds differently gets the neighbouring bf16 scale, 0.4-0.8 % apart)
            slack = 0.0 if dtype == torch.float32 else 0.07 * step / world
            assert (err > tol + slack).float().mean().item() < (5e-3 if dtype == torch.float32 else 0.08)
            exact = torch.stack([i[r * shard:(r + 1) * shard].float() for i in inputs]).mean(0)
            assert ((got - exact).norm() / exact.norm()).item() < 0.12


def test_reduce_scatter_stochastic_unbiased_and_sum():
    from nangila.parallel.fsdp_collectives import NangilaReduceScatter

    world, shard = 2, 1 << 16
    rs = NangilaReduceScatter(_arena(world), stochastic=True)
    x = torch.full((shard * world,), 0.0123, device="cuda")
    x[::64] = 0.07
    acc = torch.zeros(shard, device="cuda")
    for step in range(16):
        rs.step = step
        outs = [torch.empty(shard, device="cuda") for _ in range(world)]
        rs.reduce(outs, [x.clone(), x.clone()], 1.0)  # SUM
        acc += outs[0]
    rs.check_status()
    assert abs((acc / 16)[1::64].mean().item() - 2 * 0.0123) < 4e-4


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_all_gather_dequant(world, bits, dtype):
    from nangila.parallel.fsdp_collectives import NangilaAllGather

    ag = NangilaAllGather(_arena(world), bits=bits)
    shard = 2048 * 5 + 64
    torch.manual_seed(bits + world)
    for rep in range(2):
        inputs = [(torch.randn(shard, device="cuda") * 0.02).to(dtype) for _ in range(world)]
        outputs = [torch.zeros(shard * world, device="cuda", dtype=dtype) for _ in range(world)]
        ag.gather(outputs, inputs)
        ag.check_status()
        full = torch.cat(inputs).float()
        for r in range(1, world):
            assert torch.equal(outputs[r], outputs[0])  # identical parameters on every rank
        got = outputs[0].float()
        qmax = 127.0 if bits == 8 else 7.0
        step = _bf16_ceil(full.view(-1, 64).abs().amax(1) * (0.0078740157 if bits == 8 else 0.14285715))
        err = (got - full).abs().view(-1, 64)
        assert bool((err <= step[:, None] * 0.51 + 4e-3 * full.abs().view(-1, 64) + 1e-7).all())
        rel = ((got - full).norm() / full.norm()).item()
        assert rel < (0.01 if bits == 8 else 0.12)


def test_error_memory_is_per_unit_not_per_size():
    """Two FSDP units of the same flat size: each keeps its own error memory. With a shared one the second
    unit's result would carry the first unit's quantization error."""
    from nangila.parallel.fsdp_collectives import NangilaReduceScatter

    world, shard = 2, 4096 * 4
    n = shard * world
    torch.manual_seed(1)
    a = [(torch.randn(n, device="cuda") * 0.01).to(torch.bfloat16) for _ in range(world)]
    b = [(torch.randn(n, device="cuda") * 0.5).to(torch.bfloat16) for _ in range(world)]   # very different scale

    def run(units):
        rs = NangilaReduceScatter(_arena(world), error_feedback=True)
        outs = {}
        for step in range(3):
            for name, data in units:
                o = [torch.empty(shard, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
                rs.reduce(o, [d.clone() for d in data], 1.0 / world, unit=name)
                outs[(step, name)] = o[0].clone()
        rs.check_status()
        return outs, rs

    both, rs = run([("a", a), ("b", b)])
    alone, _ = run([("a", a)])
    assert rs.units_seen == 2
    for step in range(3):
        assert torch.equal(both[(step, "a")], alone[(step, "a")])  # unit b never touched unit a's state
    # and the error memory does its job: the running mean of the outputs approaches the exact mean
    exact = torch.stack([x[:shard].float() for x in a]).mean(0)
    err1 = (both[(0, "a")].float() - exact).norm()
    err3 = (torch.stack([both[(s, "a")].float() for s in range(3)]).mean(0) - exact).norm()
    assert err3 < 0.6 * err1


@pytest.mark.parametrize("world", [2, 8])
def test_predictor_mode_reduce_scatter(world):
    """predictor=True: the reference's prediction-residual FSDP data flow. After the history is seeded, a
    gradient that the momentum predictor tracks is reproduced far more accurately than plain INT4 would."""
    from nangila.parallel.fsdp_collectives import NangilaReduceScatter

    shard = 4096 * 3
    n = shard * world
    torch.manual_seed(2)
    base = torch.randn(n, device="cuda") * 0.02
    drift = torch.randn(n, device="cuda") * 0.002

    def run(predictor):
        rs = NangilaReduceScatter(_arena(world), predictor=predictor, stochastic=False)
        rel = []
        for step in range(6):
            ins = [(base + drift * step + torch.randn(n, device="cuda") * 1e-4).to(torch.bfloat16) for _ in range(world)]
            exact = torch.stack([i.float() for i in ins]).mean(0)
            outs = [torch.empty(shard, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
            rs.reduce(outs, ins, 1.0 / world, unit="u")
            rs.check_status()
            for r in range(world):
                rel.append(((outs[r].float() - exact[r * shard:(r + 1) * shard]).norm() / exact[r * shard:(r + 1) * shard].norm()).item())
        return rel[-world:]

    with_pred, without = run(True), run(False)
    assert max(with_pred) < 0.02, with_pred          # residual is ~10 % of the gradient: INT4 error shrinks with it
    assert min(without) > 2 * max(with_pred), (with_pred, without)
