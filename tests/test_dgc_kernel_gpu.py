"""GPU tests of the fused DGC kernel (single-GPU loopback world) against the host compressor's
semantics restated in PyTorch: accumulate, exact top-k by |v|, zero what was sent, average."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(world, **kw):
    from nangila.parallel.dgc_engine import DGCEngine
    from nangila.parallel.symm import LoopbackArena

    dev = torch.device("cuda", 0)
    return DGCEngine(LoopbackArena(world, dev), dev, **kw)


def ref_step(g, u, v, k, m):
    """One rank's DGC step in FP32: returns the dense tensor of what it sends."""
    u.mul_(m).add_(g)
    v.add_(u)
    idx = v.abs().topk(k).indices
    sent = torch.zeros_like(v)
    sent[idx] = v[idx]
    v[idx] = 0
    u[idx] = 0
    return sent


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("n,sparsity", [(10_000, 0.99), (1_000_003, 0.999), (300_000, 0.9)])
@pytest.mark.parametrize("momentum", [0.0, 0.9])
def test_matches_reference_over_steps(world, n, sparsity, momentum):
    eng = _engine(world, sparsity=sparsity, momentum=momentum)
    torch.manual_seed(world * 1000 + n)
    us = [torch.zeros(n, device="cuda") for _ in range(world)]
    vs = [torch.zeros(n, device="cuda") for _ in range(world)]
    for step in range(3):
        grads = [torch.randn(n, device="cuda") for _ in range(world)]
        k = eng.bucket_state(0, grads).k
        want = sum(ref_step(g.clone(), us[r], vs[r], k, momentum) for r, g in enumerate(grads)) / world
        eng.reduce(0, grads)
        eng.check_status()
        st = eng.buckets[0]
        for r in range(world):
            assert int(st.out_count[r][0]) == k
            assert torch.allclose(grads[r], want, atol=1e-6, rtol=1e-5), (step, r, (grads[r] - want).abs().max())
            assert torch.allclose(st.v[r], vs[r], atol=1e-6, rtol=1e-5)
            assert torch.allclose(st.u[r], us[r], atol=1e-6, rtol=1e-5)
        for r in range(1, world):
            assert torch.equal(grads[r], grads[0])


def test_accumulation_vector_of_reference_unit_test():
    # nangila-core/src/dgc.rs:229-263: sparsity 0.99 on 5 elements keeps one entry per step
    eng = _engine(1, sparsity=0.99, momentum=0.0)
    g = [torch.tensor([1.0, 0, 0, 0, 0], device="cuda")]
    eng.reduce(0, g)
    assert g[0][0].item() == 1.0
    g = [torch.tensor([0.1, 2.0, 0, 0, 0], device="cuda")]
    eng.reduce(0, g)
    assert g[0][1].item() == 2.0 and g[0][0].item() == 0.0
    g = [torch.tensor([0.3, 0, 0, 0, 0], device="cuda")]
    eng.reduce(0, g)
    eng.check_status()
    assert abs(g[0][0].item() - 0.4) < 1e-6


def test_bf16_bucket_and_ties():
    eng = _engine(2, sparsity=0.9, momentum=0.0)
    n = 4096
    grads = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    grads[0][:500] = 1.0   # 500 equal entries, k = 410: all ties are selected, cut at the capacity
    grads[1][1000:1100] = -2.0
    eng.reduce(0, grads)
    eng.check_status()
    st = eng.buckets[0]
    assert st.k == 410 and st.k <= int(st.out_count[0][0]) <= st.capacity
    assert int(st.out_count[1][0]) == 100  # fewer non-zero entries than k: zeros are never sent
    assert torch.equal(grads[0], grads[1])
    assert grads[0][1000:1100].float().eq(-1.0).all()
    sent = int(st.out_count[0][0])
    assert grads[0][:500].float().sum().item() == pytest.approx(0.5 * sent)
    assert st.v[0][:500].sum().item() == pytest.approx(500 - sent)  # what was cut stays accumulated
