"""GPU tests of the PowerSGD path: the tcgen05 GEMMs against torch.matmul, and the whole step
(loopback world) against a PyTorch FP32 restatement with the same bf16 roundings."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n", [(128, 64), (256, 256), (768, 3072), (3072, 768), (1000, 520), (64, 2304), (8192, 1024)])
@pytest.mark.parametrize("transposed", [False, True])
def test_tcgen05_gemm_matches_matmul(m, n, transposed):
    from nangila import _cuda as C

    torch.manual_seed(m + n)
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    M = (torch.randn(m, n, device="cuda") * 0.1).bfloat16()
    k = m if transposed else n
    rows = n if transposed else m
    Bt = (torch.randn(16, k, device="cuda") * 0.1).bfloat16()
    out = torch.full((rows, 16), 7.0, device="cuda")
    C.psgd_gemm(M, Bt, transposed, out, status, 1.0)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    ref = (M.float().t() if transposed else M.float()) @ Bt.float().t()
    assert torch.allclose(out, ref, atol=2e-5 * max(1.0, ref.abs().max().item()), rtol=1e-4)


def gram_schmidt(p):
    p = p.clone()
    for c in range(p.shape[1]):
        for j in range(c):
            p[:, c] -= (p[:, c] @ p[:, j]) * p[:, j]
        nrm = p[:, c].norm()
        if nrm > 1e-10:
            p[:, c] /= nrm
    return p


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("shape,rank", [((256, 512), 4), ((768, 64, 3, 3), 2), ((1024, 1000), 1)])
def test_full_step_matches_reference(world, shape, rank):
    from nangila.parallel.powersgd_engine import PowerSGDEngine, initial_qt
    from nangila.parallel.symm import LoopbackArena

    dev = torch.device("cuda", 0)
    eng = PowerSGDEngine(LoopbackArena(world, dev), dev, rank=rank)
    m = shape[0]
    n = 1
    for d in shape[1:]:
        n *= d
    torch.manual_seed(world + m)
    # low-rank signal + noise, different per rank
    base = torch.randn(m, rank, device=dev) @ torch.randn(rank, n, device=dev) * 0.05
    for step in range(3):
        grads = [(base + torch.randn(m, n, device=dev) * 0.01).reshape(shape).contiguous() for _ in range(world)]
        # every step is checked on its own: the reference starts from the engine's current state
        # (error memory and warm start), so rounding differences cannot accumulate across steps
        if step == 0:
            ef = [torch.zeros(m, n, device=dev) for _ in range(world)]
            qt = initial_qt(n, rank, dev)[:rank].float()
        else:
            st = eng.states[(0, 0)]
            ef = [e.float().clone() for e in st.ef]
            qt = st.qt[0][:rank].float().clone()
        mef = [(g.reshape(m, n) + e).bfloat16().float() for g, e in zip(grads, ef)]
        p = gram_schmidt(torch.stack([x @ qt.t() for x in mef]).mean(0))
        q = torch.stack([x.t() @ p.bfloat16().float() for x in mef]).mean(0)  # [n, r]
        want = p @ q.t()
        eng.compress_matrix((0, 0), grads)
        eng.check_status()
        for r_ in range(world):
            got = grads[r_].reshape(m, n)
            rel = ((got - want).norm() / want.norm()).item()
            assert rel < 2e-2, (step, r_, rel)
        for r_ in range(1, world):
            assert torch.equal(grads[r_], grads[0])  # identical bits on every rank
        st = eng.states[(0, 0)]
        for r_ in range(world):  # error memory = what the approximation left out
            assert torch.allclose(st.ef[r_].float(), (mef[r_] - want).bfloat16().float(), atol=2e-3)
        if step == 2:  # after a few power iterations the rank-r signal is captured
            true_mean = torch.stack(mef).mean(0)
            assert ((grads[0].reshape(m, n) - true_mean).norm() / true_mean.norm()).item() < 0.6
    st = eng.states[(0, 0)]
    # the warm start kept for the next step has orthonormal rows
    qq = st.qt[0][:rank].float()
    assert torch.allclose(qq @ qq.t(), torch.eye(rank, device=dev), atol=2e-2)


def test_rank1_matrix_is_recovered_exactly():
    # nangila-core/src/power_sgd.rs:244-277: a rank-1 matrix is reproduced by a rank-1 approximation
    from nangila.parallel.powersgd_engine import PowerSGDEngine
    from nangila.parallel.symm import LoopbackArena

    dev = torch.device("cuda", 0)
    eng = PowerSGDEngine(LoopbackArena(1, dev), dev, rank=1)
    u = torch.linspace(0.5, 1.5, 128, device=dev)
    v = torch.linspace(-1, 1, 256, device=dev)
    g = [(u[:, None] * v[None, :]).contiguous()]
    want = g[0].clone()
    eng.compress_matrix((0, 0), g)
    eng.check_status()
    assert ((g[0] - want).norm() / want.norm()).item() < 1e-2


class _FakeBucket:
    def __init__(self, grads):
        self._grads = grads

    def gradients(self):
        return self._grads


@pytest.mark.parametrize("world", [1])
def test_bucket_graph_replay_matches_separate_launches(world, monkeypatch):
    """All matrices of a bucket recorded into one CUDA graph and replayed: same results, step after step,
    as launching the kernels one by one; one launch per bucket after the recording."""
    from nangila.parallel.powersgd_engine import PowerSGDEngine
    from nangila.parallel.predres_engine import PredResEngine
    from nangila.parallel.symm import LoopbackArena

    dev = torch.device("cuda", 0)
    shapes = [(256, 128), (64, 3, 3, 64), (128, 512), (40,), (512, 64)]
    results = {}
    for graphs in ("1", "0"):
        monkeypatch.setenv("NANGILA_PSGD_GRAPH", graphs)
        arena = LoopbackArena(world, dev)
        exact = PredResEngine(arena, dev, use_side_stream=False)
        eng = PowerSGDEngine(arena, dev, rank=4, exact_engine=exact)
        torch.manual_seed(0)
        flat = torch.zeros(sum(int(torch.tensor(s).prod()) for s in shapes), device=dev, dtype=torch.bfloat16)
        views, off = [], 0
        for s in shapes:
            k = int(torch.tensor(s).prod())
            views.append(flat[off:off + k].view(*s))
            off += k
        outs = []
        for step in range(4):
            flat.copy_((torch.randn(flat.numel(), device=dev) * 0.02).to(torch.bfloat16))  # same addresses every step
            eng.reduce(7, _FakeBucket(views), flat)
            eng.check_status()
            outs.append(flat.clone())
        results[graphs] = (outs, eng.launches, eng.graph_replays)
    for a, b in zip(results["1"][0], results["0"][0]):
        # split-K partial sums are added with atomics, so the last bits may differ between two runs
        assert torch.allclose(a.float(), b.float(), atol=2e-4, rtol=2e-2)
    assert results["1"][2] == 4 and results["0"][2] == 0
    assert results["1"][1] < results["0"][1] / 4   # one launch per bucket instead of six per matrix
