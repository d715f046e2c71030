"""GPU tests of the auxiliary kernels: state hash, parallel CRC32, percentile / absmax, Sculptor
statistics, and the single-scale compatibility kernels."""
import zlib

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nbytes", [1, 3, 511, 512, 513, 4096, 100_003, 5_000_000])
def test_crc32_matches_zlib(nbytes):
    from nangila.ops import crc32

    torch.manual_seed(nbytes)
    t = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda")
    assert crc32(t) == zlib.crc32(t.cpu().numpy().tobytes())


def test_crc32_of_float_tensor_and_core_agree():
    from nangila import _C
    from nangila.ops import crc32

    x = torch.randn(12345, device="cuda")
    raw = x.cpu().numpy().tobytes()
    assert crc32(x) == zlib.crc32(raw) == _C.crc32(raw)


def test_state_hash_properties():
    from nangila.ops import state_hash

    a = torch.randn(100_001, device="cuda").bfloat16()
    b = torch.randn(777, device="cuda")
    h = state_hash([a, b])
    assert h == state_hash([a.clone(), b.clone()])
    assert h != state_hash([b, a])
    a2 = a.clone()
    a2[12345] += 1
    assert h != state_hash([a2, b])
    assert state_hash([a], seed=1) != state_hash([a], seed=2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1000, 65_537, 3_000_000])
def test_percentile_and_absmax_are_exact(dtype, n):
    from nangila.ops import absmax_percentile

    torch.manual_seed(n)
    x = (torch.randn(n, device="cuda") * 0.03).to(dtype)
    x[n // 2] = float("nan")
    x[n // 3] = float("inf")
    mx, p99, gamma, hist = absmax_percentile(x, 0.99)
    a = x.float().abs()
    a[~torch.isfinite(a)] = 0
    srt = a.sort().values
    idx = min(int(np.float32(n) * np.float32(0.99)), n - 1)
    assert mx == srt[-1].item()
    assert p99 == srt[idx].item()
    assert gamma == pytest.approx(max(p99 / 7.0, 1e-8), rel=1e-6)
    assert int(hist.sum().item()) == n and int(hist[255].item()) >= 1


def test_quantizer_gamma_matches_host_core():
    from nangila import _C
    from nangila.ops import quantizer_gamma

    x = torch.randn(50_000, device="cuda") * 0.01
    host = _C.Quantizer(4, True, False).compute_gamma(x.cpu().numpy())
    assert quantizer_gamma(x) == pytest.approx(host, rel=1e-6)


def test_device_sculptor_matches_host_sculptor():
    import nangila
    from nangila import _C
    from nangila.ops import DeviceSculptor

    dev, host = DeviceSculptor(0.9), nangila.Sculptor(0.9)
    torch.manual_seed(0)
    n = 4096
    for step in range(40):
        base = torch.randn(n, device="cuda") * (1 + 0.1 * step)
        layers = {0: base, 1: 0.5 * base + 0.01 * torch.randn(n, device="cuda") + 0.2,
                  2: torch.randn(n, device="cuda"), 3: torch.randn(2 * n, device="cuda")}
        for lid, g in layers.items():
            dev.record(lid, g)
            host.record(lid, g.cpu().numpy())
        dev.end_step()
        host.end_step()
    for a, b in [(0, 1), (0, 2), (1, 2)]:
        assert dev.correlation(a, b) == pytest.approx(host.correlation(a, b), abs=2e-3)
    assert dev.correlation(0, 3) is None
    ad, bd = dev.coupling(0, 1)
    ah, bh = host.coupling(0, 1)
    assert ad == pytest.approx(ah, abs=5e-3) and bd == pytest.approx(bh, abs=5e-3)
    assert ad == pytest.approx(0.5, abs=0.02) and bd == pytest.approx(0.2, abs=0.02)
    md = _C.TopologyMask.from_bytes(dev.generate_mask())
    mh = _C.TopologyMask.from_bytes(host.generate_mask())
    assert md.num_layers() == mh.num_layers() == 4
    assert md.num_passengers() == mh.num_passengers() == 1
    assert md.passengers()[0][:2] == mh.passengers()[0][:2]
    assert dev.num_samples() == 40


def test_compat_gamma_kernels_roundtrip():
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        from nangila import experimental as ex

    n = 100_003
    torch.manual_seed(1)
    prev = torch.randn(n, device="cuda") * 0.1
    cur = prev + torch.randn(n, device="cuda") * 0.01
    pred = cur + 0.9 * (cur - prev)
    grad = pred + torch.randn(n, device="cuda") * 0.004
    gamma = 0.004 * 2.6 / 7
    packed = torch.zeros((n + 1) // 2, dtype=torch.uint8, device="cuda")
    out = torch.empty(n, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ex.cuda_predict_and_quantize(grad.data_ptr(), cur.data_ptr(), prev.data_ptr(), 0.9, gamma, packed.data_ptr(), n,
                                 stream_ptr=stream, sync_mode=1, step=3, layer_id=5)
    ex.cuda_dequantize_and_reconstruct(packed.data_ptr(), cur.data_ptr(), prev.data_ptr(), 0.9, gamma, out.data_ptr(), n,
                                       stream_ptr=stream, sync_mode=1)
    err = (out - grad).abs()
    clipped = (grad - pred).abs() > 7 * gamma
    assert bool((err[~clipped] <= gamma * 1.001).all())
    assert abs((out - grad)[~clipped].mean().item()) < gamma * 0.02  # stochastic rounding is unbiased
    with pytest.raises(ValueError, match="Invalid sync_mode"):
        ex.cuda_predict_and_quantize(0, 0, 0, 0.9, 0.1, 0, 8, sync_mode=5)
    with pytest.raises(RuntimeError):
        ex.cuda_predict_and_quantize(0, 0, 0, 0.9, 0.1, 0, 8, sync_mode=0)  # null pointers are rejected


@pytest.mark.parametrize("rows,cols,classes", [(64, 50304, 50257), (33, 1024, 1000), (7, 8, 8), (5, 136, 129)])
def test_fused_cross_entropy_matches_fp32_reference(rows, cols, classes):
    """Loss and gradient of the fused kernel pair against F.cross_entropy on fp32 copies of the same bf16 logits."""
    import torch.nn.functional as F

    from nangila.ops.fused_ce import fused_cross_entropy

    torch.manual_seed(rows)
    logits = (torch.randn(rows, cols, device="cuda") * 3.0).to(torch.bfloat16).requires_grad_(True)
    targets = torch.randint(0, classes, (rows,), device="cuda")
    loss = fused_cross_entropy(logits, targets, classes)
    (loss * 2.5).backward()
    ref_in = logits.detach().float().requires_grad_(True)
    ref = F.cross_entropy(ref_in[:, :classes], targets)
    (ref * 2.5).backward()
    assert abs(loss.item() - ref.item()) < 2e-5 * max(1.0, abs(ref.item()))
    g, gr = logits.grad.float(), ref_in.grad
    assert torch.all(g[:, classes:] == 0)
    assert (g - gr).abs().max().item() <= 2 ** -8 * gr.abs().max().item() + 1e-7  # bf16 rounding of the gradient
    # rows sum to zero up to bf16 rounding
    assert g.sum(dim=1).abs().max().item() < 0.02 * 2.5 / rows + 1e-6


@pytest.mark.parametrize("rows,cols", [(8192, 768), (1000, 3072), (37, 2304), (5, 4), (300, 132)])
def test_colsum_matches_fp32_reference(rows, cols):
    from nangila.ops.fused_grads import colsum

    torch.manual_seed(rows + cols)
    a = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    b = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    s, none = colsum(a)
    assert none is None
    ref_s = a.float().sum(0)
    assert (s - ref_s).abs().max().item() <= 1e-4 * (a.float().abs().sum(0).max().item() + 1.0)
    s2, p = colsum(a, b)
    assert torch.equal(s, s2)  # fixed summation order: same bits
    ref_p = (a.float() * b.float()).sum(0)
    assert (p - ref_p).abs().max().item() <= 1e-4 * ((a.float() * b.float()).abs().sum(0).max().item() + 1.0)


def test_gpt2_gradients_with_and_without_the_fused_gradient_kernels(monkeypatch):
    """Same weights, same batch: parameter gradients with the column-sum kernel against PyTorch's own backward."""
    from nangila.models.gpt2 import GPT2, GPT2Config

    torch.manual_seed(0)
    model = GPT2(GPT2Config.tiny()).cuda().to(torch.bfloat16)
    tok = torch.randint(0, 1000, (4, 65), device="cuda")
    grads = {}
    for flag in ("0", "1"):
        monkeypatch.setenv("NANGILA_FUSED_GRADS", flag)
        model.zero_grad(set_to_none=True)
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        grads[flag] = {n: p.grad.float().clone() for n, p in model.named_parameters()}
        grads[flag]["loss"] = loss.detach().float()
    from nangila.ops import fused_grads

    assert fused_grads.launch_count > 0
    assert torch.equal(grads["0"]["loss"], grads["1"]["loss"])  # forward is the same computation
    for n in grads["0"]:
        a, b = grads["0"][n], grads["1"][n]
        tol = 0.02 * a.abs().max().item() + 1e-6  # bf16 rounding of reductions done in a different order
        assert (a - b).abs().max().item() <= tol, n
