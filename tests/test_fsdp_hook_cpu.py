"""The FSDP1-style hook (reference signatures) on CPU / gloo: sharded and NO_SHARD call forms."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nangila.fsdp import NangilaFSDPState, nangila_fsdp_hook

    state = NangilaFSDPState(None)
    assert state.world_size == world and state.step_counter() == 0
    torch.manual_seed(rank)
    grad = torch.randn(64)
    every = [torch.zeros(64) for _ in range(world)]
    dist.all_gather(every, grad)
    mean = torch.stack(every).mean(0)
    shard = torch.zeros(64 // world)
    nangila_fsdp_hook(state, grad.clone(), shard)           # sharded strategies: fills `output`
    ok1 = torch.allclose(shard, mean[rank * shard.numel():(rank + 1) * shard.numel()], atol=1e-6)
    full = grad.clone()
    nangila_fsdp_hook(state, full)                           # NO_SHARD: all-reduce in place
    ok2 = torch.allclose(full, mean, atol=1e-6)
    state.step()
    ok3 = state.step_counter() == 1 and NangilaFSDPState.compute_gamma(torch.tensor([0.0, -14.0])) == 2.0
    torch.save((ok1, ok2, ok3), f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_fsdp_hook_forms_on_gloo(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "res")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    for r in range(2):
        assert torch.load(f"{out}.{r}") == (True, True, True)
