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


def test_reduce_scatter_names_units_and_advances_steps():
    """Unit bookkeeping of the compressed reduce-scatter (pure host logic): identical sizes are different
    units, named explicitly or by call order, and the step advances without the caller's help when the
    first explicitly named unit comes round again."""
    from nangila.parallel.fsdp_collectives import NangilaReduceScatter

    rs = NangilaReduceScatter(error_feedback=True)
    n, dt = 4096, torch.bfloat16
    # explicit names: three identical blocks, three backward passes
    seen = []
    for step in range(3):
        for uid in (2, 1, 0):
            u = rs._unit(uid, n, dt)
            u.calls += 1
            seen.append((uid, u.index, u.calls, rs.step))
    assert rs.units_seen == 3
    assert [s[1] for s in seen[:3]] == [0, 1, 2]            # one state per unit although the sizes are equal
    assert [s[3] for s in seen] == [0, 0, 0, 1, 1, 1, 2, 2, 2]  # the step advanced by itself
    assert seen[-1][2] == 3
    # call order within a step, with end_step() as the boundary
    rs2 = NangilaReduceScatter(error_feedback=True)
    first = [rs2._unit(None, n, dt).index for _ in range(3)]
    rs2.end_step()
    second = [rs2._unit(None, n, dt).index for _ in range(3)]
    assert first == [0, 1, 2] and second == first and rs2.step == 1
    # the default rounding: stochastic without an error memory, to nearest with one
    assert NangilaReduceScatter().stochastic and not NangilaReduceScatter(error_feedback=True).stochastic
