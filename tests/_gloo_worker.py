"""Worker for the CPU/gloo DDP tests: fp32 MLP 784->256->ReLU->10, batch 32 per rank from N(0,1),
uniform labels, cross-entropy, SGD lr 0.01, seed 0."""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(rank, world, port, steps, use_hook, out_path, hook_kwargs, calib_steps=0, fixed_batch=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 10))
    ddp = DDP(model)
    hook = None
    sculptor = None
    if use_hook:
        import nangila
        from nangila.ddp import register_nangila_hook

        hook_kwargs = dict(hook_kwargs)
        faults = hook_kwargs.pop("_faults", [])
        ckpt_at = hook_kwargs.pop("_ckpt_at", None)
        resume = hook_kwargs.pop("_resume", None)
        hook = register_nangila_hook(ddp, **hook_kwargs)
        if faults:
            def packet_filter(step, layer_id, src, data, _faults=faults, _rank=rank):
                for f in _faults:
                    if f["step"] == step and f.get("layer", 0) == layer_id and f.get("src", 1) == src \
                            and f.get("on_rank", _rank) == _rank:
                        if f["kind"] == "corrupt":
                            b = bytearray(data)
                            b[len(b) // 2] ^= 0x5A
                            return bytes(b)
                        if f["kind"] == "truncate":
                            return data[: len(data) // 2]
                        if f["kind"] == "drop":
                            return b""
                return data
            hook._packet_filter = packet_filter
        if calib_steps:
            sculptor = nangila.Sculptor(hook_kwargs.get("threshold", 0.95))
    opt = torch.optim.SGD(ddp.parameters(), lr=0.01)
    g = torch.Generator().manual_seed(1000 + rank)
    losses = []
    mask_info = None
    xb = torch.randn(32, 784, generator=g)
    yb = torch.randint(0, 10, (32,), generator=g)
    start = 0
    if use_hook and resume:
        ck = torch.load(resume + f".rank{rank}", weights_only=False)
        model.load_state_dict(ck["model"])
        opt.load_state_dict(ck["opt"])
        hook.load_state_dict(ck["hook"])
        g.set_state(ck["gen"])
        start = ck["step"]
    for step in range(start, steps):
        if use_hook and ckpt_at is not None and step == ckpt_at:
            torch.save({"model": model.state_dict(), "opt": opt.state_dict(), "hook": hook.state_dict(),
                        "gen": g.get_state(), "step": step}, out_path + f".ckpt.rank{rank}")
        if fixed_batch:
            x, y = xb, yb
        else:
            x = torch.randn(32, 784, generator=g)
            y = torch.randint(0, 10, (32,), generator=g)
        opt.zero_grad()
        loss = nn.functional.cross_entropy(ddp(x), y)
        loss.backward()
        if sculptor is not None and step < calib_steps:
            for lid, p in enumerate(model.parameters()):
                sculptor.record(lid, p.grad.detach().reshape(-1).numpy())
            sculptor.end_step()
            if step == calib_steps - 1:
                mask = sculptor.generate_mask()
                h = nangila.NangilaHook(mask)
                st = h.get_stats()
                mask_info = (len(mask), st["num_drivers"], st["num_passengers"], sculptor.num_samples())
                if hook is not None:  # the calibrated topology goes to the hook that is already running
                    assert hook.set_mask(mask) == st["num_passengers"]
        opt.step()
        if hook is not None:
            hook.step()
        losses.append(float(loss.detach()))
    result = {"losses": losses, "mask_info": mask_info,
              "params": [p.detach().clone() for p in model.parameters()]}
    if hook is not None:
        result["stats"] = hook.get_stats()
        result["metrics"] = dict(hook.metrics().snapshot())
        result["prometheus"] = hook.metrics().to_prometheus()
    if rank == 0:
        torch.save(result, out_path)
    # every rank also saves its first parameter to check replicas stay identical
    torch.save(result["params"][0], out_path + f".rank{rank}")
    dist.barrier()
    dist.destroy_process_group()
