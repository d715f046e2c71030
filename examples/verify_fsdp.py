#!/usr/bin/env python
"""Verification drivers for the FSDP path, one sub-command per check (2 or more GPUs):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/verify_fsdp.py grads
    ...                                                                       examples/verify_fsdp.py overfit
    ...                                                                       examples/verify_fsdp.py sharding

* ``grads``    one backward pass: norm and relative error of the sharded gradients with the compressed
               reduce-scatter against FSDP2's own (reference: examples/verify_grads.py).
* ``overfit``  one fixed batch, 100 steps at lr 1e-2: the loss must collapse with and without compression
               (reference: examples/verify_overfit.py).
* ``sharding`` two large square layers: peak memory of stock FSDP2, of the compressed collectives, and of the
               predictor mode with its full-size history (reference: examples/verify_sharding.py).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn as nn  # noqa: E402
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard  # noqa: E402

from nangila.fsdp import apply_nangila_fsdp  # noqa: E402
from nangila.models.llama import Llama, LlamaConfig  # noqa: E402


def build_llama(dev, compress, **kw):
    torch.manual_seed(0)
    model = Llama(LlamaConfig.tiny()).to(dev)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    for blk in model.blocks:
        fully_shard(blk, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    hooks = apply_nangila_fsdp(model, **kw) if compress else (None, None)
    return model, hooks


def check_grads(dev, rank, world):
    tok = torch.randint(0, 64, (8, 33), generator=torch.Generator().manual_seed(11 + rank)).to(dev)
    out = {}
    for name, compress, kw in (("fsdp2", False, {}), ("nangila", True, dict(quantize_parameters=False))):
        model, _ = build_llama(dev, compress, **kw)
        model(tok[:, :-1], tok[:, 1:]).backward()
        out[name] = torch.cat([p.grad.to_local().float().reshape(-1) for p in model.parameters()])
    sq = torch.stack([out["fsdp2"].pow(2).sum(), out["nangila"].pow(2).sum(), (out["nangila"] - out["fsdp2"]).pow(2).sum()])
    dist.all_reduce(sq)
    n0, n1, d = sq.sqrt().tolist()
    if rank == 0:
        print(f"gradient norm: FSDP2 {n0:.6f}, compressed reduce-scatter {n1:.6f} ({abs(n1 / n0 - 1) * 100:.2f} % apart); "
              f"relative error of the gradient {d / n0:.4f}")
    return d / n0 < 0.15


def check_overfit(dev, rank, world, steps=100):
    tok = torch.randint(0, 64, (8, 33), generator=torch.Generator().manual_seed(11 + rank)).to(dev)
    ok = True
    for name, compress, kw in (("fsdp2", False, {}), ("nangila", True, dict(parameter_bits=8))):
        model, _ = build_llama(dev, compress, **kw)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
        first = last = None
        for step in range(steps):
            loss = model(tok[:, :-1], tok[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            last = loss.detach()
            first = last if first is None else first
        both = torch.stack([first, last]).float()
        dist.all_reduce(both)
        both /= world
        if rank == 0:
            print(f"{name}: loss {both[0].item():.3f} -> {both[1].item():.4f} in {steps} steps")
        ok = ok and both[1].item() < 0.1 * both[0].item()
    return ok


def check_sharding(dev, rank, world, width=8192):
    results = {}
    for name, compress, kw in (("fsdp2", False, {}), ("nangila", True, {}), ("nangila predictor", True, dict(predictor=True))):
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats(dev)
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(width, width, bias=False), nn.GELU(), nn.Linear(width, width, bias=False)).to(dev)
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
        for layer in (model[0], model[2]):
            fully_shard(layer, mp_policy=mp)
        fully_shard(model, mp_policy=mp)
        if compress:
            apply_nangila_fsdp(model, **kw)
        opt = torch.optim.SGD(model.parameters(), lr=1e-3)
        x = torch.randn(16, width, device=dev)
        for _ in range(4):
            model(x).pow(2).mean().backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
        torch.cuda.synchronize(dev)
        results[name] = torch.cuda.max_memory_allocated(dev) / 2**20
        del model, opt
    if rank == 0:
        full = 2 * width * width * 4 / 2**20
        print(f"two {width} x {width} layers = {full:.0f} MiB of FP32 parameters unsharded; peak per GPU: " +
              ", ".join(f"{k} {v:.0f} MiB" for k, v in results.items()))
    return results["nangila"] < results["fsdp2"] * 1.3 + 256


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("check", choices=["grads", "overfit", "sharding", "all"])
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    checks = {"grads": check_grads, "overfit": check_overfit, "sharding": check_sharding}
    ok = True
    for name, fn in checks.items():
        if args.check in (name, "all"):
            passed = fn(dev, rank, world)
            ok = ok and passed
            if rank == 0:
                print(f"[{name}] {'PASS' if passed else 'FAIL'}")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
