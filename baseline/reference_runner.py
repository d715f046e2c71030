#!/usr/bin/env python
"""Times the UNMODIFIED reference implementation on the headline workload.

Started by ``bench.py --impl reference`` as a child process whose import path holds ``baseline/_ref``
(where the reference is installed) and not this repository, so ``import nangila`` is the reference. The
model is a plain-PyTorch GPT-2 small written here with stock ``torch.nn`` modules only: none of the
framework's models, kernels or engines is on this path. The hook is registered exactly as the
reference's README shows: ``register_nangila_hook(ddp_model, threshold=0.95, warmup_steps=100)`` and
``hook.step()`` after every optimizer step. Prints the same JSON line as ``bench.py``.
"""
import argparse
import json
import os
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.parallel import DistributedDataParallel as DDP


class Block(nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc, self.out = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
        self.h = h

    def forward(self, x):
        b, t, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, t, 3, self.h, d // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, t, d)
        x = x + self.proj(a)
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class PlainGPT2(nn.Module):
    def __init__(self, vocab=50257, ctx=1024, d=768, layers=12, heads=12):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(ctx, d)
        self.blocks = nn.ModuleList(Block(d, heads) for _ in range(layers))
        self.lnf = nn.LayerNorm(d)

    def forward(self, idx, targets):
        t = idx.shape[1]
        x = self.wte(idx) + self.wpe(torch.arange(t, device=idx.device))
        for blk in self.blocks:
            x = blk(x)
        logits = self.lnf(x) @ self.wte.weight.t()
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=1024)
    args = ap.parse_args()
    from nangila.ddp import register_nangila_hook  # the reference's public API

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    torch.manual_seed(0)
    model = PlainGPT2().to(dev).to(torch.bfloat16)
    ddp = DDP(model, device_ids=[local], bucket_cap_mb=25, gradient_as_bucket_view=True)
    hook = register_nangila_hook(ddp, threshold=0.95, warmup_steps=100)
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-4, weight_decay=0.01, fused=True)
    mb, seq = args.micro_batch, args.seq_len
    gen = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randint(0, 50257, (mb, seq + 1), generator=gen).pin_memory() for _ in range(64)]

    def step(i):
        tok = host[i % 64].to(dev, non_blocking=True)
        loss = ddp(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        hook.step()
        return float(loss.item())

    warmup = max(args.warmup, 3)
    for i in range(warmup):
        step(i)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        last = step(i)
    e1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3
    dist.barrier()
    ms = torch.tensor([max(e0.elapsed_time(e1), wall)], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    tokens = mb * seq * world * args.steps
    if rank == 0:
        value = tokens / (ms.item() / 1e3)
        print(json.dumps({
            "impl": "reference", "metric": "GPT-2 small DDP training throughput", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms.item() / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": "gpt2-small 12L d768 h12 mlp3072 vocab50257 ctx1024 (plain torch.nn)", "global_batch": mb * world,
                       "seq_len": seq, "parallelism": f"dp{world}", "bucket_mb": 25,
                       "hook": "reference register_nangila_hook(threshold=0.95, warmup_steps=100)"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": int(host[0].numel() * 8), "d2h_bytes_per_step": 4},
            "final_loss": last}))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
