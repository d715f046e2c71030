#!/usr/bin/env python
"""FSDP2 (``fully_shard``) training of a Llama-style decoder with Nangila's fused collectives: the
gradient reduce-scatter carries block-INT4 data and the parameter all-gather carries INT8 data that is
dequantized straight into the unsharded buffer.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_fsdp_llama.py
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard  # noqa: E402

from nangila.fsdp import apply_nangila_fsdp  # noqa: E402
from nangila.models.llama import Llama, LlamaConfig  # noqa: E402
from nangila.utils import init_distributed, seed_everything  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--parameter-bits", type=int, default=8, choices=[4, 8])
    ap.add_argument("--no-compress", action="store_true")
    args = ap.parse_args()
    rank, world, dev = init_distributed()
    seed_everything(0)
    cfg = LlamaConfig.tiny() if args.tiny else LlamaConfig.llama_1_3b()
    model = Llama(cfg).to(dev)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    for blk in model.blocks:
        fully_shard(blk, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    rs = ag = None
    if not args.no_compress:
        rs, ag = apply_nangila_fsdp(model, parameter_bits=args.parameter_bits)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    gen = torch.Generator().manual_seed(1 + rank)
    seq = min(cfg.max_seq, 2048)
    for step in range(args.steps):
        tok = torch.randint(0, cfg.vocab_size, (args.micro_batch, seq + 1), generator=gen).to(dev)
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        if rs is not None:
            rs.step += 1
        if rank == 0 and step % 10 == 0:
            extra = f"  fused launches rs {rs.launches} ag {ag.launches}, NCCL fallbacks {rs.fallbacks + ag.fallbacks}" if rs else ""
            print(f"step {step:4d}  loss {float(loss):.4f}{extra}")
    for c in (rs, ag):
        if c is not None:
            c.check_status()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
