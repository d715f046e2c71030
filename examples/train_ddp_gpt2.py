#!/usr/bin/env python
"""DDP training of GPT-2 with a Nangila compression hook.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_ddp_gpt2.py \
        --steps 200 --compressor predres --checkpoint /tmp/run.pt

One process per GPU. The hook replaces DDP's bucket all-reduce with one fused kernel per bucket;
``hook.step()`` must follow every optimizer step. With ``--checkpoint`` the model, the optimizer and the
hook are saved every ``--save-every`` steps and the run resumes from the file if it exists.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
from torch.nn.parallel import DistributedDataParallel as DDP  # noqa: E402

from nangila import CompressorType  # noqa: E402
from nangila.ddp import register_nangila_hook  # noqa: E402
from nangila.models.gpt2 import GPT2, GPT2Config  # noqa: E402
from nangila.utils import init_distributed, seed_everything  # noqa: E402

COMPRESSORS = {"predres": CompressorType.PredictionResidual, "dgc": CompressorType.DGC, "powersgd": CompressorType.PowerSGD}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup-steps", type=int, default=20)
    ap.add_argument("--compressor", default="predres", choices=sorted(COMPRESSORS))
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--save-every", type=int, default=50)
    ap.add_argument("--liveness-timeout", type=float, default=0.0,
                    help="seconds of silence after which a peer counts as gone (0: no heartbeats); the run then stops with its name")
    args = ap.parse_args()
    rank, world, dev = init_distributed()
    seed_everything(0)
    cfg = GPT2Config.tiny() if args.tiny else GPT2Config.small()
    model = GPT2(cfg).to(dev)
    if dev.type == "cuda":
        model = model.to(torch.bfloat16)
    ddp = DDP(model, device_ids=[dev.index] if dev.type == "cuda" else None, bucket_cap_mb=25)
    hook = register_nangila_hook(ddp, threshold=0.95, warmup_steps=args.warmup_steps,
                                 compressor_type=int(COMPRESSORS[args.compressor]), dgc_sparsity=0.999, power_sgd_rank=4,
                                 liveness_timeout=args.liveness_timeout or None)
    hook.enable_safe_mode()  # falls back to exact averaging if the validation loss diverges
    opt = torch.optim.AdamW(ddp.parameters(), lr=3e-4, weight_decay=0.01)
    start = 0
    path = f"{args.checkpoint}.rank{rank}" if args.checkpoint else ""
    if path and os.path.exists(path):
        ck = torch.load(path, map_location=dev, weights_only=False)
        model.load_state_dict(ck["model"])
        opt.load_state_dict(ck["opt"])
        hook.load_state_dict(ck["hook"])
        start = ck["step"]
    gen = torch.Generator().manual_seed(1234 + rank)
    seq = min(cfg.n_ctx, 1024)
    for step in range(start, args.steps):
        tok = torch.randint(0, cfg.vocab_size, (args.micro_batch, seq + 1), generator=gen).to(dev)
        try:
            loss = ddp(tok[:, :-1], tok[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            hook.step()   # with heartbeats on, raises RankFailure when a peer has left
        except RuntimeError:
            hook.check_peers(wait=2.0 * args.liveness_timeout)   # a failed collective: say which rank it was, if one is gone
            raise
        if step % 10 == 0:
            hook.report_validation_loss(float(loss))
            if rank == 0:
                st = hook.get_stats()
                print(f"step {step:5d}  loss {float(loss):.4f}  compressing {st['compression_enabled']}  "
                      f"ratio {st.get('overall_compression_ratio', 1.0):.2f}")
        if path and (step + 1) % args.save_every == 0:
            torch.save({"model": model.state_dict(), "opt": opt.state_dict(), "hook": hook.state_dict(), "step": step + 1}, path)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
