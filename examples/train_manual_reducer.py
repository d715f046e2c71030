#!/usr/bin/env python
"""Manual bucketed gradient reduction without a DDP comm hook.

For loops that cannot use ``register_comm_hook`` (gradient accumulation under ``no_sync()``, custom
reducers): parameters are grouped into fixed-size buckets once; after the last micro-batch the reducer
flattens each bucket, exchanges it, and scatters the averaged gradient back.

* CUDA tensors: one fused kernel launch per bucket (``nangila.parallel.PredResEngine``): predict-subtract,
  error feedback, block-INT4, the exchange over NVLink peer memory and the reconstruction.
* CPU tensors (gloo): the packet path of the host core: ``NangilaHook.compress`` -> all-gather ->
  ``decompress_gathered`` -> mean -> ``update``.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/train_manual_reducer.py
    python examples/train_manual_reducer.py --cpu --steps 30        # single process, gloo

The reference's counterpart is ``ManualNangilaReducer`` in examples/train_llm.py:25-147, which moved every
bucket to the host, pickled the packets through ``all_gather_object`` and decoded W copies per bucket.
"""
import argparse
import os
import socket
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

import nangila
from nangila.models.gpt2 import GPT2, GPT2Config


class ManualReducer:
    def __init__(self, model: torch.nn.Module, warmup_steps: int = 20, bucket_mb: float = 25.0):
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.warmup_steps = warmup_steps
        self.step_count = 0
        self.world = dist.get_world_size()
        self.buckets, cur, size = [], [], 0
        for p in self.params:
            nbytes = p.numel() * p.element_size()
            if cur and size + nbytes > bucket_mb * (1 << 20):
                self.buckets.append(cur)
                cur, size = [], 0
            cur.append(p)
            size += nbytes
        if cur:
            self.buckets.append(cur)
        self.cuda = self.params[0].is_cuda
        self.original_bytes = self.wire_bytes = 0
        if self.cuda:
            from nangila.parallel.predres_engine import PredResEngine
            from nangila.parallel.symm import SymmArena

            dev = self.params[0].device
            self.engine = PredResEngine(SymmArena(None, dev), dev, stochastic=False, error_feedback=True)
            self.flat = [torch.empty(sum(p.numel() for p in b), dtype=b[0].dtype, device=dev) for b in self.buckets]
        else:
            cfg = nangila.NangilaConfig(warmup_steps=warmup_steps, shadow_run_steps=0)
            self.hook = nangila.NangilaHook.all_drivers(len(self.buckets), cfg)

    def reduce(self) -> None:
        """Average the gradients of all ranks in place."""
        compressed = self.step_count >= self.warmup_steps
        for i, bucket in enumerate(self.buckets):
            if self.cuda:
                flat = self.flat[i]
                torch.cat([p.grad.reshape(-1) for p in bucket], out=flat)
                st = self.engine.reduce(i, [flat], compressed=compressed, step=self.step_count)
                torch.cuda.current_stream().wait_stream(self.engine.stream)
                off = 0
                for p in bucket:
                    p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                    off += p.numel()
                self.original_bytes += flat.numel() * flat.element_size()
                self.wire_bytes += self.engine.wire_bytes(st, compressed) if self.world > 1 else 0
            else:
                flat = torch.cat([p.grad.reshape(-1).float() for p in bucket]).numpy()
                packet = bytes(self.hook.compress(i, flat))
                gathered = [None] * self.world
                dist.all_gather_object(gathered, packet)
                mean = np.zeros_like(flat)
                for pk in gathered:
                    mean += self.hook.decompress_gathered(i, pk)
                mean /= self.world
                self.hook.update(i, mean)
                off = 0
                for p in bucket:
                    p.grad.copy_(torch.from_numpy(mean[off:off + p.numel()]).view_as(p.grad))
                    off += p.numel()
                self.original_bytes += flat.nbytes
                self.wire_bytes += len(packet)

    def step(self) -> None:
        self.step_count += 1
        if self.cuda:
            self.engine.end_step()
        else:
            self.hook.step()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--accum", type=int, default=2, help="micro-batches per optimizer step (all but the last under no_sync)")
    ap.add_argument("--warmup-steps", type=int, default=10)
    ap.add_argument("--cpu", action="store_true")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if "MASTER_PORT" not in os.environ:
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        os.environ["MASTER_PORT"] = str(s.getsockname()[1])
        s.close()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    use_cuda = torch.cuda.is_available() and not args.cpu
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    cfg = GPT2Config.tiny()
    model = GPT2(cfg).to(dev)
    ddp = DDP(model, device_ids=[dev.index] if use_cuda else None)
    reducer = ManualReducer(model, warmup_steps=args.warmup_steps, bucket_mb=1.0)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    gen = torch.Generator().manual_seed(7 + rank)
    data = torch.randint(0, 64, (64, 33), generator=torch.Generator().manual_seed(7))
    first = last = None
    for step in range(args.steps):
        # every micro-batch runs under no_sync(): DDP never reduces, the manual reducer does after the last one
        for micro in range(args.accum):
            rows = torch.randint(0, 64, (4,), generator=gen)
            tok = data[rows].to(dev)
            with ddp.no_sync():
                loss = ddp(tok[:, :-1], tok[:, 1:]) / args.accum
                loss.backward()
        reducer.reduce()
        opt.step()
        opt.zero_grad(set_to_none=False)
        reducer.step()
        last = float(loss.detach()) * args.accum
        first = last if first is None else first
        if rank == 0 and step % 10 == 0:
            print(f"step {step:3d} loss {last:.4f}")
    if rank == 0:
        ratio = reducer.original_bytes / max(reducer.wire_bytes, 1) if reducer.wire_bytes else float("nan")
        print(f"first loss {first:.4f} last loss {last:.4f} buckets {len(reducer.buckets)} bytes held / bytes sent {ratio:.2f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
