#!/usr/bin/env python
"""Training throughput of the three secondary benchmark configurations, each against its stock
PyTorch counterpart (``--impl baseline``):

  resnet50-powersgd   ResNet-50, DDP, bf16 autocast, batch 128 / GPU, 224x224, SGD momentum;
                      PowerSGD rank 4 on every convolution / linear weight         -> images/s
  bert-large-dgc      BERT-large MLM, DDP, bf16 autocast, batch 16 / GPU, sequence 512, 15 % masked,
                      AdamW; Deep Gradient Compression, sparsity 0.999, momentum correction -> tokens/s
  llama-1.3b-fsdp     Llama-style 1.3 B decoder, FSDP2 ``fully_shard`` per block, bf16 parameters,
                      micro-batch 4 x 2048; block-INT4 reduce-scatter + INT8 all-gather   -> tokens/s

    python bench/train_bench.py --config resnet50-powersgd --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench/train_bench.py --config llama-1.3b-fsdp --gpus 8

Synthetic inputs (random images / token ids), random-initialised weights. Rank 0 prints one JSON line:
device-timed value (CUDA events, max over ranks, inputs resident on the device) plus ``e2e`` with the
step's inputs copied from pinned host memory and the loss read back every step. ``--small`` switches
every configuration to a tiny model for functional checks.
"""
import argparse
import json
import os
import sys
import warnings

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from nangila.utils import init_distributed, seed_everything, timed_steps  # noqa: E402


def build_resnet(args, dev, world):
    from torch.nn.parallel import DistributedDataParallel as DDP

    from nangila.ddp import register_nangila_hook
    from nangila.models.resnet import resnet50, resnet_tiny

    model = (resnet_tiny() if args.small else resnet50()).to(dev).to(memory_format=torch.channels_last)
    ddp = DDP(model, device_ids=[dev.index], bucket_cap_mb=25, gradient_as_bucket_view=True)
    hook = None
    if args.impl == "ours":
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            hook = register_nangila_hook(ddp, warmup_steps=2, compressor_type=2, power_sgd_rank=4)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    b, hw, classes = (8, 64, 10) if args.small else (128, 224, 1000)
    gen = torch.Generator().manual_seed(1 + dist.get_rank())
    host = [(torch.randn(b, 3, hw, hw, generator=gen).pin_memory(), torch.randint(0, classes, (b,), generator=gen).pin_memory())
            for _ in range(4)]

    def put(batch):
        x, y = batch
        return (x.to(dev, non_blocking=True).to(memory_format=torch.channels_last), y.to(dev, non_blocking=True))

    def loss_fn(batch):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return ddp(batch[0], batch[1])

    info = {"model": "resnet-tiny" if args.small else "resnet50 v1.5, 224x224, 1000 classes", "unit": "images/s",
            "items_per_step": b * world, "global_batch": b * world, "parallelism": f"dp{world}",
            "compressor": "PowerSGD rank 4 (tcgen05 GEMMs)" if hook else "stock DDP all-reduce", "optimizer": "SGD(momentum 0.9)"}
    return ddp, opt, hook, host, put, loss_fn, info


def build_bert(args, dev, world):
    from torch.nn.parallel import DistributedDataParallel as DDP

    from nangila.ddp import register_nangila_hook
    from nangila.models.bert import BertConfig, BertMLM, mask_tokens

    cfg = BertConfig.tiny() if args.small else BertConfig.large()
    model = BertMLM(cfg).to(dev)
    # the fused DGC kernel makes several grid-wide passes per bucket and the selection is taken per bucket, so
    # fewer, larger buckets amortise that and select more globally (--bucket-mb, same in both arms)
    ddp = DDP(model, device_ids=[dev.index], bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
    hook = None
    if args.impl == "ours":
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            hook = register_nangila_hook(ddp, warmup_steps=2, compressor_type=1, dgc_sparsity=0.999)
    opt = torch.optim.AdamW(ddp.parameters(), lr=1e-4, weight_decay=0.01, fused=True)
    b, t = (4, 64) if args.small else (16, 512)
    gen = torch.Generator().manual_seed(1 + dist.get_rank())
    host = []
    for _ in range(4):
        ids = torch.randint(5, cfg.vocab_size, (b, t), generator=gen)
        x, y = mask_tokens(ids, cfg, generator=gen)
        host.append((x.pin_memory(), y.pin_memory()))

    def put(batch):
        return batch[0].to(dev, non_blocking=True), batch[1].to(dev, non_blocking=True)

    def loss_fn(batch):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return ddp(batch[0], batch[1])

    info = {"model": "bert-tiny" if args.small else "bert-large 24L d1024 h16 mlp4096 vocab30522", "unit": "tokens/s",
            "items_per_step": b * t * world, "global_batch": b * world, "seq_len": t, "parallelism": f"dp{world}",
            "compressor": "DGC sparsity 0.999 with momentum correction" if hook else "stock DDP all-reduce",
            "bucket_mb": args.bucket_mb, "optimizer": "AdamW(fused)"}
    return ddp, opt, hook, host, put, loss_fn, info


def build_llama(args, dev, world):
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    from nangila.fsdp import apply_nangila_fsdp
    from nangila.models.llama import Llama, LlamaConfig

    cfg = LlamaConfig.tiny() if args.small else LlamaConfig.llama_1_3b()
    model = Llama(cfg).to(dev)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    for blk in model.blocks:
        fully_shard(blk, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    colls = None
    if args.impl == "ours":
        colls = apply_nangila_fsdp(model, compress_gradients=True, quantize_parameters=True, parameter_bits=8)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)
    b, t = (2, 64) if args.small else (4, 2048)
    gen = torch.Generator().manual_seed(1 + dist.get_rank())
    host = [(torch.randint(0, cfg.vocab_size, (b, t + 1), generator=gen).pin_memory(),) for _ in range(4)]

    def put(batch):
        return (batch[0].to(dev, non_blocking=True),)

    def loss_fn(batch):
        tok = batch[0]
        return model(tok[:, :-1], tok[:, 1:])

    class _Hook:  # same surface as the DDP hook for the loop below
        def step(self):
            for c in colls:
                if c is not None and hasattr(c, "step"):
                    c.step += 1

        def get_kernel_launches(self):
            return sum(c.launches for c in colls if c is not None)

        def check(self):
            for c in colls:
                if c is not None:
                    c.check_status()

        def fallbacks(self):
            return sum(c.fallbacks for c in colls if c is not None)

    info = {"model": "llama-tiny" if args.small else "llama-style 24L d2048 h16 swiglu5632 vocab32000 (1.36 B)",
            "unit": "tokens/s", "items_per_step": b * t * world, "global_batch": b * world, "seq_len": t,
            "parallelism": f"fsdp{world} (fully_shard per block)",
            "compressor": "block-INT4 reduce-scatter + INT8 all-gather (fused kernels)" if colls else "stock FSDP2 (NCCL)",
            "optimizer": "AdamW(fused)"}
    return model, opt, (_Hook() if colls else None), host, put, loss_fn, info


BUILDERS = {"resnet50-powersgd": build_resnet, "bert-large-dgc": build_bert, "llama-1.3b-fsdp": build_llama}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=sorted(BUILDERS))
    ap.add_argument("--impl", default="ours", choices=["ours", "baseline"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--bucket-mb", type=int, default=25, help="DDP bucket size of the BERT configuration")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, world, dev = init_distributed()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but the launcher started {world} rank(s); use torch.distributed.run")
    seed_everything(0)
    model, opt, hook, host, put, loss_fn, info = BUILDERS[args.config](args, dev, world)
    resident = [put(b) for b in host]

    def one(batch):
        loss = loss_fn(batch)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        if hook is not None:
            hook.step()
        return loss

    def step_device(i):
        return one(resident[i % len(resident)])

    def step_e2e(i):
        return float(one(put(host[i % len(host)])).item())

    for i in range(args.warmup):
        step_device(i)
    torch.cuda.synchronize()
    l0 = hook.get_kernel_launches() if hook is not None else 0
    ms, _, clocks, last = timed_steps(step_device, args.steps, dev)
    launches = (hook.get_kernel_launches() - l0) if hook is not None else 0
    items = info.pop("items_per_step")
    unit = info.pop("unit")
    e2e = None
    if not args.no_e2e:
        ms2, wall2, _, _ = timed_steps(step_e2e, args.steps, dev)
        ms2 = max(ms2, wall2)
        h2d = sum(t.numel() * t.element_size() for t in host[0])
        e2e = {"value": items * args.steps / (ms2 / 1e3), "unit": unit, "ms_per_step": ms2 / args.steps,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4}
    if hook is not None:
        (hook.check() if hasattr(hook, "check") else hook._check_device_status())
    if rank == 0:
        out = {"metric": f"{args.config} training throughput", "value": items * args.steps / (ms / 1e3), "unit": unit,
               "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic (random inputs, random-init weights)", "impl": args.impl, "config": info,
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": float(last)}
        if hook is not None and hasattr(hook, "get_stats"):
            out["compression_ratio"] = hook.get_stats().get("overall_compression_ratio")
        if hook is not None and hasattr(hook, "fallbacks"):
            out["nccl_fallbacks"] = hook.fallbacks()
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
