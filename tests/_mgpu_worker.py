"""Multi-GPU worker (one process per GPU, launched by torch.distributed.run): checks the fused
exchange over real peer memory against NCCL, and DDP loss parity with and without the hook."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def check_exchange(dev, rank, world, results):
    from nangila.parallel.predres_engine import PredResEngine
    from nangila.parallel.symm import SymmArena

    arena = SymmArena(None, dev)
    eng = PredResEngine(arena, dev, stochastic=True, error_feedback=True, adaptive_gain=False)
    results["provider"] = arena.provider
    for dtype in (torch.float32, torch.bfloat16):
        for n in (4096 * 3 + 5, 1 << 20, 5_000_000):
            idx = hash((str(dtype), n)) % 1000
            torch.manual_seed(100 + rank)
            g = (torch.randn(n, device=dev) * 0.01).to(dtype)
            want = g.float().clone()
            dist.all_reduce(want)
            want /= world
            mine = g.clone()
            eng.reduce(idx, [mine], compressed=False)
            eng.check_status()
            tol = 1e-6 if dtype == torch.float32 else 2e-4
            err = (mine.float() - want).abs().max().item()
            assert err <= tol + 8e-3 * want.abs().max().item() * (dtype == torch.bfloat16), (dtype, n, err)
            # every rank holds the same bytes
            chk = mine.float().sum().double().reshape(1)
            allc = [torch.zeros_like(chk) for _ in range(world)]
            dist.all_gather(allc, chk)
            assert all(torch.equal(a, allc[0]) for a in allc), "ranks disagree (uncompressed)"
            # compressed step: bounded error against the exact mean, identical on all ranks
            g2 = (want + torch.randn(n, device=dev) * 0.002).to(dtype)
            want2 = g2.float().clone()
            dist.all_reduce(want2)
            want2 /= world
            mine2 = g2.clone()
            eng.reduce(idx, [mine2], compressed=True, step=1)
            eng.check_status()
            rel = ((mine2.float() - want2).norm() / want2.norm()).item()
            assert rel < 0.2, (dtype, n, rel)
            chk = mine2.float().sum().double().reshape(1)
            dist.all_gather(allc, chk)
            assert all(torch.equal(a, allc[0]) for a in allc), "ranks disagree (compressed)"
            results[f"rel_err_{str(dtype)[6:]}_{n}"] = rel


def train(dev, rank, world, use_hook, steps, compressor_type=0, prefer_cpp=True):
    from torch.nn.parallel import DistributedDataParallel as DDP

    from nangila.ddp import register_nangila_hook
    from nangila.models.gpt2 import GPT2, GPT2Config

    torch.manual_seed(0)
    cfg = GPT2Config.tiny()
    model = GPT2(cfg).to(dev)
    ddp = DDP(model, device_ids=[dev.index], bucket_cap_mb=1)
    hook = None
    if use_hook:
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            hook = register_nangila_hook(ddp, warmup_steps=10, sync_mode=1, compressor_type=compressor_type, prefer_cpp=prefer_cpp,
                                         dgc_sparsity=0.99 if compressor_type == 1 else 0.999,
                                         power_sgd_rank=4 if compressor_type == 2 else 1)
    opt = torch.optim.AdamW(ddp.parameters(), lr=3e-3)
    gen = torch.Generator().manual_seed(7)  # same data stream on every rank; each takes its slice
    data = torch.randint(0, 64, (64, 33), generator=gen)  # small vocabulary subset: learnable
    losses = []
    for step in range(steps):
        rows = torch.randint(0, 64, (4 * world,), generator=gen)[rank * 4:(rank + 1) * 4]
        tok = data[rows].to(dev)
        loss = ddp(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        if hook is not None:
            hook.step()
        losses.append(loss.detach())
    out = torch.stack(losses).float()
    dist.all_reduce(out)
    out /= world
    p0 = next(model.parameters()).detach().float().sum().double().reshape(1)
    allp = [torch.zeros_like(p0) for _ in range(world)]
    dist.all_gather(allp, p0)
    assert all(torch.equal(a, allp[0]) for a in allp), "model replicas diverged"
    stats = hook.get_stats() if hook is not None else None
    return out.tolist(), stats


def train_fsdp(dev, rank, world, compress, steps):
    """FSDP2 on a tiny Llama: per-block fully_shard, bf16 mixed precision, optional fused collectives."""
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    from nangila.fsdp import apply_nangila_fsdp
    from nangila.models.llama import Llama, LlamaConfig

    torch.manual_seed(0)
    model = Llama(LlamaConfig.tiny()).to(dev)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
    for blk in model.blocks:
        fully_shard(blk, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    rs = ag = None
    if compress:
        rs, ag = apply_nangila_fsdp(model, parameter_bits=8)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    gen = torch.Generator().manual_seed(7)
    data = torch.randint(0, 64, (64, 33), generator=gen)
    losses = []
    for step in range(steps):
        rows = torch.randint(0, 64, (4 * world,), generator=gen)[rank * 4:(rank + 1) * 4]
        tok = data[rows].to(dev)
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        if rs is not None:
            rs.step += 1
        losses.append(loss.detach())
    out = torch.stack(losses).float()
    dist.all_reduce(out)
    out /= world
    info = None
    if compress:
        rs.check_status()
        ag.check_status()
        info = {"rs_launches": rs.launches, "ag_launches": ag.launches, "fallbacks": rs.fallbacks + ag.fallbacks}
    return out.tolist(), info


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    out_path = sys.argv[2] if len(sys.argv) > 2 else None
    results = {"world": world}
    if what in ("all", "exchange"):
        check_exchange(dev, rank, world, results)
    if what in ("all", "train"):
        base, _ = train(dev, rank, world, False, 60)
        ours, stats = train(dev, rank, world, True, 60)
        results["loss_base"] = sum(base[-10:]) / 10
        results["loss_ours"] = sum(ours[-10:]) / 10
        results["loss_first"] = base[0]
        results["compression_ratio"] = stats["overall_compression_ratio"]
        results["launches"] = stats["kernel_launches"]
        results["cpp_hook"] = bool(stats.get("cpp_hook"))
        py_losses, py_stats = train(dev, rank, world, True, 60, prefer_cpp=False)
        results["loss_ours_python_hook"] = sum(py_losses[-10:]) / 10
        assert not py_stats.get("cpp_hook") and py_stats["kernel_launches"] > 0
        assert abs(results["loss_ours_python_hook"] - results["loss_base"]) < 0.15 * results["loss_base"] + 0.05, results
        assert results["loss_base"] < 0.8 * base[0], "baseline did not learn"
        assert abs(results["loss_ours"] - results["loss_base"]) < 0.15 * results["loss_base"] + 0.05, results
    if what in ("all", "compressors"):
        base, _ = train(dev, rank, world, False, 60)
        for ctype, name in ((1, "dgc"), (2, "powersgd")):
            ours, stats = train(dev, rank, world, True, 60, compressor_type=ctype)
            results[f"loss_{name}"] = sum(ours[-10:]) / 10
            results[f"ratio_{name}"] = stats["overall_compression_ratio"]
            assert results[f"loss_{name}"] < 0.9 * base[0], (name, results)
        results["loss_base"] = sum(base[-10:]) / 10
    if what in ("all", "fsdp"):
        base, _ = train_fsdp(dev, rank, world, False, 60)
        ours, info = train_fsdp(dev, rank, world, True, 60)
        results["fsdp_loss_base"] = sum(base[-10:]) / 10
        results["fsdp_loss_ours"] = sum(ours[-10:]) / 10
        results["fsdp"] = info
        assert results["fsdp_loss_base"] < 0.8 * base[0], "FSDP baseline did not learn"
        assert abs(results["fsdp_loss_ours"] - results["fsdp_loss_base"]) < 0.2 * results["fsdp_loss_base"] + 0.05, results
        assert info["rs_launches"] > 0 and info["ag_launches"] > 0
    if rank == 0:
        print("MGPU_RESULT " + json.dumps(results), flush=True)
        if out_path:
            with open(out_path, "w") as f:
                json.dump(results, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
