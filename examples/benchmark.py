#!/usr/bin/env python
"""Compression ratio and throughput of the public hook API on a synthetic gradient stream.

    python examples/benchmark.py --size 1000000 --iterations 100 [--device cuda]

The stream drifts slowly (each step is the last one plus a small change), which is what the predictor is built
for. Host path: ``NangilaHook.compress`` / ``decompress`` / ``update`` on a CPU tensor. Device path
(``--device cuda``): ``compress_gpu`` / ``decompress_gpu`` / ``update_gpu``, same wire format. Counterpart of the
reference's ``examples/experimental/benchmark.py``, which only prints that it is not implemented.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import nangila  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser(description="compression ratio and throughput of the hook API")
    ap.add_argument("--size", type=int, default=1_000_000, help="elements per tensor")
    ap.add_argument("--iterations", type=int, default=100)
    ap.add_argument("--warmup-steps", type=int, default=5, help="steps sent uncompressed before compression starts (no shadow run here)")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    args = ap.parse_args()

    cfg = nangila.NangilaConfig(warmup_steps=args.warmup_steps, shadow_run_steps=0)
    hook = nangila.NangilaHook.all_drivers(1, cfg)
    gen = torch.Generator().manual_seed(0)
    base = torch.randn(args.size, generator=gen) * 0.01
    drift = torch.randn(args.size, generator=gen) * 1e-4
    dev = torch.device(args.device)
    if dev.type == "cuda" and not torch.cuda.is_available():
        print("no CUDA device", file=sys.stderr)
        return 2
    base, drift = base.to(dev), drift.to(dev)
    sync = torch.cuda.synchronize if dev.type == "cuda" else (lambda: None)

    raw_bytes = packet_bytes = 0
    t_comp = t_dec = 0.0
    err_num = err_den = 0.0
    for step in range(args.iterations + args.warmup_steps):
        grad = base + step * drift + 1e-5 * torch.randn(args.size, generator=gen).to(dev)
        sync()
        t0 = time.perf_counter()
        packet = hook.compress_gpu(0, grad) if dev.type == "cuda" else hook.compress(0, grad)
        sync()
        t1 = time.perf_counter()
        out = hook.decompress_gpu(0, packet, args.size) if dev.type == "cuda" else hook.decompress(0, packet)
        sync()
        t2 = time.perf_counter()
        if dev.type == "cuda":
            hook.update_gpu(0, out)
        else:
            hook.update(0, out)
        hook.step()
        if step >= args.warmup_steps:
            raw_bytes += args.size * 4
            packet_bytes += packet.numel() if hasattr(packet, "numel") else len(packet)
            t_comp += t1 - t0
            t_dec += t2 - t1
            out_t = out if isinstance(out, torch.Tensor) else torch.as_tensor(out)
            err_num += float((out_t.reshape(-1).to(grad) - grad).pow(2).sum())
            err_den += float(grad.pow(2).sum())
    n = args.iterations
    print(json.dumps({
        "device": args.device, "elements": args.size, "iterations": n,
        "compression_ratio": raw_bytes / max(packet_bytes, 1),
        "compress_melem_per_s": args.size * n / t_comp / 1e6, "decompress_melem_per_s": args.size * n / t_dec / 1e6,
        "relative_rms_error": (err_num / max(err_den, 1e-300)) ** 0.5,
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
