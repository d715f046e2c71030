#!/usr/bin/env python
"""Standalone all-reduce sweep: the fused compressed exchange (and its exact mode) against NCCL
all-reduce on N(0, 1e-3) bf16 gradient buffers from 1 MB to 1 GB.

    python bench/allreduce_sweep.py                      # 1 GPU: HBM roofline of the kernel
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/allreduce_sweep.py

Every number is device time (CUDA events on the launching stream), warm-up first, max over ranks.
Buffers rotate through a pool larger than the 126 MB L2. Per size it prints one JSON line with
  algbw  = buffer bytes / time                      ("effective GB/s": what the caller experiences)
  busbw  = algbw * 2 (W-1) / W                      (NCCL's bus-bandwidth convention)
  wire   = bytes this rank stores into peers / time  (what actually crosses NVLink)
  hbm    = algorithmic HBM bytes of the fused kernel / time
and the roofline fraction: max(wire bytes / 770 GB/s, HBM bytes / measured copy bandwidth) / time.

The reference has only a raw NCCL GB/s loop (tests/test_stress.py:195-206).
"""
import argparse
import json
import os
import socket
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool


def measured_hbm_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0


def time_ms(fn, iters: int, warmup: int = 3) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    if dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-mb", type=float, default=1)
    ap.add_argument("--max-mb", type=float, default=1024)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--iters", type=int, default=0)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--gain", type=float, default=1.0,
                    help="prediction gain of the compressed mode (0 = the history is neither read nor probed)")
    ap.add_argument("--loopback", type=int, default=0,
                    help="emulate this many ranks on ONE GPU (one cooperative launch); for profiling the multi-rank "
                         "phases under a single-process profiler")
    ap.add_argument("--out", default="")
    ap.add_argument("--only", default="", help="comma list of: nccl,exact,compressed")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in os.environ:
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        os.environ["MASTER_PORT"] = str(s.getsockname()[1])
        s.close()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from nangila.parallel.predres_engine import PredResEngine
    from nangila.parallel.symm import LoopbackArena, SymmArena

    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    esize = 2 if dtype == torch.bfloat16 else 4
    nvr = 1
    if args.loopback > 1:
        assert world == 1, "--loopback runs in a single process"
        arena = LoopbackArena(args.loopback, dev)
        nvr = world = args.loopback
    else:
        arena = SymmArena(None, dev, segment_bytes=256 << 20)
    eng = PredResEngine(arena, dev, use_side_stream=False, adaptive_gain=False, ctas=args.ctas or None)
    eng.fixed_gain = args.gain
    if args.gain == 0.0:
        eng.probe_every = 1 << 30
    hbm = measured_hbm_gbs()
    which = set(args.only.split(",")) if args.only else {"nccl", "exact", "compressed"}
    rows = []
    mb = args.min_mb
    while mb <= args.max_mb + 1e-9:
        nbytes = int(mb * (1 << 20))
        n = nbytes // esize
        pool = max(2, min(8, int((300 << 20) // max(nbytes, 1)) + 1))  # rotate through > 2x L2
        iters = args.iters or (50 if nbytes <= (16 << 20) else 20 if nbytes <= (256 << 20) else 8)
        bufs = [[(torch.randn(n, device=dev) * 1e-3).to(dtype) for _ in range(nvr)] for _ in range(pool)]
        row = {"mb": mb, "bytes": nbytes, "world": world, "dtype": args.dtype, "pool": pool, "iters": iters, "gain": args.gain,
               "loopback_ranks_on_one_gpu": nvr if nvr > 1 else None}
        scale = 2.0 * (world - 1) / world if world > 1 else 1.0
        if "nccl" in which and world > 1 and nvr == 1:
            t = time_ms(lambda i: dist.all_reduce(bufs[i % pool][0]), iters)
            row["nccl_ms"] = t
            row["nccl_algbw_gbs"] = nbytes / t / 1e6
            row["nccl_busbw_gbs"] = nbytes * scale / t / 1e6
        for mode in ("exact", "compressed"):
            if mode not in which:
                continue
            comp = mode == "compressed"
            # one bucket state per pool entry so that state traffic is not L2-resident either
            base = 1000 * int(mb * 16) + (500 if comp else 0)
            for j in range(pool):  # build history / allocate outside the timed region
                eng.reduce(base + j, bufs[j], compressed=False)
            eng.check_status()
            t = time_ms(lambda i: eng.reduce(base + i % pool, bufs[i % pool], compressed=comp, step=i), iters)
            eng.check_status()
            st = eng.buckets[base]
            wire = eng.wire_bytes(st, comp)
            ssize = st.state_dtype.itemsize
            if comp:
                q = 0.5 + 2.0 / 64
                hist = 2 * ssize if args.gain != 0.0 else 0  # history reads in phase 1 and again in phase 3
                hbm_bytes = n * (esize + hist + 2 * ssize + q) + n * q * 2 + n * (q + hist + esize + ssize)
            else:
                hbm_bytes = n * (esize * 2) + n * esize * 2 + n * (esize + esize + ssize)
            bound_ms = max(wire / (NVLINK_GBS * 1e6), hbm_bytes / (hbm * 1e6))
            row[f"{mode}_ms"] = t
            row[f"{mode}_algbw_gbs"] = nbytes / t / 1e6
            row[f"{mode}_busbw_gbs"] = nbytes * scale / t / 1e6
            row[f"{mode}_wire_gbs"] = wire / t / 1e6
            row[f"{mode}_hbm_gbs"] = hbm_bytes / t / 1e6
            row[f"{mode}_roofline_frac"] = bound_ms / t
            row[f"{mode}_bound"] = "nvlink" if wire / (NVLINK_GBS * 1e6) > hbm_bytes / (hbm * 1e6) else "hbm"
            for j in range(pool):
                eng.buckets.pop(base + j, None)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        del bufs
        torch.cuda.empty_cache()
        mb *= 4 if mb >= 4 else 2
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"hbm_gbs_measured": hbm, "nvlink_gbs": NVLINK_GBS, "rows": rows}, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
