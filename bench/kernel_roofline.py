#!/usr/bin/env python
"""Achieved fraction of roofline of every fused kernel, one JSON line per kernel and size.

    python bench/kernel_roofline.py                       # 1 GPU: the HBM side of each kernel
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/kernel_roofline.py

For each kernel the bound is the slowest of
  * algorithmic HBM bytes / measured copy bandwidth (MEASURED_PEAKS.json, else 6650 GB/s),
  * bytes this rank must store into its peers / 770 GB/s (measured peer copy, per direction),
  * FLOPs / measured bf16 GEMM rate (PowerSGD projections only),
and ``frac`` = bound / device time (CUDA events, warm-up first, max over ranks, working set rotated
through a pool larger than the 126 MB L2). "Algorithmic bytes" are the compulsory ones of the
operation as specified — each input read once, each output written once — so passes a kernel makes
beyond that (the radix-select passes of DGC, say) count against it.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 770.0


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def time_ms(fn, iters, warmup=3):
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
    ap.add_argument("--mb", type=float, default=256, help="gradient buffer size per rank in MB (bf16 elements)")
    ap.add_argument("--only", default="", help="comma list of: predres,dgc,powersgd,rs,ag")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from nangila.parallel.dgc_engine import DGCEngine
    from nangila.parallel.fsdp_collectives import NangilaAllGather, NangilaReduceScatter
    from nangila.parallel.powersgd_engine import PowerSGDEngine
    from nangila.parallel.predres_engine import PredResEngine
    from nangila.parallel.symm import SymmArena

    hbm, tflops, src = peaks()
    which = set(args.only.split(",")) if args.only else {"predres", "dgc", "powersgd", "rs", "ag"}
    n = int(args.mb * (1 << 20)) // 2
    n -= n % (8 * world * 2048)
    pool = max(2, min(4, int((300 << 20) // max(2 * n, 1)) + 1))
    arena = SymmArena(None, dev, segment_bytes=512 << 20)
    rows = []

    def emit(kernel, ms, hbm_bytes, wire_bytes=0.0, flops=0.0, **extra):
        t_hbm = hbm_bytes / (hbm * 1e6)
        t_wire = wire_bytes / (NVLINK_GBS * 1e6)
        t_flop = flops / (tflops * 1e9)
        bound = max(t_hbm, t_wire, t_flop)
        row = {"kernel": kernel, "world": world, "elements": n, "ms": ms, "hbm_gbs": hbm_bytes / ms / 1e6,
               "wire_gbs": wire_bytes / ms / 1e6, "tflops": flops / ms / 1e9,
               "bound": "hbm" if bound == t_hbm else ("nvlink" if bound == t_wire else "tensor"),
               "bound_ms": bound, "frac_of_" + src: bound / ms, **extra}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    w1 = (world - 1) / world
    q4 = 0.5 + 2.0 / 64  # bytes per element of the block-INT4 format
    mk = lambda dt=torch.bfloat16: [(torch.randn(n, device=dev) * 1e-3).to(dt) for _ in range(pool)]  # noqa: E731

    if "predres" in which:
        eng = PredResEngine(arena, dev, use_side_stream=False, adaptive_gain=False)
        bufs = mk()
        for gain, name in ((1.0, "predres_bucket (history read, gain 1)"), (0.0, "predres_bucket (gain 0)")):
            eng.fixed_gain = gain
            eng.probe_every = 1 << 30 if gain == 0.0 else 8
            base = 100 if gain else 200
            for j in range(pool):
                eng.reduce(base + j, [bufs[j]], compressed=False)
            ms = time_ms(lambda i: eng.reduce(base + i % pool, [bufs[i % pool]], compressed=True, step=i), args.iters)
            eng.check_status()
            hist = 4 if gain else 0
            if world == 1:  # one pass: read g, ef (+ history), write ef, g, history
                hb = n * (2 + 2 + hist + 2 + 2 + 2)
            else:
                hb = n * (2 + hist + 4 + q4) + n * q4 * 2 + n * (q4 + hist + 2 + 2)
            emit(name, ms, hb, 2 * n * q4 * w1, algbw_gbs=2 * n / ms / 1e6)
            for j in range(pool):
                eng.buckets.pop(base + j, None)
        del bufs

    if "dgc" in which:
        eng = DGCEngine(arena, dev, sparsity=0.999)
        # One bucket state (gradient + u + v = 12 bytes per element, far larger than L2) fed with a cycle of
        # independent zero-mean gradients, as in training: after the untimed calls the accumulated |v|
        # and with it the selection threshold move by about 1 % per call, which is the regime the
        # candidate list is built for. The kernel overwrites its input, so every call gets a fresh copy
        # whose time is measured separately and subtracted.
        noise = [torch.randn(n, device=dev) * 1e-3 for _ in range(8)]
        work = torch.empty_like(noise[0])
        for w in range(64):
            work.copy_(noise[w % 8])
            eng.reduce(0, work)

        def dgc_call(i):
            work.copy_(noise[i % 8])
            eng.reduce(0, work)

        t_copy = time_ms(lambda i: work.copy_(noise[i % 8]), args.iters)
        ms = time_ms(dgc_call, args.iters) - t_copy
        eng.check_status()
        k = eng.buckets[0].k
        # read g, u, v; write u, v; one selection pass over v; dense result written once
        hb = n * (4 + 8 + 8 + 4 + 4)
        tele = eng.buckets[0].scratch[0][2048 + 2048 + 512:2048 + 2048 + 512 + 4].tolist()  # cursor, candidates seen, path
        emit("dgc_fused (sparsity 0.999, fp32)", ms, hb, 8.0 * k * (world - 1), k=k, refill_copy_ms_subtracted=t_copy,
             selected=tele[0], candidates_seen=tele[3], selection_from_candidate_list=bool(tele[2]))
        del noise, eng, work

    if "powersgd" in which:
        m_rows = 4096
        cols = (n // m_rows) // 8 * 8
        eng = PowerSGDEngine(arena, dev, rank=4)
        mats = [(torch.randn(m_rows, cols, device=dev) * 1e-3).to(torch.bfloat16) for _ in range(pool)]
        for j in range(pool):
            eng.compress_matrix((j, 0), [mats[j]])
        ms = time_ms(lambda i: eng.compress_matrix((i % pool, 0), [mats[i % pool]]), args.iters)
        eng.check_status()
        el = m_rows * cols
        # prep: read g, ef, write m+ef; two projections read m+ef once each; reconstruct reads m+ef, writes g, ef
        hb = el * (2 + 2 + 2) + el * 2 * 2 + el * (2 + 2 + 2)
        emit("powersgd step (prep + 2 tcgen05 GEMMs + 2 exchanges + reconstruct), rank 4", ms, hb,
             (m_rows + cols) * 4 * 4 * (world - 1), 2 * 2.0 * el * 16, shape=[m_rows, cols])
        G = eng._glue
        st = eng.states[(0, 0)]
        ms = time_ms(lambda i: G.psgd_gemm(eng.states[(i % pool, 0)].mef[0], eng.states[(i % pool, 0)].qt[0], False,
                                           eng.states[(i % pool, 0)].p_local[0], eng.status[0], 2.0), args.iters)
        emit("psgd_gemm P = M Q (tcgen05, K-major)", ms, el * 2, 0.0, 2.0 * el * 16, shape=[m_rows, cols])
        ms = time_ms(lambda i: G.psgd_gemm(eng.states[(i % pool, 0)].mef[0], eng.states[(i % pool, 0)].pt[0], True,
                                           eng.states[(i % pool, 0)].q_local[0], eng.status[0], 2.0), args.iters)
        emit("psgd_gemm Q = M^T P (tcgen05, MN-major A)", ms, el * 2, 0.0, 2.0 * el * 16, shape=[m_rows, cols])
        del mats, eng, st

    if "rs" in which:
        rs = NangilaReduceScatter(arena=arena)
        bufs = mk()
        outs = [torch.empty(n // world, dtype=torch.bfloat16, device=dev) for _ in range(pool)]
        rs.reduce([outs[0]], [bufs[0]], 1.0 / world)
        ms = time_ms(lambda i: rs.reduce([outs[i % pool]], [bufs[i % pool]], 1.0 / world), args.iters)
        rs.check_status()
        hb = n * (2 + q4) + n * q4 + (n / world) * 2
        emit("reduce-scatter, block-INT4 (fsdp)", ms, hb, n * q4 * w1, nccl_equiv_algbw_gbs=2 * n / ms / 1e6)
        if world > 1:
            ms = time_ms(lambda i: dist.reduce_scatter_tensor(outs[i % pool], bufs[i % pool], op=dist.ReduceOp.AVG), args.iters)
            emit("NCCL reduce_scatter_tensor (bf16)", ms, n * 2 + n / world * 2, n * 2 * w1)
        del bufs, outs

    if "ag" in which:
        ag = NangilaAllGather(arena=arena, bits=8)
        shard = n // world
        ins = [(torch.randn(shard, device=dev) * 0.02).to(torch.bfloat16) for _ in range(pool)]
        outs = [torch.empty(n, dtype=torch.bfloat16, device=dev) for _ in range(pool)]
        ag.gather([outs[0]], [ins[0]])
        ms = time_ms(lambda i: ag.gather([outs[i % pool]], [ins[i % pool]]), args.iters)
        ag.check_status()
        q8 = 1.0 + 2.0 / 64
        hb = shard * 2 + n * q8 * 2 + n * 2  # read shard, slots written and read once, unsharded output written
        emit("all-gather, INT8 dequantizing (fsdp)", ms, hb, shard * q8 * (world - 1), nccl_equiv_algbw_gbs=2 * n / ms / 1e6)
        if world > 1:
            ms = time_ms(lambda i: dist.all_gather_into_tensor(outs[i % pool], ins[i % pool]), args.iters)
            emit("NCCL all_gather_into_tensor (bf16)", ms, shard * 2 + n * 2, shard * 2 * (world - 1))

    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
