#!/usr/bin/env python
"""FP64 CSR SpMV benchmark of the circuit simulator's device kernel.

The workload is the one of the reference's GPU benchmark (a tridiagonal matrix, the pattern of an RC
ladder; 1 M rows, 200 products: ``nangila-spice/nangila-node/src/bin/bench_gpu.rs``) plus a size that
does not fit in L2, and the library baseline: the same product through ``torch.sparse_csr_tensor``
(cuSPARSE). Vectors stay on the device in both arms; timing is by CUDA events after warm-up.

    python bench/spmv_bench.py [--rows 1000000 16000000] [--iters 200] [--out FILE]
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nangila.utils.benchmarking import ClockSampler  # noqa: E402
from nangila_spice.gpu import DeviceCsr, tridiagonal  # noqa: E402


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def timed(fn, iters: int) -> float:
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="+", default=[1_000_000, 16_000_000])
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    hbm, src = peaks()
    stream = torch.cuda.current_stream().cuda_stream
    results = []
    for n in args.rows:
        row_ptr, col, val = tridiagonal(n)
        nnz = int(val.size)
        m = DeviceCsr(row_ptr, col, val)
        x = torch.randn(n, dtype=torch.float64, device="cuda")
        y = torch.empty_like(x)
        sampler = ClockSampler(0).start()
        ours = timed(lambda: m.matvec_device(x, y, stream), args.iters)
        clocks = sampler.stop()
        m.check_status()
        os.environ["NANGILA_SPMV_TILE"] = "1024"
        ms_ = DeviceCsr(row_ptr, col, val)
        os.environ.pop("NANGILA_SPMV_TILE")
        y3 = torch.empty_like(x)
        small = timed(lambda: ms_.matvec_device(x, y3, stream), args.iters)
        assert torch.equal(y, y3)
        ms_.close()
        mp = DeviceCsr(row_ptr, col, val, plain_loads=True)
        y2 = torch.empty_like(x)
        plain = timed(lambda: mp.matvec_device(x, y2, stream), args.iters)
        assert torch.equal(y, y2)
        mp.close()
        A = torch.sparse_csr_tensor(torch.from_numpy(row_ptr.astype(np.int64)).cuda().to(torch.int32), torch.from_numpy(col).cuda(),
                                    torch.from_numpy(val).cuda(), size=(n, n))
        ref_y = A @ x
        err = (ref_y - y).abs().max().item()
        lib = timed(lambda: torch.mv(A, x), args.iters)
        # algorithmic traffic: values + column indices + row pointers + x read once + y written once
        bytes_moved = nnz * 12 + (n + 1) * 4 + n * 16
        rec = {"kernel": "spmv_row_blocks_bulk_kernel", "rows": n, "nnz": nnz, "ms": ours, "plain_load_variant_ms": plain, "tile_1024_variant_ms": small, "gbs": bytes_moved / ours / 1e6,
               f"frac_of_{src}_hbm": bytes_moved / ours / 1e6 / hbm, "cusparse_ms": lib, "speedup_vs_cusparse": lib / ours,
               "max_abs_diff_vs_cusparse": err, "working_set_mb": bytes_moved / 1e6, "fits_l2": bytes_moved < 126e6, "clocks": clocks}
        print(json.dumps(rec), flush=True)
        results.append(rec)
        m.close()
        del A, x, y
    if args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
