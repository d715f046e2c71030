#!/usr/bin/env python
"""Fused cross-entropy (csrc/kernels/fused_ce.cu) against PyTorch's eager path on the LM-head shape of
the GPT-2 benchmark (rows x 50304 bf16 logits, 50257 classes): forward + backward time and the
fraction of the measured copy bandwidth the fused pair reaches (3 passes over the logits).

    python bench/ce_bench.py [--rows 8192] [--iters 20]
"""
import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nangila.ops.fused_ce import fused_cross_entropy  # noqa: E402


def timed(fn, iters):
    for _ in range(3):
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
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=50304)
    ap.add_argument("--classes", type=int, default=50257)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    try:
        hbm = float(json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")))["hbm_gbs"])
        src = "measured"
    except Exception:
        hbm, src = 6650.0, "fallback"
    logits = (torch.randn(args.rows, args.cols, device="cuda") * 2.0).to(torch.bfloat16).requires_grad_(True)
    targets = torch.randint(0, args.classes, (args.rows,), device="cuda")

    def fused():
        logits.grad = None
        fused_cross_entropy(logits, targets, args.classes).backward()

    def eager():
        logits.grad = None
        F.cross_entropy(logits[:, :args.classes].float(), targets).backward()

    ms_f, ms_e = timed(fused, args.iters), timed(eager, args.iters)
    nbytes = 3 * args.rows * args.cols * 2  # forward read, backward read, gradient write
    print(json.dumps({"kernel": "ce_forward_kernel + ce_backward_kernel", "rows": args.rows, "cols": args.cols, "fused_ms": ms_f, "eager_ms": ms_e,
                      "speedup": ms_e / ms_f, "gbs": nbytes / ms_f / 1e6, f"frac_of_{src}_hbm": nbytes / ms_f / 1e6 / hbm}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
