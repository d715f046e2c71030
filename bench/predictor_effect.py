#!/usr/bin/env python
"""What the momentum predictor buys, and when the gain controller switches it on.

Two synthetic gradient streams through the fused bucket kernel (one GPU; ``--ranks N`` emulates N ranks in one
launch): ``drift``, a gradient that moves slowly from step to step plus per-rank noise (what fine-tuning or a
late, smooth phase of training looks like), and ``noise``, independent draws every step (what uniform random
tokens give). For each: the gain the controller settles on per bucket, the residual energy relative to the
gradient, and the error of the reconstructed mean against the exact mean, with the adaptive gain and with the
gain forced to 0. One JSON line per (stream, setting).

    python bench/predictor_effect.py --ranks 2 --mb 64
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def run(stream: str, forced_zero: bool, ranks: int, n: int, buckets: int, steps: int, dev) -> dict:
    from nangila.parallel.predres_engine import PredResEngine
    from nangila.parallel.symm import LoopbackArena

    eng = PredResEngine(LoopbackArena(ranks, dev), dev, stochastic=False, error_feedback=True, use_side_stream=False,
                        adaptive_gain=not forced_zero)
    if forced_zero:
        eng.fixed_gain = 0.0
    torch.manual_seed(0)
    base = [torch.randn(n, device=dev) * 0.02 for _ in range(buckets)]
    drift = [torch.randn(n, device=dev) * 0.002 for _ in range(buckets)]
    errs, resid = [], []
    for step in range(steps):
        for b in range(buckets):
            if stream == "drift":
                grads = [(base[b] + drift[b] * step + torch.randn(n, device=dev) * 5e-4).to(torch.bfloat16) for _ in range(ranks)]
            else:
                grads = [(torch.randn(n, device=dev) * 0.02).to(torch.bfloat16) for _ in range(ranks)]
            exact = torch.stack([g.float() for g in grads]).mean(0)
            eng.reduce(b, grads, compressed=step >= 2, step=step)
            if step >= steps - 8:
                errs.append(((grads[0].float() - exact).norm() / exact.norm()).item())
        eng.end_step()
    eng.check_status()
    gains = [eng.buckets[b].pred_gain for b in range(buckets)]
    for b in range(buckets):
        st = eng.buckets[b]
        if st.totals[1] > 0:
            resid.append((st.totals[0] / st.totals[1]) ** 0.5)
    return {"stream": stream, "gain": "forced 0" if forced_zero else "adaptive", "ranks": ranks, "elements_per_bucket": n,
            "gain_per_bucket": [round(g, 3) for g in gains], "buckets_with_prediction": sum(1 for g in gains if g > 0) / buckets,
            "residual_over_gradient": round(sum(resid) / len(resid), 4) if resid else None,
            "reconstruction_rel_error_last_steps": round(sum(errs) / len(errs), 5)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--mb", type=float, default=32)
    ap.add_argument("--buckets", type=int, default=4)
    ap.add_argument("--steps", type=int, default=40)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    n = int(args.mb * (1 << 20) / 2)
    for stream in ("drift", "noise"):
        for forced in (False, True):
            print(json.dumps(run(stream, forced, args.ranks, n, args.buckets, args.steps, dev)), flush=True)


if __name__ == "__main__":
    main()
