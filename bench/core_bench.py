#!/usr/bin/env python
"""Host micro-benchmarks of the C++ core, the counterpart of the reference's Criterion benches
(nangila-core/benches/compressor.rs, predictor.rs, quantizer.rs): compressor round trips at 1 M
elements, predictor predict / update, quantize / dequantize at several sizes, CRC32 and the state hash.

    python bench/core_bench.py [--repeat 5]

Prints one JSON line per benchmark: best-of-N seconds, elements (or bytes) per second.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np  # noqa: E402

import nangila._C as C  # noqa: E402


def best(fn, repeat):
    fn()
    times = []
    for _ in range(repeat):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return min(times)


def report(name, seconds, count, unit="elements"):
    print(json.dumps({"bench": name, "seconds": seconds, f"{unit}_per_s": count / seconds}), flush=True)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--repeat", type=int, default=5)
    args = ap.parse_args()
    rng = np.random.default_rng(0)
    n = 1 << 20
    g = (rng.normal(size=n) * 0.01).astype(np.float32)

    for ctype, name in ((0, "prediction_residual"), (1, "dgc"), (2, "power_sgd")):
        cfg = C.NangilaConfig(compressor_type=ctype, dgc_sparsity=0.999, power_sgd_rank=4)
        comp = C.HostCompressor(cfg)
        x = g.reshape(1024, 1024) if ctype == 2 else g
        for _ in range(3):  # seed history / warm-start
            comp.update(0, comp.decompress(comp.compress(x, 0), 0))
            comp.step()
        holder = {}

        def c():
            holder["p"] = comp.compress(x, 0)

        report(f"compress_{name}_1M", best(c, args.repeat), n)
        report(f"decompress_{name}_1M", best(lambda: comp.decompress(holder["p"], 0), args.repeat), n)

    pred = C.Predictor(0.9, 0)
    pred.update(0, g)
    pred.step()
    pred.update(0, g * 1.01)
    pred.step()
    report("predictor_predict_1M", best(lambda: pred.predict(0), args.repeat), n)
    report("predictor_update_1M", best(lambda: pred.update(0, g), args.repeat), n)

    q = C.Quantizer.int4()
    for size in (1 << 10, 1 << 14, 1 << 17, 1 << 20):
        x = g[:size]
        holder = {}

        def quant():
            holder["c"] = q.quantize(x)

        report(f"quantize_{size}", best(quant, args.repeat), size)
        report(f"dequantize_{size}", best(lambda: q.dequantize(holder["c"]), args.repeat), size)
    report("full_roundtrip_1M", best(lambda: q.dequantize(q.quantize(g)), args.repeat), n)

    raw = g.tobytes()
    report("crc32_4MB", best(lambda: C.crc32(raw), args.repeat), len(raw), "bytes")
    report("siphash13_4MB", best(lambda: C.siphash13(raw), args.repeat), len(raw), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
