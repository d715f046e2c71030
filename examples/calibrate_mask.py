#!/usr/bin/env python
"""Sculptor calibration: record per-layer gradients for a few steps, derive the Driver / Passenger
topology, save the mask, build a hook from it and push one gradient through compress / decompress.
Runs on CPU."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn as nn  # noqa: E402

import nangila  # noqa: E402


def main() -> int:
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(64, 64), nn.Tanh(), nn.Linear(64, 64), nn.Tanh(), nn.Linear(64, 8))
    sculptor = nangila.Sculptor(threshold=0.9)
    for step in range(40):
        x = torch.randn(32, 64)
        loss = model(x).pow(2).mean()
        model.zero_grad()
        loss.backward()
        for layer_id, p in enumerate(model.parameters()):
            sculptor.record(layer_id, p.grad.detach().reshape(-1).numpy())
        sculptor.end_step()
    mask = sculptor.generate_mask()
    path = os.path.join(tempfile.mkdtemp(), "topology.mask")
    with open(path, "wb") as f:
        f.write(mask)
    cfg = nangila.NangilaConfig(warmup_steps=0, shadow_run_steps=0)
    hook = nangila.NangilaHook.from_mask_file(path, cfg)
    st = hook.get_stats()
    print(f"mask: {len(mask)} bytes, {st['num_drivers']} drivers, {st['num_passengers']} passengers -> {path}")
    g = next(model.parameters()).grad.detach().reshape(-1).numpy()
    for _ in range(3):  # the first packets seed the predictor
        packet = hook.compress(0, g)
        hook.update(0, hook.decompress_gathered(0, packet))
        hook.step()
    packet = hook.compress(0, g)
    rec = hook.decompress_gathered(0, packet)
    print(f"layer 0: {g.nbytes} bytes -> {len(packet)} bytes, max error {np.abs(rec - g).max():.3e}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
