"""Looking at ``.nz`` files: a plot when matplotlib is installed, a text chart otherwise, and a
comparison of a compressed waveform with its source. Counterpart of the reference's ``nz_viewer.py``."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from .nz_reader import NzWaveform, read_nz


def ascii_chart(time: np.ndarray, values: np.ndarray, width: int = 72, height: int = 12, label: str = "") -> str:
    if not len(time):
        return f"{label}: (empty)"
    idx = np.linspace(0, len(time) - 1, min(width, len(time))).astype(int)
    v = np.asarray(values, float)[idx]
    lo, hi = float(v.min()), float(v.max())
    span = hi - lo if hi > lo else 1.0
    rows = [[" "] * len(idx) for _ in range(height)]
    for x, val in enumerate(v):
        rows[height - 1 - int(round((val - lo) / span * (height - 1)))][x] = "*"
    lines = [f"{label}  [{lo:+.4f} V .. {hi:+.4f} V]  t = {time[0]:.3e} .. {time[-1]:.3e} s"]
    lines += ["|" + "".join(r) for r in rows]
    return "\n".join(lines)


def plot_nz(path: str, nodes: Optional[Sequence[str]] = None, output: Optional[str] = None, max_nodes: int = 8) -> str:
    """Draws the chosen nets. Returns the path of the image written (matplotlib) or the text chart."""
    w = read_nz(path)
    chosen = [n for n in (nodes or w.node_names) if n in w.signals][:max_nodes]
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        return "\n\n".join([w.summary()] + [ascii_chart(w.time, w.signals[n], label=n) for n in chosen])
    fig, ax = plt.subplots(figsize=(9, 4))
    for n in chosen:
        ax.plot(w.time, w.signals[n], label=n)
    ax.set_xlabel("time (s)")
    ax.set_ylabel("V")
    ax.set_title(w.summary())
    ax.legend()
    out = output or (path + ".png")
    fig.savefig(out, dpi=120)
    plt.close(fig)
    return out


def compare_waveforms(nz: NzWaveform, original: dict, time: Optional[Sequence[float]] = None) -> dict:
    """Per-net maximum absolute error of a decoded file against the uncompressed signals."""
    errs = {}
    for name, ref in original.items():
        if name in nz.signals:
            errs[name] = float(np.abs(np.asarray(ref, float) - nz.signals[name]).max())
    worst = max(errs.values()) if errs else float("nan")
    return {"per_node": errs, "max_abs_error": worst, "within_bound": bool(errs) and worst <= nz.header.error_bound * (1 + 1e-9)}
