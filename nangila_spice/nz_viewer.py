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


_TIME_UNITS = {"ps": 1e12, "ns": 1e9, "us": 1e6, "ms": 1e3, "s": 1.0}


def _time_unit(span: float, requested: str = "auto") -> str:
    """The unit the time axis is written in: the requested one, or the largest in which ``span`` is at least 1."""
    if requested in _TIME_UNITS:
        return requested
    for unit in ("s", "ms", "us", "ns"):
        if span * _TIME_UNITS[unit] >= 1.0:
            return unit
    return "ps"


def _load(source) -> NzWaveform:
    if isinstance(source, NzWaveform):
        return source
    if isinstance(source, (str, bytes)) or hasattr(source, "__fspath__"):
        return read_nz(source)
    raise TypeError(f"expected a path or an NzWaveform, got {type(source).__name__}")


def _pyplot():
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt

        return plt
    except Exception:
        return None


def plot_nz(source, nodes: Optional[Sequence[str]] = None, output: Optional[str] = None, max_nodes: int = 8, *, title: Optional[str] = None,
            show_error_bound: bool = False, output_path: Optional[str] = None, figsize: tuple = (12, 6), time_scale: str = "auto") -> str:
    """Draws the chosen nets of a ``.nz`` file (a path) or of an ``NzWaveform``. With matplotlib: an image (``output_path``
    / ``output``, default ``<file>.png``), whose path is returned; ``show_error_bound`` shades the band the decoded samples
    are guaranteed to lie in, ``time_scale`` is ``auto``, ``ps``, ``ns``, ``us`` or ``ms``. Without matplotlib: the text
    chart is returned (and written to ``output_path`` when one is given). The keyword names are the reference's
    (nz_viewer.py:17-128)."""
    w = _load(source)
    missing = [n for n in (nodes or []) if n not in w.signals]
    chosen = [n for n in (nodes or w.node_names) if n in w.signals][:max_nodes]
    unit = _time_unit(float(w.header.t_end - w.header.t_start), time_scale)
    heading = title or w.summary()
    out = output_path or output
    plt = _pyplot()
    if plt is None or not chosen:
        notes = [f"(not in the file: {', '.join(missing)})"] if missing else []
        text = "\n\n".join([heading] + notes + [ascii_chart(w.time, w.signals[n], label=n) for n in chosen])
        if out and not str(out).lower().endswith((".png", ".pdf", ".svg", ".jpg")):
            with open(out, "w") as fh:
                fh.write(text + "\n")
        return text
    fig, ax = plt.subplots(figsize=figsize)
    t = np.asarray(w.time) * _TIME_UNITS[unit]
    for n in chosen:
        line, = ax.plot(t, w.signals[n], label=n, linewidth=1.5)
        if show_error_bound and w.header.error_bound > 0:
            ax.fill_between(t, w.signals[n] - w.header.error_bound, w.signals[n] + w.header.error_bound, alpha=0.15, color=line.get_color())
    ax.set_xlabel(f"time ({unit})")
    ax.set_ylabel("V")
    ax.set_title(heading)
    ax.grid(True, alpha=0.3)
    ax.legend(loc="best")
    if out is None:
        out = (source if isinstance(source, str) else "waveform.nz") + ".png"
    fig.savefig(out, dpi=150, bbox_inches="tight")
    plt.close(fig)
    return out


def compression_errors(nz: NzWaveform, original: dict) -> dict:
    """Per-net maximum absolute error of a decoded file against the uncompressed signals (``{name: samples}``)."""
    errs = {}
    for name, ref in original.items():
        if name in nz.signals:
            errs[name] = float(np.abs(np.asarray(ref, float) - nz.signals[name]).max())
    worst = max(errs.values()) if errs else float("nan")
    return {"per_node": errs, "max_abs_error": worst, "within_bound": bool(errs) and worst <= nz.header.error_bound * (1 + 1e-9)}


def compare_waveforms(*args, **kwargs) -> dict:
    """Error of a compressed waveform against its source, in either calling form:

    * ``compare_waveforms(nz, {"net": samples, ...})``: per-net errors (``compression_errors``);
    * ``compare_waveforms(original_time, original_values, nz_source, node, title=None, output_path=None)``, the
      reference's (nz_viewer.py:131-211): one net, the original interpolated onto the file's time points when the two
      axes differ; with matplotlib and an ``output_path`` also a two-panel figure (both curves, and their difference
      against the error bound).

    Both return ``{"per_node", "max_abs_error", "within_bound"}``."""
    if len(args) >= 2 and isinstance(args[0], NzWaveform) and isinstance(args[1], dict):
        return compression_errors(args[0], args[1])
    names = ("original_time", "original_values", "nz_source", "node", "title", "output_path")
    call = dict(zip(names, args))
    call.update(kwargs)
    w = _load(call["nz_source"])
    node = call["node"]
    if node not in w.signals:
        raise KeyError(f"net {node!r} is not in the file (it has: {', '.join(w.node_names[:8])}...)")
    t0, v0 = np.asarray(call["original_time"], float), np.asarray(call["original_values"], float)
    same_axis = len(t0) == len(w.time) and np.allclose(t0, w.time, rtol=0, atol=1e-18)
    ref = v0 if same_axis else np.interp(w.time, t0, v0)
    result = compression_errors(w, {node: ref})
    plt = _pyplot()
    if plt is not None and call.get("output_path"):
        unit = _time_unit(float(w.header.t_end - w.header.t_start))
        t = np.asarray(w.time) * _TIME_UNITS[unit]
        fig, (top, bottom) = plt.subplots(2, 1, figsize=(12, 7), sharex=True)
        top.plot(t, ref, label="original", linewidth=1.5)
        top.plot(t, w.signals[node], label=".nz", linewidth=1.0, linestyle="--")
        top.set_ylabel("V")
        top.set_title(call.get("title") or f"{node}: original and compressed")
        top.legend(loc="best")
        bottom.plot(t, w.signals[node] - ref, linewidth=1.0)
        for sign in (-1.0, 1.0):
            bottom.axhline(sign * w.header.error_bound, color="gray", linestyle=":")
        bottom.set_xlabel(f"time ({unit})")
        bottom.set_ylabel("difference (V)")
        fig.savefig(call["output_path"], dpi=150, bbox_inches="tight")
        plt.close(fig)
    return result
