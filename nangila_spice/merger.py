"""Waveform container and merging of per-partition results.

API counterpart: ``nangila-spice/src/nangila_spice/merger.py:22-264`` of the reference. Storage here
is columnar (one NumPy array per net on a shared time axis) instead of a list of per-point dicts.
"""
from __future__ import annotations

import csv
import json
from dataclasses import dataclass, field
from typing import Iterable, Optional

import numpy as np


@dataclass
class WaveformPoint:
    time: float
    voltages: dict[str, float] = field(default_factory=dict)


class PartitionWaveform:
    """What one solver node wrote: its nets on its own time axis; ghost nets are listed so the merge
    can drop them in favour of their owner's copy. The reference's keyword forms are accepted as well:
    ``voltages=`` for ``traces=`` and ``node_mapping=`` (local name -> global name, applied to the traces)."""

    def __init__(self, partition_id: int, times: Iterable[float] = (), traces: Optional[dict] = None, ghost_nodes: Optional[set] = None, *,
                 voltages: Optional[dict] = None, node_mapping: Optional[dict] = None):
        if isinstance(times, dict) and traces is not None and not isinstance(traces, dict):
            times, traces = traces, times   # reference order: (partition_id, node_mapping, times, voltages) passed positionally
        data = traces if traces is not None else (voltages or {})
        if node_mapping:
            data = {node_mapping.get(name, name): values for name, values in data.items()}
        self.partition_id = partition_id
        self.times = times
        self.traces = data
        self.ghost_nodes = set(ghost_nodes or ())
        self.node_mapping = dict(node_mapping or {})

    @property
    def voltages(self) -> dict:
        return self.traces


class Waveform:
    """Columnar waveform: ``times`` and one array per net in ``traces``. Also constructible the reference's way, from
    ``points=[WaveformPoint(time, voltages={...}), ...]`` (with ``node_names=`` fixing the order of the nets)."""

    def __init__(self, times: Iterable[float] = (), traces: Optional[dict[str, Iterable[float]]] = None, title: str = "", *,
                 node_names: Optional[list] = None, points: Optional[list] = None):
        self.title = title
        if points is not None:
            names = list(node_names) if node_names is not None else list(dict.fromkeys(n for p in points for n in p.voltages))
            times = [p.time for p in points]
            traces = {n: [p.voltages.get(n, 0.0) for p in points] for n in names}
        as_array = lambda x: np.ascontiguousarray(x if isinstance(x, np.ndarray) else list(x), dtype=np.float64)  # noqa: E731
        self.times = as_array(times)
        self.traces: dict[str, np.ndarray] = {}
        for name, values in (traces or {}).items():
            arr = as_array(values)
            if arr.size != self.times.size:
                raise ValueError(f"trace '{name}' has {arr.size} samples for {self.times.size} time points")
            self.traces[name] = arr

    @property
    def node_names(self) -> list[str]:
        return list(self.traces)

    @property
    def num_points(self) -> int:
        return int(self.times.size)

    @property
    def num_nodes(self) -> int:
        return len(self.traces)

    @property
    def time_range(self) -> tuple[float, float]:
        return (float(self.times[0]), float(self.times[-1])) if self.times.size else (0.0, 0.0)

    @property
    def points(self) -> list[WaveformPoint]:
        return [WaveformPoint(float(t), {n: float(v[i]) for n, v in self.traces.items()}) for i, t in enumerate(self.times)]

    def voltage(self, node: str, time: float) -> Optional[float]:
        """Linear interpolation; ``None`` for an unknown net or a time outside the simulated span."""
        tr = self.traces.get(node)
        if tr is None or not self.times.size or time < self.times[0] or time > self.times[-1]:
            return None
        return float(np.interp(time, self.times, tr))

    def node_trace(self, node: str) -> list[tuple[float, float]]:
        tr = self.traces.get(node)
        return [] if tr is None else list(zip(self.times.tolist(), tr.tolist()))

    def summary(self) -> str:
        t0, t1 = self.time_range
        lines = [f"Waveform '{self.title}': {self.num_nodes} nets, {self.num_points} points, t = {t0:.3e} .. {t1:.3e} s"]
        for name in list(self.traces)[:12]:
            v = self.traces[name]
            if v.size:
                lines.append(f"  {name:<24} min {v.min():+.4f}  max {v.max():+.4f}  final {v[-1]:+.4f}")
        if self.num_nodes > 12:
            lines.append(f"  ... {self.num_nodes - 12} more")
        return "\n".join(lines)

    @classmethod
    def from_native(cls, result: dict, title: str = "") -> "Waveform":
        """From the dict the native ``simulate`` / ``simulate_partitioned`` calls return. Nets that
        appear more than once (a supply replicated into several partitions) are kept once."""
        values = np.asarray(result["values"], dtype=np.float64)
        names = result["node_names"]
        if values.ndim != 2:
            values = values.reshape(len(result["time"]), -1)
        by_net = np.ascontiguousarray(values.T)  # one transpose: each trace is then a contiguous row
        traces = {}
        for j, name in enumerate(names):
            if name not in traces and j < by_net.shape[0]:
                traces[name] = by_net[j]
        return cls(np.asarray(result["time"], dtype=np.float64), traces, title)

    @classmethod
    def from_json_file(cls, path: str) -> "Waveform":
        with open(path) as f:
            d = json.load(f)
        names = d.get("node_names", [])
        if "traces" in d and "time" in d:   # the columnar form export_json writes
            return cls(d["time"], {n: d["traces"][n] for n in names if n in d["traces"]}, d.get("title", d.get("netlist", "")))
        pts = d.get("waveform", [])
        return cls([p["time"] for p in pts], {n: [p["voltages"].get(n, 0.0) for p in pts] for n in names}, d.get("netlist", d.get("title", "")))


def merge_waveforms(parts: list[PartitionWaveform], title: str = "merged") -> Waveform:
    """Joins partition results on the first partition's time axis (others are interpolated onto it).
    A net is taken from the partition that owns it: ghost copies never override an owner's trace."""
    if not parts:
        return Waveform(title=title)
    base = np.asarray(parts[0].times, dtype=np.float64)
    traces: dict[str, np.ndarray] = {}
    for want_ghost in (False, True):
        for p in sorted(parts, key=lambda q: q.partition_id):
            t = np.asarray(p.times, dtype=np.float64)
            for name, vals in p.traces.items():
                if (name in p.ghost_nodes) != want_ghost or name in traces:
                    continue
                v = np.asarray(vals, dtype=np.float64)
                traces[name] = v if (t.size == base.size and np.array_equal(t, base)) else np.interp(base, t, v)
    return Waveform(base, traces, title)


def merge_from_json_files(paths: list[str], ghost_nodes: Optional[list[set[str]]] = None, title: str = "merged") -> Waveform:
    parts = []
    for i, path in enumerate(paths):
        w = Waveform.from_json_file(path)
        parts.append(PartitionWaveform(i, w.times.tolist(), {n: v.tolist() for n, v in w.traces.items()},
                                       set(ghost_nodes[i]) if ghost_nodes and i < len(ghost_nodes) else set()))
    return merge_waveforms(parts, title)


def export_csv(waveform: Waveform, output_path: str) -> None:
    names = waveform.node_names
    with open(output_path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["time"] + [f"V({n})" for n in names])   # the reference's column names
        cols = [waveform.traces[n] for n in names]
        for i, t in enumerate(waveform.times):
            w.writerow([repr(float(t))] + [repr(float(c[i])) for c in cols])


def export_json(waveform: Waveform, output_path: str) -> None:
    """Columnar (``time`` + ``traces``); up to 200 000 samples the reference's per-point list (``waveform``: time and a
    ``voltages`` dict per point) is written as well, so that its readers work on ordinary results. Beyond that the list
    would be many times the size of the arrays."""
    payload = {"title": waveform.title, "node_names": waveform.node_names, "num_points": waveform.num_points,
               "time": waveform.times.tolist(), "traces": {n: v.tolist() for n, v in waveform.traces.items()}}
    if waveform.num_points * max(waveform.num_nodes, 1) <= 200_000:
        payload["waveform"] = [{"time": float(t), "voltages": {n: float(v[i]) for n, v in waveform.traces.items()}} for i, t in enumerate(waveform.times)]
    with open(output_path, "w") as f:
        json.dump(payload, f)
