"""Process / voltage / temperature sweeps over a deck.

The golden corner is simulated once; corners close to it are derived with the first-order delta
model of the native core (``csrc/spice/pvt.hpp``), the others are really simulated. Native calls
release the interpreter lock, so the corners run in a thread pool.

API counterpart: ``nangila-spice/src/nangila_spice/pvt_orchestrator.py:31-476`` of the reference
(whose speed-up figure divides an assumed 10 ms per full simulation by the sweep time; here the
full-simulation time is the measured time of the golden run).
"""
from __future__ import annotations

import itertools
import json
import os
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import List, Optional

import numpy as np


class ProcessCorner(Enum):
    TT = "TT"
    FF = "FF"
    SS = "SS"
    FS = "FS"
    SF = "SF"

    @property
    def mobility_factor(self) -> float:
        return {"TT": 1.0, "FF": 1.15, "SS": 0.85, "FS": 1.1, "SF": 0.9}[self.value]

    @property
    def is_nominal(self) -> bool:
        return self is ProcessCorner.TT


@dataclass
class CornerSpec:
    process: ProcessCorner
    vdd: float
    temperature: float
    name: str = ""

    def __post_init__(self):
        if not self.name:
            self.name = f"{self.process.value}_{self.vdd:.2f}V_{self.temperature:.0f}C"

    @classmethod
    def nominal(cls) -> "CornerSpec":
        return cls(ProcessCorner.TT, 1.8, 27.0, "TT_1V8_27C")

    @property
    def is_nominal(self) -> bool:
        return self.process == ProcessCorner.TT and abs(self.vdd - 1.8) < 0.01 and abs(self.temperature - 27.0) < 0.1

    @property
    def thermal_voltage(self) -> float:
        return 8.617e-5 * (self.temperature + 273.15)

    def delta_params(self, reference: "CornerSpec") -> dict:
        return {"delta_vdd": self.vdd - reference.vdd, "delta_temp": self.temperature - reference.temperature,
                "mobility_factor": self.process.mobility_factor / reference.process.mobility_factor}

    def is_linearisable(self, reference: "CornerSpec") -> bool:
        d = self.delta_params(reference)
        return abs(d["delta_vdd"]) < 0.3 and abs(d["delta_temp"]) < 50.0 and abs(d["mobility_factor"] - 1.0) < 0.2


def generate_corner_grid(process_corners: Optional[List[ProcessCorner]] = None, vdd_values: Optional[List[float]] = None,
                         temp_values: Optional[List[float]] = None) -> List[CornerSpec]:
    """Default grid: 5 process corners x 5 supplies (+-10 % of 1.8 V) x 8 temperatures = 200 corners."""
    process_corners = process_corners or list(ProcessCorner)
    vdd_values = vdd_values or [1.62, 1.71, 1.80, 1.89, 1.98]
    temp_values = temp_values or [-40.0, -10.0, 0.0, 27.0, 55.0, 85.0, 105.0, 125.0]
    return [CornerSpec(p, v, t) for p, v, t in itertools.product(process_corners, vdd_values, temp_values)]


def generate_1000_corner_grid() -> List[CornerSpec]:
    """5 x 10 x 20 = 1000 corners."""
    return generate_corner_grid(list(ProcessCorner), list(np.linspace(1.62, 1.98, 10)), list(np.linspace(-40.0, 125.0, 20)))


_RC_DECK = """* golden RC stage
V1 vdd 0 DC 1.8
R1 vdd out 1k
C1 out 0 10f
.ic V(out)=0
.end
"""


def _by_net(names, values) -> dict:
    """``{net: samples}`` view of a (points x nets) array (empty when no waveform was asked for)."""
    if values is None:
        return {}
    arr = np.asarray(values, dtype=np.float64)
    return {n: arr[:, j] for j, n in enumerate(names) if arr.ndim == 2 and j < arr.shape[1]}


def simulate_corner(corner: CornerSpec, golden_waveform: Optional[dict] = None, use_delta: bool = True, netlist_path: Optional[str] = None,
                    tstop: float = 200e-12, dt: float = 1e-12, want_waveform: bool = True) -> dict:
    """One corner: a delta reconstruction from ``golden_waveform`` when allowed and close enough,
    else a full simulation of the deck (a built-in RC stage when no deck is given). The golden run is handed to
    the native delta solver once and kept in ``golden_waveform["_solver"]``."""
    from . import _native

    t0 = time.perf_counter()
    nominal = CornerSpec.nominal()
    if use_delta and golden_waveform is not None and corner.is_linearisable(nominal):
        solver = golden_waveform.get("_solver")
        if solver is None:
            solver = _native.PvtDeltaSolver(list(golden_waveform["time"]), np.asarray(golden_waveform["values"], dtype=np.float64))
            golden_waveform["_solver"] = solver
        r = solver.solve(corner.process.value, corner.vdd, corner.temperature, want_waveform)
        # "corner_name", "experimental", "execution_mode" and "waveforms" are the reference's keys (its corners are synthetic and all
        # marked experimental); here only the delta model is an approximation, the rest is the solver
        values = r.get("waveform")
        return {"corner": corner.name, "corner_name": corner.name, "used_delta": bool(r["used_delta_mode"]), "peak_delta_v": float(r["peak_delta_v"]),
                "time": golden_waveform["time"], "values": values, "node_names": golden_waveform["node_names"],
                "waveforms": _by_net(golden_waveform["node_names"], values), "experimental": True, "execution_mode": "experimental_delta",
                "wall_time": time.perf_counter() - t0}
    text = Path(netlist_path).read_text() if netlist_path else _RC_DECK
    js, _ = _native.parse_spice(text, Path(netlist_path).name if netlist_path else "rc_stage", corner.process.value, corner.vdd, corner.temperature)
    r = _native.simulate(js, tstop, dt)
    peak = 0.0
    if golden_waveform is not None:
        a, b = np.asarray(r["values"], float), np.asarray(golden_waveform["values"], float)
        if a.shape == b.shape and a.size:
            peak = float(np.abs(a - b).max())
    return {"corner": corner.name, "corner_name": corner.name, "used_delta": False, "peak_delta_v": peak, "time": r["time"], "values": r["values"],
            "node_names": r["node_names"], "waveforms": _by_net(r["node_names"], r["values"]), "experimental": False, "execution_mode": "solver",
            "wall_time": time.perf_counter() - t0, "completed": bool(r["stats"]["completed"])}


@dataclass
class SweepConfig:
    max_workers: int = 8
    delta_mode: bool = True
    tolerance_v: float = 1e-3
    output_dir: str = "/tmp/nangila_pvt"
    save_waveforms: bool = False
    tstop: float = 200e-12
    dt: float = 1e-12


@dataclass
class SweepResult:
    total_corners: int = 0
    completed: int = 0
    failed: int = 0
    delta_mode_used: int = 0
    full_sim_used: int = 0
    total_wall_time: float = 0.0
    peak_delta_v: float = 0.0
    speedup_vs_full: float = 1.0
    corner_results: List[dict] = field(default_factory=list)

    @property
    def success_rate(self) -> float:
        return self.completed / self.total_corners if self.total_corners else 0.0

    @property
    def avg_time_per_corner(self) -> float:
        return self.total_wall_time / self.completed if self.completed else 0.0

    def summary(self) -> str:
        return (f"PVT sweep: {self.completed}/{self.total_corners} corners | {self.total_wall_time:.2f}s total | "
                f"{self.avg_time_per_corner * 1000:.2f}ms/corner | speedup {self.speedup_vs_full:.1f}x vs full simulation of every corner | "
                f"peak dV={self.peak_delta_v * 1e3:.3f}mV | delta mode: {self.delta_mode_used}/{self.completed}")

    def to_json(self, path: str) -> None:
        data = {"summary": self.summary(), "total_corners": self.total_corners, "completed": self.completed, "failed": self.failed,
                "delta_mode_used": self.delta_mode_used, "full_sim_used": self.full_sim_used, "total_wall_time": self.total_wall_time,
                "peak_delta_v_v": self.peak_delta_v, "speedup_vs_full": self.speedup_vs_full,
                "avg_time_per_corner_ms": self.avg_time_per_corner * 1000}
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        with open(path, "w") as f:
            json.dump(data, f, indent=2)


class PvtOrchestrator:
    """Golden corner first, then every other corner in parallel."""

    def __init__(self, config: Optional[SweepConfig] = None):
        self.config = config or SweepConfig()
        self.golden_waveform: Optional[dict] = None

    def run_sweep(self, corners: List[CornerSpec], netlist_path: Optional[str] = None) -> SweepResult:
        cfg = self.config
        corners = list(corners)
        if not any(c.is_nominal for c in corners):
            corners = [CornerSpec.nominal()] + corners
        result = SweepResult(total_corners=len(corners))
        t0 = time.perf_counter()
        golden = simulate_corner(CornerSpec.nominal(), None, False, netlist_path, cfg.tstop, cfg.dt)
        golden_time = golden["wall_time"]
        self.golden_waveform = golden
        result.corner_results.append(self._strip(golden))
        result.completed += 1
        result.full_sim_used += 1
        rest = [c for c in corners if not c.is_nominal]

        def one(c: CornerSpec) -> dict:
            return simulate_corner(c, self.golden_waveform, cfg.delta_mode, netlist_path, cfg.tstop, cfg.dt, want_waveform=cfg.save_waveforms)

        with ThreadPoolExecutor(max_workers=max(1, cfg.max_workers)) as ex:
            futures = [ex.submit(one, c) for c in rest]
            for fut in futures:
                try:
                    res = fut.result()
                except Exception:
                    result.failed += 1
                    continue
                result.completed += 1
                result.peak_delta_v = max(result.peak_delta_v, res["peak_delta_v"])
                if res["used_delta"]:
                    result.delta_mode_used += 1
                else:
                    result.full_sim_used += 1
                result.corner_results.append(self._strip(res))
        result.total_wall_time = time.perf_counter() - t0
        result.speedup_vs_full = result.total_corners * golden_time / max(result.total_wall_time, 1e-9)
        if cfg.save_waveforms:
            result.to_json(os.path.join(cfg.output_dir, "sweep.json"))
        return result

    def _strip(self, res: dict) -> dict:
        if self.config.save_waveforms:
            return {k: v for k, v in res.items() if k != "_solver"}
        return {k: v for k, v in res.items() if k not in ("time", "values", "waveforms", "_solver")}
