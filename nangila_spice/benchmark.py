"""Benchmark harness of the front end: synthetic deck generators, a scaling study over partition
counts and a report writer. API counterpart: ``nangila-spice/src/nangila_spice/benchmark.py``."""
from __future__ import annotations

import csv
import json
import os
import platform
import tempfile
import time
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class BenchmarkResult:
    name: str
    element_count: int
    node_count: int
    partition_count: int
    wall_time_secs: float
    timesteps: int
    time_per_step: float
    throughput: float  # elements * steps / second
    rollbacks: int = 0
    prediction_hit_rate: float = 0.0
    speedup: float = 1.0
    max_abs_error_vs_single: float = 0.0

    @property
    def summary_line(self) -> str:
        return (f"{self.name}: {self.element_count} elements, {self.partition_count} parts | {self.wall_time_secs:.3f}s, "
                f"{self.throughput:.0f} elem*steps/s, {self.speedup:.2f}x vs 1 partition, max err {self.max_abs_error_vs_single:.2e} V")


@dataclass
class BenchmarkSuite:
    name: str
    results: List[BenchmarkResult] = field(default_factory=list)
    timestamp: str = ""
    platform: str = ""

    def add(self, result: BenchmarkResult) -> None:
        self.results.append(result)

    def summary(self) -> str:
        lines = [f"=== Benchmark suite: {self.name} ===", f"Platform: {self.platform}", f"Timestamp: {self.timestamp}", ""]
        lines += [f"  {r.summary_line}" for r in self.results]
        if self.results:
            lines += ["", f"  Average speedup: {sum(r.speedup for r in self.results) / len(self.results):.2f}x",
                      f"  Max speedup: {max(r.speedup for r in self.results):.2f}x",
                      f"  Total elements: {sum(r.element_count for r in self.results)}"]
        return "\n".join(lines)

    def to_csv(self, path: str) -> None:
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["name", "elements", "nodes", "partitions", "wall_time_s", "timesteps", "time_per_step_s", "throughput", "rollbacks",
                        "hit_rate", "speedup", "max_abs_error_v"])
            for r in self.results:
                w.writerow([r.name, r.element_count, r.node_count, r.partition_count, f"{r.wall_time_secs:.6f}", r.timesteps,
                            f"{r.time_per_step:.9f}", f"{r.throughput:.0f}", r.rollbacks, f"{r.prediction_hit_rate:.4f}", f"{r.speedup:.3f}",
                            f"{r.max_abs_error_vs_single:.3e}"])

    def to_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"suite": self.name, "platform": self.platform, "timestamp": self.timestamp,
                       "results": [r.__dict__ for r in self.results]}, f, indent=2)


def generate_cim_netlist(n_rows: int, n_cols: int) -> str:
    """Compute-in-memory crossbar deck: word-line drivers, a resistor per cell, bit-line capacitors."""
    lines = [f"* CiM array {n_rows}x{n_cols}"]
    for r in range(n_rows):
        lines.append(f"VWL{r} wl{r} 0 DC {1.8 if r == 0 else 0.0}")
    for r in range(n_rows):
        for c in range(n_cols):
            lines.append(f"RC{r}_{c} wl{r} bl{c} {'1meg' if (r + c) % 3 == 0 else '10k'}")
    for c in range(n_cols):
        lines.append(f"CBL{c} bl{c} 0 100f")
    lines += [".ic " + " ".join(f"V(bl{c})=0" for c in range(n_cols)), ".end"]
    return "\n".join(lines) + "\n"


def generate_rc_ladder_netlist(n_stages: int, r: float = 1e3, c: float = 1e-12) -> str:
    lines = [f"* RC ladder, {n_stages} stages", "VIN n0 0 PULSE(0 1.8 0 10p 10p 1n 2n)"]
    for i in range(n_stages):
        lines.append(f"R{i} n{i} n{i + 1} {r!r}")
        lines.append(f"C{i} n{i + 1} 0 {c!r}")
    lines.append(".end")
    return "\n".join(lines) + "\n"


def run_scaling_study(netlist_text, name=None, partition_counts: Optional[List[int]] = None, tstop: float = 200e-12, dt: float = 1e-12,
                      method: str = "auto", *, label: Optional[str] = None) -> BenchmarkSuite:
    """The same deck at several partition counts; errors are against the single-matrix run.

    Also the reference's form, ``run_scaling_study(circuit_generator, sizes, partition_counts, label="Scaling Study")``
    (benchmark.py:175-219, where the figures are estimates): every size the generator is called with is simulated at
    every partition count, and the results of all sizes come back in one suite."""
    if callable(netlist_text):
        generator, sizes = netlist_text, list(name or [])
        title = label or "Scaling Study"
        suite = BenchmarkSuite(name=title, timestamp=time.strftime("%Y-%m-%d %H:%M:%S"), platform=f"{platform.system()} {platform.machine()}")
        for size in sizes:
            one = run_scaling_study(generator(size), f"{title.replace(' ', '_')}_{size}", partition_counts, tstop, dt, method)
            for r in one.results:
                suite.add(r)
        return suite
    import numpy as np

    from .orchestrator import SimulationConfig, run_simulation

    name = name or label or "scaling"
    suite = BenchmarkSuite(name=name, timestamp=time.strftime("%Y-%m-%d %H:%M:%S"), platform=f"{platform.system()} {platform.machine()}")
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, f"{name}.sp")
        with open(path, "w") as f:
            f.write(netlist_text)
        base_time = None
        for k in partition_counts or [1, 2, 4]:
            res = run_simulation(SimulationConfig(netlist_path=path, partitions=k, tstop=tstop, dt=dt, method=method))
            if not res.success:
                raise RuntimeError(f"{name} with {k} partitions failed: {res.error}")
            stats = res.solver_stats.get("stats", {})
            steps = int(stats.get("total_steps", stats.get("steps", round(tstop / dt))))
            # solve time only: the validation run of partitioned cases is not part of the measurement
            wall = float(stats.get("wall_time_secs", res.wall_time_secs))
            if base_time is None:
                base_time = wall
            elements = sum(p.num_devices for p in res.partition_result.partitions) if k > 1 else res.partition_result.partitions[0].num_devices
            hits, misses = stats.get("prediction_hits", 0), stats.get("prediction_misses", 0)
            suite.add(BenchmarkResult(name=f"{name}_k{len(res.partition_result.partitions)}", element_count=elements,
                                      node_count=res.waveform.num_nodes, partition_count=len(res.partition_result.partitions),
                                      wall_time_secs=wall, timesteps=steps, time_per_step=wall / max(steps, 1),
                                      throughput=elements * steps / max(wall, 1e-12), rollbacks=int(stats.get("resolves", stats.get("rollbacks", 0))),
                                      prediction_hit_rate=hits / (hits + misses) if hits + misses else 1.0, speedup=base_time / max(wall, 1e-12),
                                      max_abs_error_vs_single=res.reference_comparison.max_abs_error if res.reference_comparison else 0.0))
    del np
    return suite


def generate_performance_report(suite: BenchmarkSuite, output_dir: str) -> str:
    os.makedirs(output_dir, exist_ok=True)
    suite.to_csv(os.path.join(output_dir, f"{suite.name}.csv"))
    suite.to_json(os.path.join(output_dir, f"{suite.name}.json"))
    path = os.path.join(output_dir, f"{suite.name}.md")
    with open(path, "w") as f:
        f.write(f"# {suite.name}\n\n{suite.platform}, {suite.timestamp}\n\n| case | elements | partitions | wall s | steps | speedup | max err V |\n|---|---|---|---|---|---|---|\n")
        for r in suite.results:
            f.write(f"| {r.name} | {r.element_count} | {r.partition_count} | {r.wall_time_secs:.4f} | {r.timesteps} | {r.speedup:.2f} | {r.max_abs_error_vs_single:.2e} |\n")
    return path
