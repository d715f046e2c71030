"""Simulation front end: hardware discovery, partition-count choice, running the solver (one
process per partition file, or every partition inside one process), merging and validation.

API counterpart: ``nangila-spice/src/nangila_spice/orchestrator.py:47-688`` of the reference. There a
partitioned request falls back to the single-node solver by default because independent solver
processes cannot exchange boundary values; here partitions exchange boundary voltages every step
(``mode="in_process"``, the default for more than one partition), and the merged result is checked
against a single-matrix run of the same deck when ``validate_partitioned_against_reference`` is set.
``mode="processes"`` keeps the process-per-partition launch for decks whose partitions do not
interact (or for ghost-free debugging) and reports the result as experimental.
"""
from __future__ import annotations

import json
import os
import platform
import re
import shutil
import socket
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

from .correctness import WaveformComparison, compare_waveforms, find_nangila_binary, waveform_to_data, within_v1_contract
from .merger import PartitionWaveform, Waveform, export_csv, export_json, merge_waveforms
from .parser import Netlist, parse_netlist
from .partitioner import PartitionResult, partition_netlist


@dataclass
class HardwareTopology:
    cpu_count: int
    numa_nodes: int
    total_ram_gb: float
    gpu_count: int
    hostname: str
    os_name: str

    def summary(self) -> str:
        return (f"{self.cpu_count} cores, {self.total_ram_gb:.1f}GB RAM, {self.numa_nodes} NUMA nodes, {self.gpu_count} GPUs, "
                f"{self.hostname} ({self.os_name})")


@dataclass
class SimulationConfig:
    netlist_path: str
    partitions: Optional[int] = None
    method: str = "auto"
    reltol: float = 1e-3
    tstop: float = 1e-6
    dt: float = 1e-12
    predict_depth: int = 5
    output_dir: Optional[str] = None
    output_format: str = "csv"
    validate_partitioned_against_reference: bool = True
    reference_vdd: float = 1.8
    prefer_single_node_fallback_for_partitioned: bool = False
    verbose: bool = False
    mode: str = "auto"  # 'auto' | 'in_process' | 'processes' (one nangila-node per partition, boundary values over TCP)
    adaptive: bool = False  # single-matrix runs: variable internal step, waveform still on the dt grid
    speculate: bool = True  # partitions run windows of steps ahead on predictions between exchanges (False: one step per exchange)
    io_timeout_secs: float = 30.0  # processes mode: how long a process waits for a peer before it gives up
    process: str = "TT"
    vdd: float = 1.8
    temp: float = 27.0
    solver: str = "lu"
    record_every: int = 1
    record_nodes: Optional[list] = None  # single-matrix runs: the waveform keeps these nets only (names compared without case)
    threads: Optional[int] = None  # worker threads of the in-process partitioned run (default: one per partition, at most the core count)


@dataclass
class SimulationResult:
    waveform: Waveform
    partition_result: PartitionResult
    hardware: HardwareTopology
    wall_time_secs: float
    per_partition_times: list[float] = field(default_factory=list)
    success: bool = True
    error: Optional[str] = None
    experimental: bool = False
    validation_status: str = "validated_single_node"
    warnings: list[str] = field(default_factory=list)
    reference_comparison: Optional[WaveformComparison] = None
    solver_stats: dict = field(default_factory=dict)

    def summary(self) -> str:
        status = "SUCCESS" if self.success else "FAILED"
        if self.experimental:
            status += " (EXPERIMENTAL)"
        lines = ["=== Nangila SPICE Simulation Results ===", f"Status: {status}", f"Validation: {self.validation_status}",
                 f"Wall time: {self.wall_time_secs:.3f}s", f"Hardware: {self.hardware.summary()}",
                 f"Partitions: {len(self.partition_result.partitions)} ({self.partition_result.method})",
                 f"Ghost nodes: {self.partition_result.total_boundary_nodes}", "", self.waveform.summary()]
        if self.reference_comparison is not None:
            c = self.reference_comparison
            lines.append(f"vs single matrix: max {c.max_abs_error:.3e} V, rms {c.rms_error:.3e} V over {len(c.shared_nodes)} nets")
        lines += [f"warning: {w}" for w in self.warnings]
        if self.error:
            lines.append(f"error: {self.error}")
        return "\n".join(lines)


def discover_hardware() -> HardwareTopology:
    cpus = os.cpu_count() or 1
    ram = 0.0
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemTotal:"):
                    ram = float(line.split()[1]) / 1024 / 1024
                    break
    except OSError:
        pass
    numa = 1
    try:
        numa = max(1, len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node")]))
    except OSError:
        pass
    # GPUs are counted from the driver's device nodes: importing torch for this costs seconds per process
    gpus = 0
    try:
        torch = sys.modules.get("torch")
        if torch is not None:
            gpus = torch.cuda.device_count() if torch.cuda.is_available() else 0
        else:
            gpus = len([d for d in os.listdir("/dev") if re.fullmatch(r"nvidia\d+", d)])
    except Exception:
        pass
    return HardwareTopology(cpus, numa, ram, gpus, socket.gethostname(), platform.system())


def auto_partition_count(hw: HardwareTopology, num_devices: int) -> int:
    """One partition per ~500 devices, at most one per core, at least one."""
    return max(1, min(hw.cpu_count, num_devices // 500))


def _is_nonlinear_netlist(netlist: Netlist) -> bool:
    return any(d.dev_type in ("M", "D", "Q", "J") for d in netlist.flatten().devices)


def _log(config: SimulationConfig, msg: str) -> None:
    if config.verbose:
        print(f"[nangila] {msg}")


def _single_run(config: SimulationConfig, flat: dict, adaptive: bool = False) -> tuple[Waveform, dict]:
    from . import _native

    if config.solver == "cuda":
        from .gpu import enable_device_solver

        enable_device_solver()
    r = _native.simulate(json.dumps(flat), config.tstop, config.dt, config.reltol, config.solver, config.record_every, config.predict_depth,
                         adaptive=adaptive, record_nodes=list(config.record_nodes or []))
    return Waveform.from_native(r, title=flat.get("name", "")), {"stats": r["stats"], "newton": r["newton"]}


def _run_processes(config: SimulationConfig, pr: PartitionResult, workdir: str) -> tuple[Waveform, list[float], dict]:
    """One ``nangila-node`` process per partition. The processes find each other through a rendezvous directory,
    advance in lockstep and exchange boundary voltages over TCP every sweep; each writes the nets it owns."""
    exe = find_nangila_binary()
    if exe is None:
        raise FileNotFoundError("nangila-node is not built: run `python -m nangila._build --spice`")
    k = len(pr.partitions)
    rendezvous = os.path.join(workdir, "rendezvous")
    os.makedirs(rendezvous, exist_ok=True)
    for name in os.listdir(rendezvous):  # addresses of an earlier run in the same directory would mislead the new processes
        if name.endswith(".addr"):
            os.unlink(os.path.join(rendezvous, name))
    procs, outs = [], []
    t0 = time.perf_counter()
    for part in pr.partitions:
        pfile = os.path.join(workdir, f"partition_{part.partition_id}.json")
        out = os.path.join(workdir, f"waveform_{part.partition_id}.json")
        Path(pfile).write_text(json.dumps(part.netlist))
        outs.append(out)
        cmd = [exe, "--partition", pfile, "--node-id", str(part.partition_id), "-k", str(k), "--tstop", repr(config.tstop), "--dt", repr(config.dt),
               "--reltol", repr(config.reltol), "--predict-depth", str(config.predict_depth), "--record-every", str(config.record_every),
               "--waveform-json", out, "--io-timeout-ms", str(int(config.io_timeout_secs * 1000)),
               "--connect-timeout-ms", str(int(config.io_timeout_secs * 1000))]
        if k > 1:
            cmd += ["--rendezvous", rendezvous] + ([] if config.speculate else ["--lockstep"])
        procs.append(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    logs, times = [], []
    for proc in procs:
        _, err = proc.communicate()
        logs.append(err)
        times.append(time.perf_counter() - t0)
    bad = [(i, p.returncode) for i, p in enumerate(procs) if p.returncode != 0]
    if bad:
        i, rc = bad[0]
        tail = logs[i].strip().splitlines()[-1] if logs[i].strip() else ""
        raise RuntimeError(f"partition {i}: nangila-node exit {rc}: {tail[-300:]}")
    waves = []
    for part, out in zip(pr.partitions, outs):
        w = Waveform.from_json_file(out)
        waves.append(PartitionWaveform(part.partition_id, w.times.tolist(), {n: v.tolist() for n, v in w.traces.items()}, set()))
    stats = {"completed": True, "processes": k, "log_tail": [lg.strip().splitlines()[-1] if lg.strip() else "" for lg in logs]}
    return merge_waveforms(waves, title=Path(config.netlist_path).name), times, stats


def run_simulation(config: SimulationConfig) -> SimulationResult:
    """Parse, partition, solve, merge, validate, export."""
    from . import _native

    t_start = time.perf_counter()
    hw = discover_hardware()
    netlist = parse_netlist(config.netlist_path)
    k = config.partitions if config.partitions else auto_partition_count(hw, netlist.flatten().num_devices)
    nonlinear = _is_nonlinear_netlist(netlist)
    flat = netlist.to_native(config.process, config.vdd, config.temp)
    warnings = [f"parser: {w}" for w in flat.pop("warnings", [])]
    pr = partition_netlist(netlist, k, config.method, process=config.process, vdd=config.vdd, temp=config.temp)
    k = len(pr.partitions)
    _log(config, f"{flat['num_nodes']} nets, {len(flat['elements'])} elements, {k} partition(s)")
    result = SimulationResult(Waveform(), pr, hw, 0.0)
    result.warnings = warnings
    try:
        if k == 1 or config.prefer_single_node_fallback_for_partitioned:
            result.waveform, result.solver_stats = _single_run(config, flat, adaptive=config.adaptive)
            result.validation_status = "validated_single_node" if k == 1 else "single_node_fallback"
            if k > 1:
                result.warnings.append("partitioned request served by the single-matrix solver (prefer_single_node_fallback_for_partitioned)")
            result.success = bool(result.solver_stats["stats"]["completed"])
        else:
            mode = "in_process" if config.mode == "auto" else config.mode
            if mode == "in_process":
                threads = config.threads or max(1, min(k, hw.cpu_count))
                r = _native.simulate_partitioned(pr.partition_files(), config.tstop, config.dt, config.reltol, config.predict_depth, True,
                                                 config.record_every, threads, config.speculate)
                result.waveform = Waveform.from_native(r, title=Path(config.netlist_path).name)
                result.solver_stats = {"stats": r["stats"]}
                result.success = bool(r["stats"]["completed"])
                if r["stats"]["unconverged_steps"]:
                    result.warnings.append(f"{r['stats']['unconverged_steps']} steps hit the relaxation sweep limit")
            elif mode == "processes":
                with tempfile.TemporaryDirectory() as tmp:
                    result.waveform, result.per_partition_times, pstats = _run_processes(config, pr, config.output_dir or tmp)
                result.solver_stats = {"stats": pstats}
                result.success = True
            else:
                raise ValueError(f"unknown mode '{config.mode}'")
            result.validation_status = "partitioned_unvalidated"
            if config.validate_partitioned_against_reference:
                ref, _ = _single_run(config, flat)
                cmp_ = compare_waveforms(waveform_to_data(ref, "single"), waveform_to_data(result.waveform, "partitioned"), vdd=config.reference_vdd)
                result.reference_comparison = cmp_
                ok, profile = within_v1_contract(cmp_, nonlinear=nonlinear, vdd=config.reference_vdd)
                result.validation_status = "partitioned_validated" if ok else "partitioned_outside_contract"
                if not ok:
                    result.warnings.append(f"partitioned result differs from the single-matrix run by {cmp_.max_abs_error:.3e} V "
                                           f"(contract {profile.max_abs_tol:.1e} V); returning the single-matrix waveform")
                    result.waveform = ref
    except Exception as e:  # surfaced in the result, as the reference's front end does
        result.success = False
        result.error = f"{type(e).__name__}: {e}"
    result.wall_time_secs = time.perf_counter() - t_start
    if config.output_dir and result.success:
        os.makedirs(config.output_dir, exist_ok=True)
        stem = Path(config.netlist_path).stem
        # <deck name>.<format>, and the same file under the name the reference uses (waveform.<format>)
        ext = "json" if config.output_format == "json" else "csv"
        target = os.path.join(config.output_dir, f"{stem}.{ext}")
        (export_json if ext == "json" else export_csv)(result.waveform, target)
        alias = os.path.join(config.output_dir, f"waveform.{ext}")
        if os.path.abspath(alias) != os.path.abspath(target):
            shutil.copyfile(target, alias)
    return result


def dc_sweep(netlist_path: str, source_node: str, start: float, stop: float, step: float, process: str = "TT", vdd: float = 1.8,
             temp: float = 27.0) -> Waveform:
    """DC transfer curves: the voltage source that holds ``source_node`` (against ground) goes from ``start`` to ``stop``
    in steps of ``step``; every point is an operating point found from the previous one. The result is a ``Waveform``
    whose ``times`` are the swept voltages, so ``voltage()``, ``summary()`` and the exporters work on it; points where
    Newton did not converge hold NaN. The reference has no DC analysis."""
    import numpy as np

    from . import _native
    from .parser import parse_netlist

    if step == 0 or (stop - start) * step < 0:
        raise ValueError("step must be non-zero and point from start to stop")
    count = int(np.floor((stop - start) / step + 1e-9)) + 1
    values = [start + i * step for i in range(count)]
    flat = parse_netlist(netlist_path).to_native(process, vdd, temp)
    flat.pop("warnings", None)
    r = _native.dc_sweep(json.dumps(flat), source_node, values)
    vals = np.asarray(r["values"], dtype=np.float64)
    traces = {name: vals[:, j] for j, name in enumerate(r["node_names"]) if j < vals.shape[1]}
    return Waveform(np.asarray(values, dtype=np.float64), traces, f"dc sweep of {source_node}")
