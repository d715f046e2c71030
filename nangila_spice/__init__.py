"""Nangila SPICE: a predictive-partitioned transient circuit simulator.

    from nangila_spice import simulate
    result = simulate("circuit.sp", partitions=4, tstop=1e-9, dt=1e-12)
    print(result.summary())

The solver core is native (``csrc/spice`` -> ``nangila_spice._native`` and the ``nangila-node``
process); its GPU part is the FP64 CSR kernel in ``libnangila_kernels.so`` (``nangila_spice.gpu``).
Public names follow ``nangila-spice/src/nangila_spice/__init__.py`` of the reference.
"""
from __future__ import annotations

from importlib import import_module
from typing import Any, Optional

__version__ = "0.2.0"

_EXPORT_MAP = {
    "parse_netlist": (".parser", "parse_netlist"), "Netlist": (".parser", "Netlist"), "Device": (".parser", "Device"),
    "Subcircuit": (".parser", "Subcircuit"),
    "build_circuit_graph": (".graph", "build_circuit_graph"), "CircuitGraph": (".graph", "CircuitGraph"),
    "partition_netlist": (".partitioner", "partition_netlist"), "partition_flat": (".partitioner", "partition_flat"),
    "Partition": (".partitioner", "Partition"), "PartitionResult": (".partitioner", "PartitionResult"),
    "Waveform": (".merger", "Waveform"), "WaveformPoint": (".merger", "WaveformPoint"), "merge_waveforms": (".merger", "merge_waveforms"),
    "export_csv": (".merger", "export_csv"), "export_json": (".merger", "export_json"),
    "discover_hardware": (".orchestrator", "discover_hardware"), "HardwareTopology": (".orchestrator", "HardwareTopology"),
    "SimulationConfig": (".orchestrator", "SimulationConfig"), "SimulationResult": (".orchestrator", "SimulationResult"),
    "run_simulation": (".orchestrator", "run_simulation"), "dc_sweep": (".orchestrator", "dc_sweep"),
    "PvtOrchestrator": (".pvt_orchestrator", "PvtOrchestrator"), "SweepConfig": (".pvt_orchestrator", "SweepConfig"),
    "SweepResult": (".pvt_orchestrator", "SweepResult"), "generate_corner_grid": (".pvt_orchestrator", "generate_corner_grid"),
    "simulate_corner": (".pvt_orchestrator", "simulate_corner"), "CornerSpec": (".pvt_orchestrator", "CornerSpec"),
    "ProcessCorner": (".pvt_orchestrator", "ProcessCorner"),
    "WaveformData": (".correctness", "WaveformData"), "WaveformComparison": (".correctness", "WaveformComparison"),
    "V1ToleranceProfile": (".correctness", "V1ToleranceProfile"), "compare_waveforms": (".correctness", "compare_waveforms"),
    "find_ngspice_binary": (".correctness", "find_ngspice_binary"), "find_nangila_binary": (".correctness", "find_nangila_binary"),
    "run_ngspice_waveform": (".correctness", "run_ngspice_waveform"), "run_nangila_waveform": (".correctness", "run_nangila_waveform"),
    "v1_tolerance_profile": (".correctness", "v1_tolerance_profile"), "within_v1_contract": (".correctness", "within_v1_contract"),
    "CorrectnessCase": (".correctness", "CorrectnessCase"), "BlockedCorrectnessCase": (".correctness", "BlockedCorrectnessCase"),
    "official_correctness_cases": (".correctness", "official_correctness_cases"),
    "phase1_automated_correctness_cases": (".correctness", "phase1_automated_correctness_cases"),
    "extended_phase1_correctness_cases": (".correctness", "extended_phase1_correctness_cases"),
    "blocked_official_correctness_cases": (".correctness", "blocked_official_correctness_cases"),
    "large_phase1_correctness_cases": (".correctness", "large_phase1_correctness_cases"),
    "huge_phase1_correctness_cases": (".correctness", "huge_phase1_correctness_cases"),
    "collect_flattened_nodes": (".correctness", "collect_flattened_nodes"), "collect_observable_nodes": (".correctness", "collect_observable_nodes"),
    "check_logic_levels": (".correctness", "check_logic_levels"), "evaluate_bench": (".benchcircuits", "evaluate_bench"),
    "read_nz": (".nz_reader", "read_nz"), "DeviceCsr": (".gpu", "DeviceCsr"),
}


def simulate(netlist_path: str, partitions: Optional[int] = None, reltol: float = 1e-3, tstop: float = 1e-6, dt: float = 1e-12,
             output_dir: Optional[str] = None, output_format: str = "csv", validate_partitioned_against_reference: bool = True,
             reference_vdd: float = 1.8, **kwargs: Any):
    """Runs a transient simulation of a SPICE deck and returns a ``SimulationResult``."""
    cfg = __getattr__("SimulationConfig")(netlist_path=netlist_path, partitions=partitions, reltol=reltol, tstop=tstop, dt=dt,
                                          output_dir=output_dir, output_format=output_format,
                                          validate_partitioned_against_reference=validate_partitioned_against_reference,
                                          reference_vdd=reference_vdd, **kwargs)
    return __getattr__("run_simulation")(cfg)


def __getattr__(name: str) -> Any:
    if name not in _EXPORT_MAP:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    module_name, attr = _EXPORT_MAP[name]
    value = getattr(import_module(module_name, __name__), attr)
    globals()[name] = value
    return value


def __dir__() -> list[str]:
    return sorted(list(globals().keys()) + list(_EXPORT_MAP.keys()))
