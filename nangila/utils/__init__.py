"""Helpers shared by the benchmarks, examples and tests (no kernels here)."""
from .benchmarking import ClockSampler, timed_steps
from .distributed import init_distributed, local_device, seed_everything

__all__ = ["ClockSampler", "timed_steps", "init_distributed", "local_device", "seed_everything"]
