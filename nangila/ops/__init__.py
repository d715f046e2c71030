"""Device operations of the framework as plain functions over torch tensors.

Each function is a thin wrapper over one hand-written sm_100a kernel (``nangila._cuda``); the fused
exchange kernels are driven through the engines in ``nangila.parallel`` instead.
"""
from .reductions import absmax_percentile, crc32, quantizer_gamma, state_hash  # noqa: F401
from .sculptor_stats import DeviceSculptor  # noqa: F401
