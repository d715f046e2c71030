"""Nangila: prediction-residual gradient compression for PyTorch distributed training, built for
NVIDIA B200 (sm_100a).

The public surface matches the reference package (python/nangila/__init__.py:9-45):
``NangilaConfig, NangilaHook, Sculptor, SyncMode, CompressorType, cuda_available, __version__,
NangilaDDPHook, NangilaCppHook, CPP_HOOK_AVAILABLE, register_nangila_hook`` and the lazily imported
``experimental`` sub-module. The classes come from the C++ core (``nangila._C``); the device kernels
are reached through ``nangila._cuda`` and the engines in ``nangila.parallel``.
"""
import importlib

try:
    from ._C import (  # noqa: F401
        CompressorType,
        NangilaConfig,
        NangilaHook,
        Sculptor,
        SyncMode,
        __version__,
    )
except ImportError:  # the extension is built in-tree on first use
    from . import _build as _nb

    _nb.build_core()
    from ._C import (  # noqa: F401
        CompressorType,
        NangilaConfig,
        NangilaHook,
        Sculptor,
        SyncMode,
        __version__,
    )


def cuda_available() -> bool:
    """True when the compiled sm_100a kernels are loadable and a CUDA device is visible
    (reference: nangila-hook/src/python.rs:560-570)."""
    try:
        import torch

        if not torch.cuda.is_available():
            return False
        from . import _cuda  # noqa: F401

        return True
    except Exception:
        return False


from .ddp import CPP_HOOK_AVAILABLE, NangilaCppHook, NangilaDDPHook, register_nangila_hook  # noqa: E402
from . import gpu_methods as _gpu_methods  # noqa: E402

_gpu_methods.install()  # NangilaHook.compress_gpu / decompress_gpu / update_gpu


def __getattr__(name):
    if name == "experimental":
        return importlib.import_module(".experimental", __name__)
    raise AttributeError(f"module 'nangila' has no attribute {name!r}")


__all__ = [
    "NangilaConfig",
    "NangilaHook",
    "Sculptor",
    "SyncMode",
    "CompressorType",
    "cuda_available",
    "__version__",
    "NangilaDDPHook",
    "NangilaCppHook",
    "CPP_HOOK_AVAILABLE",
    "register_nangila_hook",
    "experimental",
]
