"""Experimental APIs that are not part of the Nangila v0.1 support contract
(reference: python/nangila/experimental.py:1-32)."""
import warnings

warnings.warn(
    "nangila.experimental exposes beta and unstable APIs that are excluded from the v0.1 "
    "support contract.",
    stacklevel=2,
)

from .fsdp import NangilaFSDPState, nangila_fsdp_hook  # noqa: E402


def _raw():
    try:
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        from . import _cuda

        return _cuda
    except Exception as exc:
        raise RuntimeError("CUDA not compiled. Rebuild with CUDA support.") from exc


def _check_sync_mode(sync_mode):
    if sync_mode not in (0, 1, 2):
        raise ValueError(f"Invalid sync_mode {sync_mode}. Use SyncMode.ASYNC (0), ALWAYS (1), or PERIODIC (2)")


_calls = 0


def _maybe_sync(glue, stream_ptr, sync_mode):
    global _calls
    _calls += 1
    if sync_mode == 1 or (sync_mode == 2 and _calls % 100 == 0):
        err = glue.stream_synchronize(stream_ptr)
        if err != 0:
            raise RuntimeError(f"CUDA error after kernel: {glue.error_string(err)}")


def cuda_predict_and_quantize(gradient_ptr, g_current_ptr, g_previous_ptr, momentum, gamma, output_ptr, n,
                              stream_ptr=0, sync_mode=2, step=0, layer_id=0):
    """Raw launch: INT4-quantize ``gradient - (g_t + momentum (g_t - g_{t-1}))`` with one scale ``gamma``.
    Arguments are device addresses (``tensor.data_ptr()``) of FP32 buffers of ``n`` elements and a
    ``ceil(n/2)``-byte output (reference: nangila-hook/src/python.rs:592-647)."""
    _check_sync_mode(sync_mode)
    glue = _raw()
    err = glue.raw_predict_and_quantize(gradient_ptr, g_current_ptr, g_previous_ptr, float(momentum), float(gamma),
                                        output_ptr, int(n), stream_ptr, int(step), int(layer_id))
    if err != 0:
        raise RuntimeError(f"predict_and_quantize failed: {glue.error_string(err)}")
    _maybe_sync(glue, stream_ptr, sync_mode)


def cuda_dequantize_and_reconstruct(packed_ptr, g_current_ptr, g_previous_ptr, momentum, gamma, output_ptr, n,
                                    stream_ptr=0, sync_mode=2):
    """Raw launch: ``out = g_t + momentum (g_t - g_{t-1}) + q * gamma`` (python.rs:664-751)."""
    _check_sync_mode(sync_mode)
    glue = _raw()
    err = glue.raw_dequantize_and_reconstruct(packed_ptr, g_current_ptr, g_previous_ptr, float(momentum), float(gamma),
                                              output_ptr, int(n), stream_ptr)
    if err != 0:
        raise RuntimeError(f"dequantize_and_reconstruct failed: {glue.error_string(err)}")
    _maybe_sync(glue, stream_ptr, sync_mode)


__all__ = ["NangilaFSDPState", "nangila_fsdp_hook", "cuda_predict_and_quantize", "cuda_dequantize_and_reconstruct"]
