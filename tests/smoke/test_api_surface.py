"""API-surface smoke tests, the same checks as the reference's default pytest tier
(tests/smoke/test_simple_compression.py, tests/smoke/test_cuda_error_handling.py)."""
import warnings

import numpy as np
import pytest

import nangila
from nangila import NangilaConfig, NangilaHook, SyncMode


def test_config_kwargs_and_syncmode_ints():
    cfg = NangilaConfig(momentum=0.9, threshold=0.95, warmup_steps=10, shadow_run_steps=5, quantize_bits=4)
    assert cfg.warmup_steps == 10 and cfg.shadow_run_steps == 5
    assert SyncMode.ASYNC == 0 and SyncMode.ALWAYS == 1 and SyncMode.PERIODIC == 2


def test_syncmode_constructor_and_repr():
    for v, name in ((0, "ASYNC"), (1, "ALWAYS"), (2, "PERIODIC")):
        m = SyncMode(v)
        assert repr(m) == f"SyncMode.{name}" and int(m) == v and m == v
    with pytest.raises(ValueError):
        SyncMode(99)
    with pytest.raises(ValueError):
        SyncMode(-1)


def test_cuda_functions_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    assert nangila.cuda_available() is False
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ex = nangila.experimental
    with pytest.raises(RuntimeError, match="CUDA not compiled"):
        ex.cuda_predict_and_quantize(0, 0, 0, 0.9, 0.1, 0, 16)
    with pytest.raises(RuntimeError, match="CUDA not compiled"):
        ex.cuda_dequantize_and_reconstruct(0, 0, 0, 0.9, 0.1, 0, 16)


def test_invalid_sync_mode_is_rejected_everywhere():
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ex = nangila.experimental
    with pytest.raises(ValueError, match="Invalid sync_mode"):
        ex.cuda_predict_and_quantize(0, 0, 0, 0.9, 0.1, 0, 16, sync_mode=3)
    from nangila.ddp import _validate_sync_mode

    with pytest.raises(ValueError, match="Invalid sync_mode"):
        _validate_sync_mode(7)
    assert _validate_sync_mode(SyncMode(1)) == 1


def test_experimental_import_warns():
    import importlib
    import sys

    sys.modules.pop("nangila.experimental", None)
    with pytest.warns(UserWarning, match="excluded from the v0.1"):
        importlib.import_module("nangila.experimental")


def test_all_drivers_hook_and_simple_compression():
    hook = NangilaHook.all_drivers(10)
    assert hook.current_step() == 0 and not hook.is_compression_enabled()
    g = np.random.default_rng(0).normal(size=1000).astype(np.float32)
    assert np.array_equal(hook.decompress(0, hook.compress(0, g)), g)
    hook.set_gpu_mode(True)
    hook.set_partial_retransmit(False)
    hook.set_hash_verify_interval(50)
    assert isinstance(hook.predictor_hash(), int) and not hook.should_verify_hash()


def test_advanced_knobs_warn():
    from nangila.ddp import _warn_if_advanced_ddp_options

    with pytest.warns(UserWarning, match="excluded from the Nangila v0.1 stable support contract"):
        _warn_if_advanced_ddp_options(1, 0.999, 1)
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        _warn_if_advanced_ddp_options(0, 0.999, 1)
