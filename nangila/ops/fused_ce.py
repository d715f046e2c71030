"""Fused softmax cross-entropy for bf16 logits whose trailing columns are padding (``csrc/kernels/fused_ce.cu``).

``fused_cross_entropy(logits, targets, num_classes)`` equals
``F.cross_entropy(logits[:, :num_classes].float(), targets)`` (mean over rows) without the fp32 copy, the
log-softmax tensor and the fp32 gradient: the forward reads the logits once, the backward reads them
once more and writes the bf16 gradient with zeros in the padded columns.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch
import torch.nn.functional as F

_LIB: Optional[ctypes.CDLL] = None
launch_count = 0  # kernels launched by this module (forward and backward count one each)


def _lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = Path(__file__).resolve().parent.parent / "libnangila_kernels.so"
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run `python -m nangila._build --kernels`")
        lib = ctypes.CDLL(str(path))
        lib.nangila_ce_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                           ctypes.c_int64, ctypes.c_void_p]
        lib.nangila_ce_backward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.c_int, ctypes.c_int64, ctypes.c_void_p]
        _LIB = lib
    return _LIB


class _FusedCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, targets: torch.Tensor, num_classes: int) -> torch.Tensor:
        rows, stride = logits.shape
        losses = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        stream = torch.cuda.current_stream(logits.device).cuda_stream
        global launch_count
        launch_count += 1
        rc = _lib().nangila_ce_forward(logits.data_ptr(), targets.data_ptr(), losses.data_ptr(), lse.data_ptr(), rows, num_classes, stride, stream)
        if rc != 0:
            raise RuntimeError(f"nangila_ce_forward failed with CUDA error {rc}")
        ctx.save_for_backward(logits, targets, lse)
        ctx.num_classes = num_classes
        return losses.mean()

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        logits, targets, lse = ctx.saved_tensors
        rows, stride = logits.shape
        grad = torch.empty_like(logits)
        g = grad_output.detach().to(torch.float32).reshape(1).contiguous()
        stream = torch.cuda.current_stream(logits.device).cuda_stream
        global launch_count
        launch_count += 1
        rc = _lib().nangila_ce_backward(logits.data_ptr(), targets.data_ptr(), lse.data_ptr(), g.data_ptr(), grad.data_ptr(), rows,
                                        ctx.num_classes, stride, stream)
        if rc != 0:
            raise RuntimeError(f"nangila_ce_backward failed with CUDA error {rc}")
        return grad, None, None


def fused_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, num_classes: Optional[int] = None) -> torch.Tensor:
    """Mean cross-entropy of ``logits[:, :num_classes]`` against ``targets``. CUDA bf16 logits with a
    row length that is a multiple of 8 take the fused kernels; anything else (or ``NANGILA_FUSED_CE=0``) takes
    PyTorch's path."""
    if logits.dim() != 2:
        logits = logits.reshape(-1, logits.size(-1))
    targets = targets.reshape(-1)
    v = logits.size(1) if num_classes is None else int(num_classes)
    if (os.environ.get("NANGILA_FUSED_CE", "1") != "0" and logits.is_cuda and logits.dtype == torch.bfloat16 and logits.size(1) % 8 == 0 and logits.is_contiguous()
            and logits.data_ptr() % 16 == 0 and 0 < v <= logits.size(1)):
        return _FusedCrossEntropy.apply(logits, targets.to(torch.int64).contiguous(), v)
    return F.cross_entropy(logits[:, :v].float(), targets)
