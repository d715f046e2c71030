"""Linear and LayerNorm whose parameter gradients use the fused column-sum kernel (``csrc/kernels/colsum.cu``).

Forward results are PyTorch's (cuBLAS GEMM with its bias epilogue; ``F.layer_norm``). What changes is
the backward of the small reductions over the token dimension: the bias gradient of a linear layer
and the weight / bias gradients of a LayerNorm, each of which is its own small reduction kernel in eager PyTorch.

Off by default, ``NANGILA_FUSED_GRADS=1`` turns both on. The kernels remove device time, but every custom autograd
function adds Python work per layer, so they pay off only where the host runs well ahead of the GPU; in an eager step
whose enqueue time is close to its device time the extra host work lands on the critical path.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

_LIB: Optional[ctypes.CDLL] = None
launch_count = 0  # column-sum launches (each is a partial + a final kernel)


def _lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = Path(__file__).resolve().parent.parent / "libnangila_kernels.so"
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run `python -m nangila._build --kernels`")
        lib = ctypes.CDLL(str(path))
        lib.nangila_colsum_scratch_floats.restype = ctypes.c_int64
        lib.nangila_colsum_scratch_floats.argtypes = [ctypes.c_int]
        lib.nangila_colsum.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                       ctypes.c_void_p]
        _LIB = lib
    return _LIB


def _eligible(t: torch.Tensor) -> bool:
    return (os.environ.get("NANGILA_FUSED_GRADS", "0") == "1" and t.is_cuda and t.dtype == torch.bfloat16 and t.size(-1) % 4 == 0)


def colsum(a: torch.Tensor, b: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``(a.sum(0), (a * b).sum(0))`` in fp32 for contiguous 2-D bf16 CUDA tensors (``b`` optional)."""
    global launch_count
    rows, cols = a.shape
    lib = _lib()
    scratch = torch.empty(lib.nangila_colsum_scratch_floats(cols), dtype=torch.float32, device=a.device)
    out = torch.empty((2 if b is not None else 1, cols), dtype=torch.float32, device=a.device)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    rc = lib.nangila_colsum(a.data_ptr(), b.data_ptr() if b is not None else None, rows, cols, scratch.data_ptr(), out.data_ptr(), stream)
    if rc != 0:
        raise RuntimeError(f"nangila_colsum failed with CUDA error {rc}")
    launch_count += 1
    return out[0], (out[1] if b is not None else None)


class _LinearBias(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
        ctx.save_for_backward(x, weight)
        return F.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.size(-1))
        dx = (dy2 @ weight).view_as(x) if ctx.needs_input_grad[0] else None
        dw = dy2.t() @ x2 if ctx.needs_input_grad[1] else None
        db = colsum(dy2)[0].to(dy.dtype) if ctx.needs_input_grad[2] else None
        return dx, dw, db


class _Affine(torch.autograd.Function):
    """y = x_hat * w + b over the last dimension."""

    @staticmethod
    def forward(ctx, xhat: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
        ctx.save_for_backward(xhat, weight)
        return torch.addcmul(bias, xhat, weight)

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        xhat, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.size(-1))
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        db, dw = colsum(dy2, xhat.reshape(-1, xhat.size(-1)))
        dx = dy * weight if ctx.needs_input_grad[0] else None
        return dx, dw.to(weight.dtype), db.to(weight.dtype)


def linear(x: torch.Tensor, lin: torch.nn.Linear) -> torch.Tensor:
    """``lin(x)`` with the bias gradient from the column-sum kernel (bf16 CUDA tensors; PyTorch's path otherwise)."""
    if lin.bias is None or not _eligible(x) or lin.weight.size(0) % 4 != 0 or not torch.is_grad_enabled():
        return lin(x)
    return _LinearBias.apply(x, lin.weight, lin.bias)


def layer_norm(x: torch.Tensor, ln: torch.nn.LayerNorm) -> torch.Tensor:
    """``ln(x)`` with the weight / bias gradients from the column-sum kernel (bf16 CUDA tensors; PyTorch's path otherwise)."""
    if ln.weight is None or ln.bias is None or not _eligible(x) or not torch.is_grad_enabled() or not x.is_contiguous():
        return ln(x)
    xhat = F.layer_norm(x, ln.normalized_shape, None, None, ln.eps)
    return _Affine.apply(xhat, ln.weight, ln.bias)
