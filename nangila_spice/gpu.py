"""Device side of the circuit simulator: a CSR matrix resident on the GPU, ``y = A x`` on it and a
Jacobi-preconditioned BiCGSTAB, through the C interface of ``libnangila_kernels.so``
(``csrc/kernels/nangila_spice_kernels.h``).

The reference's counterpart is ``GpuSolver`` with its cuSPARSE bridge
(``nangila-spice/nangila-node/src/gpu_solver.rs:330-512``, ``cuda/cusparse_solver.cu:17-123``).
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Optional, Sequence, Tuple

import numpy as np

_LIB: Optional[ctypes.CDLL] = None


def kernels_library() -> ctypes.CDLL:
    """Loads the kernel library built in-tree next to the ``nangila`` package; raises if it is missing."""
    global _LIB
    if _LIB is None:
        path = Path(__file__).resolve().parent.parent / "nangila" / "libnangila_kernels.so"
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run `python -m nangila._build --kernels`")
        lib = ctypes.CDLL(str(path))
        lib.nangila_spmv_create.restype = ctypes.c_void_p
        lib.nangila_spmv_destroy.argtypes = [ctypes.c_void_p]
        lib.nangila_spmv_load.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.nangila_spmv_update_values.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.nangila_spmv_host.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.nangila_spmv_device.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.nangila_spmv_status.argtypes = [ctypes.c_void_p]
        lib.nangila_spmv_dims.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.nangila_spmv_build_row_blocks.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
        lib.nangila_spmv_launch.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_void_p]
        lib.nangila_spmv_bicgstab.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_double, ctypes.c_int,
                                              ctypes.c_void_p, ctypes.c_void_p]
        _LIB = lib
    return _LIB


def enable_device_solver() -> str:
    """Points the simulator core at the kernel library, so ``solver="cuda"`` (the linear systems of the
    Newton iteration solved by BiCGSTAB on the GPU, matrix resident, values refreshed per iteration)
    can bind it at run time. Returns the path."""
    from . import _native

    path = Path(__file__).resolve().parent.parent / "nangila" / "libnangila_kernels.so"
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m nangila._build --kernels`")
    _native.set_cuda_library(str(path))
    return str(path)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with CUDA error {rc}")


def build_row_blocks(row_ptr: np.ndarray) -> np.ndarray:
    """Row-block table of a CSR pattern (host computation; no GPU needed)."""
    lib = kernels_library()
    rp = np.ascontiguousarray(row_ptr, dtype=np.int32)
    n = rp.size - 1
    count = lib.nangila_spmv_build_row_blocks(rp.ctypes.data, n, None, 0)
    out = np.zeros(count + 1, dtype=np.int32)
    lib.nangila_spmv_build_row_blocks(rp.ctypes.data, n, out.ctypes.data, count + 1)
    return out


class DeviceCsr:
    """An ``n x n`` FP64 CSR matrix kept on the current CUDA device."""

    def __init__(self, row_ptr: Sequence[int], col: Sequence[int], val: Sequence[float], plain_loads: bool = False):
        """``plain_loads`` selects the kernel variant that stages with ordinary loads instead of bulk
        copies (the default); it exists for comparison and for debugging."""
        import os

        self._lib = kernels_library()
        previous = os.environ.get("NANGILA_SPMV_PLAIN")
        os.environ["NANGILA_SPMV_PLAIN"] = "1" if plain_loads else "0"
        try:
            self._load(row_ptr, col, val)
        finally:
            if previous is None:
                os.environ.pop("NANGILA_SPMV_PLAIN", None)
            else:
                os.environ["NANGILA_SPMV_PLAIN"] = previous

    def _load(self, row_ptr, col, val) -> None:
        self._ctx = self._lib.nangila_spmv_create()
        if not self._ctx:
            raise MemoryError("nangila_spmv_create")
        rp = np.ascontiguousarray(row_ptr, dtype=np.int32)
        ci = np.ascontiguousarray(col, dtype=np.int32)
        va = np.ascontiguousarray(val, dtype=np.float64)
        if ci.size != va.size or rp.size < 2:
            raise ValueError("inconsistent CSR arrays")
        self.n, self.nnz = rp.size - 1, int(va.size)
        _check(self._lib.nangila_spmv_load(self._ctx, self.n, self.nnz, rp.ctypes.data, ci.ctypes.data, va.ctypes.data), "nangila_spmv_load")

    @property
    def num_row_blocks(self) -> int:
        nb = ctypes.c_int(0)
        self._lib.nangila_spmv_dims(self._ctx, None, None, ctypes.byref(nb))
        return nb.value

    def check_status(self) -> None:
        """Raises if a kernel of this matrix gave up waiting for one of its copies (synchronises)."""
        _check(self._lib.nangila_spmv_status(self._ctx), "spmv kernel (bulk copy wait)")

    def update_values(self, val: Sequence[float]) -> None:
        va = np.ascontiguousarray(val, dtype=np.float64)
        if va.size != self.nnz:
            raise ValueError("value count differs from the loaded pattern")
        _check(self._lib.nangila_spmv_update_values(self._ctx, va.ctypes.data), "nangila_spmv_update_values")

    def matvec(self, x: Sequence[float]) -> np.ndarray:
        """``A @ x`` with host vectors (copied to the device and back)."""
        xv = np.ascontiguousarray(x, dtype=np.float64)
        if xv.size != self.n:
            raise ValueError("vector length differs from the matrix size")
        y = np.empty(self.n, dtype=np.float64)
        _check(self._lib.nangila_spmv_host(self._ctx, xv.ctypes.data, y.ctypes.data), "nangila_spmv_host")
        return y

    def matvec_device(self, x, y, stream: int = 0) -> None:
        """``y = A @ x`` on torch CUDA float64 tensors; queued on ``stream`` (a raw handle), no copies."""
        if x.numel() != self.n or y.numel() != self.n or not x.is_cuda or not y.is_cuda:
            raise ValueError("x and y must be CUDA tensors of the matrix size")
        import torch

        if x.dtype != torch.float64 or y.dtype != torch.float64 or not x.is_contiguous() or not y.is_contiguous():
            raise ValueError("x and y must be contiguous float64 tensors")
        _check(self._lib.nangila_spmv_device(self._ctx, x.data_ptr(), y.data_ptr(), stream), "nangila_spmv_device")

    def solve(self, b: Sequence[float], tol: float = 1e-10, max_iter: int = 2000) -> Tuple[np.ndarray, int, float, bool]:
        """BiCGSTAB from ``x = 0``: returns ``(x, iterations, relative residual, converged)``."""
        bv = np.ascontiguousarray(b, dtype=np.float64)
        if bv.size != self.n:
            raise ValueError("vector length differs from the matrix size")
        x = np.zeros(self.n, dtype=np.float64)
        it, rel = ctypes.c_int(0), ctypes.c_double(0.0)
        rc = self._lib.nangila_spmv_bicgstab(self._ctx, bv.ctypes.data, x.ctypes.data, tol, max_iter, ctypes.byref(it), ctypes.byref(rel))
        if rc not in (0, -1):
            _check(rc, "nangila_spmv_bicgstab")
        return x, it.value, rel.value, rc == 0

    def close(self) -> None:
        if self._ctx:
            self._lib.nangila_spmv_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def tridiagonal(n: int, diag: float = 2.0, off: float = -1.0) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """CSR arrays of the n x n tridiagonal matrix (the RC-ladder pattern of the reference's GPU benchmark)."""
    counts = np.full(n, 3, dtype=np.int64)
    counts[0] -= 1
    counts[-1] -= 1
    row_ptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=row_ptr[1:])
    col = np.empty(row_ptr[-1], dtype=np.int32)
    val = np.empty(row_ptr[-1], dtype=np.float64)
    idx = np.arange(n)
    dpos = row_ptr[:-1] + (idx > 0)
    col[dpos] = idx
    val[dpos] = diag
    col[dpos[1:] - 1] = idx[1:] - 1
    val[dpos[1:] - 1] = off
    col[dpos[:-1] + 1] = idx[:-1] + 1
    val[dpos[:-1] + 1] = off
    return row_ptr.astype(np.int32), col, val
