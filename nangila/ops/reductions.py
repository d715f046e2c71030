"""Small device reductions: state hash, parallel CRC32, max / percentile of |x|."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch


def _glue():
    from ..parallel.predres_engine import _glue as g

    return g()


def state_hash(tensors: Sequence[torch.Tensor], seed: int = 0) -> int:
    """64-bit hash of the bytes of ``tensors`` (order of the list matters, launch geometry does not).
    Ranks that hold identical state get identical hashes; used for the periodic cross-rank predictor
    check (reference: nangila-core/src/predictor.rs:455-477 on the host)."""
    out = _glue().state_hash([t.contiguous() for t in tensors], seed)
    return int(out.item()) & 0xFFFFFFFFFFFFFFFF


def crc32(t: torch.Tensor) -> int:
    """IEEE CRC32 of a device buffer, equal to ``zlib.crc32`` of its bytes
    (reference: nangila-cuda/src/kernels/crc32.cu:56-72, single-threaded there)."""
    return int(_glue().crc32(t.contiguous()).item()) & 0xFFFFFFFF


def absmax_percentile(x: torch.Tensor, percentile: float = 0.99, qmax: float = 7.0) -> Tuple[float, float, float, torch.Tensor]:
    """Returns ``(max |x|, value at the percentile of |x|, gamma, histogram)`` where the percentile
    is the host quantizer's order statistic ``sorted(|x|)[int(n * percentile)]``, gamma =
    ``max(that / qmax, 1e-8)`` and the histogram has 256 linear bins of ``|x| / max``
    (reference: nangila-cuda/src/kernels/gamma.cu, nangila-core/src/quantizer.rs:81-96)."""
    n = x.numel()
    idx = min(int(float(torch.tensor(n, dtype=torch.float32) * torch.tensor(percentile, dtype=torch.float32))), n - 1)
    k = n - idx  # rank from the top
    out, hist = _glue().absmax_hist(x.contiguous().view(-1), k, qmax)
    vals = out.tolist()
    return vals[0], vals[1], vals[2], hist


def quantizer_gamma(x: torch.Tensor, bits: int = 4) -> float:
    """The single-scale quantizer's gamma for ``x``: p99(|x|) / (2^(bits-1) - 1), floored at 1e-8."""
    return absmax_percentile(x, 0.99, float((1 << (bits - 1)) - 1))[2]
