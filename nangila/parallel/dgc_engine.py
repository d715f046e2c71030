"""Host driver of the fused DGC kernel: per-bucket velocity / accumulator state, the symmetric
receive slots for every rank's sparse list, and one cooperative launch per bucket call.

Replaces DGCCompressor (nangila-core/src/dgc.rs:44-186: per-layer residual map, sort-based top-k)
plus the all-gather of packets around it; adds the momentum correction the reference omits.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .predres_engine import STATUS_MESSAGES, _glue
from .symm import LoopbackArena, Region

_GROUP_CTAS = 296  # default CTAs per launch in a real process group
_LIST_CTAS = 444  # CTAs whose equal segments of the candidate list the scratch buffer has slack for


@dataclass
class DGCBucket:
    n: int
    k: int
    capacity: int
    region: Region
    recv_off: int
    flag_off: int
    u: List[torch.Tensor]
    v: List[torch.Tensor]
    scratch: List[torch.Tensor]
    out_count: List[torch.Tensor]
    epoch: int = 0


def keep_count(n: int, sparsity: float) -> int:
    """ceil(n * (1 - sparsity)) in float32 arithmetic, like the host compressor (dgc.rs:116-120)."""
    import numpy as np

    return max(1, int(math.ceil(float(np.float32(n) * (np.float32(1.0) - np.float32(sparsity))))))


class DGCEngine:
    def __init__(self, arena, device: torch.device, sparsity: float = 0.999, momentum: float = 0.9,
                 stream: Optional[torch.cuda.Stream] = None, timeout_s: Optional[float] = None,
                 ctas: Optional[int] = None):
        self.arena = arena
        self.device = torch.device(device)
        self.world = arena.world
        self.rank = arena.rank
        self.loopback = isinstance(arena, LoopbackArena)
        self.nvr = self.world if self.loopback else 1
        self.sparsity = float(sparsity)
        self.momentum = float(momentum)
        self.stream = stream
        self.timeout_s = float(os.environ.get("NANGILA_WAIT_TIMEOUT_MS", "2000")) / 1e3 if timeout_s is None else timeout_s
        self.ctas = ctas or int(os.environ.get("NANGILA_DGC_CTAS", "0")) or None  # CTAs per launch (default: as many as the candidate list is sized for)
        self.buckets: Dict[int, DGCBucket] = {}
        self.status = [torch.zeros(8, dtype=torch.int32, device=self.device) for _ in range(self.nvr)]
        self.launches = 0
        self._glue = _glue()

    def _grid(self, n: int) -> int:
        # the candidate-list scratch is sized for _LIST_CTAS CTAs; the launcher clamps to what the device can hold at once.
        # A real group runs two thirds of that: the kernel then shares the GPU with backward instead of queueing for it.
        cap = self.ctas or (max(1, _LIST_CTAS // self.nvr) if self.loopback else _GROUP_CTAS)
        return max(1, min(cap, (n + 1023) // 1024))  # 4 elements per thread and pass

    def bucket_state(self, index: int, grads: List[torch.Tensor]) -> DGCBucket:
        n = grads[0].numel()
        st = self.buckets.get(index)
        if st is not None and st.n == n:
            return st
        k = min(keep_count(n, self.sparsity), n)
        capacity = (k + k // 8 + 64 + 3) // 4 * 4  # room for ties at the threshold
        total, recv_off, flag_off, scratch_words = self._glue.dgc_region_layout(capacity, self.world)
        region = self.arena.allocate(int(total))
        z = lambda m, dt: torch.zeros(m, dtype=dt, device=self.device)  # noqa: E731
        st = DGCBucket(n=n, k=k, capacity=capacity, region=region, recv_off=recv_off, flag_off=flag_off,
                       u=[z(n, torch.float32) for _ in range(self.nvr)], v=[z(n, torch.float32) for _ in range(self.nvr)],
                       # fixed words + the candidate list (index, bits) of the list-based selection. Unsent entries
                       # pile up just below the threshold (about 17 k of them within 4 % of it), and every CTA owns an
                       # equal segment of the list, hence the slack.
                       scratch=[z(scratch_words + 2 * (32 * k + 128 * _LIST_CTAS), torch.int32) for _ in range(self.nvr)],
                       out_count=[z(2, torch.int32) for _ in range(self.nvr)])
        self.buckets[index] = st
        return st

    def reduce(self, index: int, grads) -> int:
        """Queue the fused DGC exchange; ``grads`` (a tensor, or one per emulated rank) is replaced by
        the dense mean of all ranks' selected entries. Returns k, the entries this rank sends."""
        if isinstance(grads, torch.Tensor):
            grads = [grads]
        st = self.bucket_state(index, grads)
        st.epoch += 1
        self.launches += 1
        args = dict(grad=grads, u=st.u, v=st.v, scratch=st.scratch, status=self.status, out_count=st.out_count,
                    region_ptrs=st.region.ptrs, recv_off=st.recv_off, flag_off=st.flag_off,
                    rank0=0 if self.loopback else self.rank, k=st.k, capacity=st.capacity, epoch=st.epoch,
                    momentum=self.momentum, timeout_s=self.timeout_s, grid_x=self._grid(st.n))
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                self._glue.dgc_launch(**args)
        else:
            self._glue.dgc_launch(**args)
        return st.k

    def check_status(self) -> None:
        (self.stream.synchronize() if self.stream is not None else torch.cuda.synchronize(self.device))
        for s in self.status:
            w = s.cpu().tolist()
            if w[0] != 0:
                s.zero_()
                raise RuntimeError(f"nangila: fused DGC exchange failed on rank {w[1]} "
                                   f"({STATUS_MESSAGES.get(w[0], 'code %d' % w[0])}); waiting for rank {w[2]}")
