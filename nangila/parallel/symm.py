"""Peer-mapped ("symmetric") device memory for the fused exchange kernels.

A :class:`SymmArena` hands out byte regions that exist at the same offset on every rank of a process
group and whose peer addresses every rank knows, so a kernel on rank *a* can store straight into
rank *b*'s copy over NVLink. Three providers:

* ``torch``  – ``torch.distributed._symmetric_memory`` (allocation + rendezvous through the group's
  store); the default for groups of more than one rank;
* ``ipc``    – plain ``cudaMalloc`` memory exported with CUDA IPC handles that travel through
  ``all_gather_object``; selected with ``NANGILA_SYMM_BACKEND=ipc`` or automatically when the
  first provider is unavailable;
* ``local``  – an ordinary tensor, for a group of one rank.

:class:`LoopbackArena` gives ``world`` separate buffers on ONE device. It is the single-GPU stand-in
for a group (each "rank" is a slice of one cooperative kernel launch) used by the kernel tests.

The reference has no counterpart: it moves packets with ``all_gather`` of padded byte tensors
(python/nangila/ddp.py:249-260, nangila_ddp/src/ddp_hook.cpp:260-288).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

_ALIGN = 256
_CANARY = 0xA5          # NANGILA_CHECKED=1: every region is followed by a guard block of this byte
_CANARY_BYTES = 256


def _round_up(x: int, a: int = _ALIGN) -> int:
    return (x + a - 1) // a * a


class _Segment:
    """One allocation that is mapped on every rank. ``ptrs[r]`` is rank r's base address as seen
    from this process; ``local`` is this rank's own tensor."""

    def __init__(self, local: torch.Tensor, ptrs: List[int], keepalive: object = None):
        self.local = local
        self.ptrs = ptrs
        self.nbytes = local.numel()
        self.used = 0
        self._keepalive = keepalive

    def take(self, nbytes: int) -> Optional[int]:
        nbytes = _round_up(nbytes)
        if self.used + nbytes > self.nbytes:
            return None
        off = self.used
        self.used += nbytes
        return off


class Region:
    """A byte range present on every rank. ``ptrs[r]`` = address of rank r's copy."""

    def __init__(self, seg: _Segment, offset: int, nbytes: int):
        self.segment = seg
        self.offset = offset
        self.nbytes = nbytes
        self.ptrs = [p + offset for p in seg.ptrs]
        self.local = seg.local[offset:offset + nbytes]


def _provider_for(world: int) -> str:
    if world == 1:
        return "local"
    return os.environ.get("NANGILA_SYMM_BACKEND", "torch").lower()


class SymmArena:
    """Growable arena of symmetric segments for one process group. ``allocate`` is a collective when
    it has to add a segment (all ranks must then call it in the same order with the same size)."""

    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, segment_bytes: int = 64 << 20):
        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device)
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.segment_bytes = segment_bytes
        self.segments: List[_Segment] = []
        self._guards: List[torch.Tensor] = []
        self.provider = _provider_for(self.world)

    # -- providers ---------------------------------------------------------------------------
    def _new_segment_local(self, nbytes: int) -> _Segment:
        t = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        return _Segment(t, [t.data_ptr()])

    def _new_segment_torch(self, nbytes: int) -> _Segment:
        import torch.distributed._symmetric_memory as symm_mem

        # The kernels use plain peer stores, not multimem; do not bind the memory to a multicast
        # object unless asked to (a rank that dies while bound can fault its peers' links).
        if os.environ.get("NANGILA_USE_MULTIMEM", "0") != "1":
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        name = self.group.group_name
        try:
            symm_mem.enable_symm_mem_for_group(name)
        except Exception:
            pass
        t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        hdl = symm_mem.rendezvous(t, group=name)
        t.zero_()
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        return _Segment(t, ptrs, keepalive=hdl)

    def _new_segment_ipc(self, nbytes: int) -> _Segment:
        # cudaMalloc-backed storage (not an expandable segment) so that it can be exported.
        t = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        storage = t.untyped_storage()
        handle = storage._share_cuda_()
        base_off = t.storage_offset()
        gathered: List[object] = [None] * self.world
        dist.all_gather_object(gathered, (handle, base_off), group=self.group)
        ptrs: List[int] = []
        keep = []
        for r, (h, off) in enumerate(gathered):
            if r == self.rank:
                ptrs.append(t.data_ptr())
                continue
            h = list(h)
            h[0] = self.device.index if self.device.index is not None else torch.cuda.current_device()
            peer_storage = torch.UntypedStorage._new_shared_cuda(*h)
            keep.append(peer_storage)
            ptrs.append(peer_storage.data_ptr() + off)
        return _Segment(t, ptrs, keepalive=keep)

    def _new_segment(self, nbytes: int) -> _Segment:
        nbytes = _round_up(max(nbytes, self.segment_bytes), 2 << 20)
        if self.provider == "local":
            seg = self._new_segment_local(nbytes)
        elif self.provider == "ipc":
            seg = self._new_segment_ipc(nbytes)
        else:
            try:
                seg = self._new_segment_torch(nbytes)
            except Exception as exc:  # pragma: no cover - depends on the installed torch / driver
                if os.environ.get("NANGILA_SYMM_BACKEND"):
                    raise
                import warnings

                warnings.warn(f"nangila: torch symmetric memory unavailable ({exc!r}); using CUDA IPC")
                self.provider = "ipc"
                seg = self._new_segment_ipc(nbytes)
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)  # everybody's zero-fill has landed before any kernel stores
        self.segments.append(seg)
        return seg

    # -- public --------------------------------------------------------------------------------
    def reserve(self, nbytes: int) -> None:
        """Make sure at least ``nbytes`` can be handed out without another collective."""
        free = sum(s.nbytes - s.used for s in self.segments[-1:])
        if free < nbytes:
            self._new_segment(nbytes)

    def allocate(self, nbytes: int) -> Region:
        checked = os.environ.get("NANGILA_CHECKED", "0") == "1"
        want = _round_up(nbytes) + (_CANARY_BYTES if checked else 0)
        off = None
        for seg in self.segments:
            off = seg.take(want)
            if off is not None:
                break
        if off is None:
            seg = self._new_segment(want)
            off = seg.take(want)
            assert off is not None
        region = Region(seg, off, nbytes)
        if checked:
            guard = seg.local[off + _round_up(nbytes):off + _round_up(nbytes) + _CANARY_BYTES]
            guard.fill_(_CANARY)
            self._guards.append(guard)
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
        return region

    def check_canaries(self) -> None:
        """Checked mode: raise if any kernel (local or a peer's) wrote past the end of a region of this
        rank. The guards are filled at allocation and never written afterwards."""
        for i, g in enumerate(self._guards):
            if not bool((g == _CANARY).all()):
                bad = int((g != _CANARY).nonzero()[0])
                raise RuntimeError(f"nangila: guard block after symmetric region {i} was overwritten at byte {bad} "
                                   f"(rank {self.rank})")


class LoopbackArena:
    """``world`` separate buffers on one device: the single-GPU emulation of a group."""

    def __init__(self, world: int, device: torch.device):
        self.world = world
        self.rank = 0
        self.device = torch.device(device)
        self.provider = "loopback"
        self._guards: List[torch.Tensor] = []

    def reserve(self, nbytes: int) -> None:
        return None

    def allocate(self, nbytes: int) -> Region:
        nbytes = _round_up(nbytes)
        checked = os.environ.get("NANGILA_CHECKED", "0") == "1"
        total = nbytes + (_CANARY_BYTES if checked else 0)
        bufs = [torch.zeros(total, dtype=torch.uint8, device=self.device) for _ in range(self.world)]
        if checked:
            for b in bufs:
                b[nbytes:].fill_(_CANARY)
                self._guards.append(b[nbytes:])
        seg = _Segment(bufs[0], [b.data_ptr() for b in bufs], keepalive=bufs)
        return Region(seg, 0, nbytes)

    def check_canaries(self) -> None:
        for i, g in enumerate(self._guards):
            if not bool((g == _CANARY).all()):
                raise RuntimeError(f"nangila: guard block {i} of the loopback arena was overwritten")
