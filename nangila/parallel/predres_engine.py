"""Host driver of the fused prediction-residual bucket kernel.

One :class:`PredResEngine` per process group keeps, for every gradient bucket it has seen, the
device state the kernel needs (two-step history, error-feedback memories, the bucket's symmetric
exchange region, its epoch counter) and queues exactly one kernel launch per bucket call on a
dedicated high-priority stream, so the exchange overlaps with the rest of backward.

Replaces the per-bucket sequence of the reference hook — compress kernel, two all-gathers with host
synchronisation, one reconstruct kernel per rank, mean, history copies (python/nangila/ddp.py:236-284,
nangila_ddp/src/ddp_hook.cpp:104-335) — and its per-layer GPU history buffers with pointer-swap
rotation (nangila-cuda/src/state.rs:99-184).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .symm import LoopbackArena, Region

_DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

STATUS_MESSAGES = {
    2: "timeout in phase 2: a chunk owner did not receive every rank's contribution",
    3: "timeout in phase 3: a reduced chunk did not arrive from its owner",
    4: "timeout in an intra-GPU grid barrier",
    5: "bad argument",
    6: "timeout waiting for a bulk copy into shared memory",
}


def _glue():
    """The compiled torch glue. Raises with a clear message when it has not been built."""
    try:
        from .. import _cuda  # type: ignore
    except ImportError as exc:  # pragma: no cover
        raise RuntimeError(
            "nangila: the CUDA extension (nangila/_cuda*.so) is not built; run `python -m nangila._build`"
        ) from exc
    return _cuda


def default_chunk_elems(n: int, world: int, resident: int = 0) -> int:
    """Chunk size (elements). Each phase of the kernel walks the chunks in waves of ``resident`` CTAs (what the
    device holds at once, divided by the emulated ranks): the size is the smallest multiple of 4096 that covers
    the bucket in whole waves with no chunk above 131072 elements, so the last wave is as full as the others.
    ``NANGILA_CHUNK`` overrides."""
    env = os.environ.get("NANGILA_CHUNK")
    if env:
        return int(env)
    return int(_glue().predres_chunk_elems(int(n), int(resident)))


@dataclass
class BucketState:
    n: int
    grad_dtype: torch.dtype
    state_dtype: torch.dtype
    chunk: int
    region: Region
    layout: Tuple[int, int, int, int]
    prev: List[torch.Tensor]
    curr: List[torch.Tensor]
    ef: List[Optional[torch.Tensor]]
    ef2: List[Optional[torch.Tensor]]
    stats: List[torch.Tensor]
    slot: int = 0                       # row of this bucket in the engine's statistics table
    pred_gain: float = 1.0              # kappa: 1 = full momentum prediction, 0 = none
    miss_ema: Optional[float] = None    # running ||g - g_hat||^2 / ||g||^2
    cooldown: int = 0
    probe_every: int = 0                # calls between probes of the history while the gain is 0 (0: engine default)
    next_probe: int = 0                 # call number of the next probe
    last_probe: int = 0                 # call number of the most recent probe
    totals: List[float] = field(default_factory=lambda: [0.0, 0.0, 0.0, 0.0])
    epoch: int = 0
    calls: int = 0
    compressed_calls: int = 0
    extra: dict = field(default_factory=dict)

    def swap(self) -> None:
        self.prev, self.curr = self.curr, self.prev


class PredResEngine:
    """Drives ``nangila_predres_launch``.

    ``arena`` is a :class:`SymmArena` (real group; one rank per process) or a :class:`LoopbackArena`
    (all ``world`` ranks emulated in one launch on this device).
    """

    def __init__(self, arena, device: torch.device, momentum: float = 0.9, error_feedback: bool = True,
                 state_dtype: Optional[torch.dtype] = None, stochastic: bool = True, seed: int = 42,
                 timeout_s: Optional[float] = None, ctas: Optional[int] = None, use_side_stream: bool = True,
                 owner_error_feedback: bool = False, adaptive_gain: bool = True, max_buckets: int = 512):
        self.arena = arena
        self.device = torch.device(device)
        self.world = arena.world
        self.rank = arena.rank
        self.loopback = isinstance(arena, LoopbackArena)
        self.nvr = self.world if self.loopback else 1
        self.momentum = float(momentum)
        self.error_feedback = error_feedback
        self.state_dtype = state_dtype
        self.stochastic = stochastic
        self.seed = seed
        self.timeout_s = float(os.environ.get("NANGILA_WAIT_TIMEOUT_MS", "2000")) / 1e3 if timeout_s is None else timeout_s
        self.ctas = int(os.environ.get("NANGILA_COMM_CTAS", "0")) if ctas is None else ctas
        self.owner_error_feedback = owner_error_feedback
        self.adaptive_gain = adaptive_gain and os.environ.get("NANGILA_PRED_GAIN") is None
        self.fixed_gain = float(os.environ.get("NANGILA_PRED_GAIN", "1"))
        # with a zero gain the kernel skips the history loads except on every probe_every-th call
        self.probe_every = max(1, int(os.environ.get("NANGILA_PROBE_EVERY", "8")))
        # two ranks use the kernel's gather mode (one quantization, two phases); from three ranks on every rank would
        # dequantize all contributions of every chunk itself, and the three-phase form does less work per rank
        self.gather_max_world = min(4, int(os.environ.get("NANGILA_GATHER_MAX_WORLD", "2")))
        # leave the history unwritten between probes while the gain is 0 (NANGILA_SKIP_HISTORY=0: always write it)
        self.skip_history = os.environ.get("NANGILA_SKIP_HISTORY", "1") != "0"
        self.buckets: Dict[int, BucketState] = {}
        # one row of 8 floats per (bucket, emulated rank): {sum e^2, sum g^2, sum miss^2, sum ef^2, ...}
        self.max_buckets = max_buckets
        self._next_slot = 0
        self.stats_table = torch.zeros(max_buckets * self.nvr, 8, dtype=torch.float32, device=self.device)
        self._stats_host = torch.zeros(max_buckets * self.nvr, 8, dtype=torch.float32).pin_memory() \
            if torch.cuda.is_available() else torch.zeros(max_buckets * self.nvr, 8)
        self._stats_event: Optional[torch.cuda.Event] = None
        self.status = [torch.zeros(8, dtype=torch.int32, device=self.device) for _ in range(self.nvr)]
        self.launches = 0
        self.nvtx = os.environ.get("NANGILA_NVTX", "0") == "1"      # one NVTX range per bucket launch
        self.timing = os.environ.get("NANGILA_TIMING", "0") == "1"  # CUDA events around every launch
        self._events: Dict[int, tuple] = {}
        self.stream: Optional[torch.cuda.Stream] = None
        if use_side_stream:
            self.stream = torch.cuda.Stream(device=self.device, priority=-1)
        self._glue = _glue()
        self._resident: Optional[int] = None  # CTAs per (emulated) rank the device holds at once

    # ------------------------------------------------------------------------------------------
    def _grid(self, st: BucketState) -> int:
        nchunks = (st.n + st.chunk - 1) // st.chunk
        owned = (nchunks + self.world - 1) // self.world
        want = owned * self.world
        if self.ctas > 0:
            cap = self.ctas
        else:
            cap = 1 << 20  # the launcher clamps to what the device can hold at once (divided by the emulated ranks)
        return max(1, min(want, cap))

    def _take_slot(self, index: int) -> int:
        """Row of the statistics table for a bucket; a rebuilt bucket keeps the row of its index."""
        old = self.buckets.get(index)
        if old is not None:
            return old.slot
        slot = self._next_slot % self.max_buckets
        self._next_slot += 1
        return slot

    def _state_dtype_for(self, grad_dtype: torch.dtype) -> torch.dtype:
        if self.state_dtype is not None:
            return self.state_dtype
        return torch.float32 if grad_dtype == torch.float32 else torch.bfloat16

    def bucket_state(self, index: int, grads: List[torch.Tensor]) -> BucketState:
        g0 = grads[0]
        n = g0.numel()
        st = self.buckets.get(index)
        if st is not None and st.n == n and st.grad_dtype == g0.dtype:
            return st
        if g0.dtype not in _DTYPE_CODE:
            raise TypeError(f"nangila: unsupported gradient dtype {g0.dtype}")
        if self._resident is None:
            self._resident = max(1, int(self._glue.predres_resident_ctas()) // self.nvr)
        chunk = default_chunk_elems(n, self.world, self._resident)
        total, r1, r2, f1, f2 = self._glue.predres_region_layout(n, self.world, chunk, _DTYPE_CODE[g0.dtype])
        region = self.arena.allocate(int(total))
        sdt = self._state_dtype_for(g0.dtype)
        nchunks = (n + chunk - 1) // chunk
        owned = (nchunks + self.world - 1) // self.world
        mk = lambda m, dt=sdt: torch.zeros(m, dtype=dt, device=self.device)  # noqa: E731
        st = BucketState(
            n=n, grad_dtype=g0.dtype, state_dtype=sdt, chunk=chunk, region=region, layout=(r1, r2, f1, f2),
            prev=[mk(n) for _ in range(self.nvr)], curr=[mk(n) for _ in range(self.nvr)],
            ef=[mk(n) if self.error_feedback else None for _ in range(self.nvr)],
            ef2=[mk(owned * chunk) if (self.error_feedback and self.owner_error_feedback) else None
                 for _ in range(self.nvr)],
            stats=[], slot=self._take_slot(index), pred_gain=self.fixed_gain,
        )
        st.stats = [self.stats_table[st.slot * self.nvr + v] for v in range(self.nvr)]
        for t in st.stats:
            t.zero_()
        self.buckets[index] = st
        return st

    def reduce(self, index: int, grads: List[torch.Tensor], compressed: bool, step: int = 0,
               split_phases: bool = False) -> BucketState:
        """Queue the fused exchange for one bucket. ``grads`` has one tensor per emulated rank (one
        in a real group). The result overwrites ``grads`` in place; the history advances.
        ``split_phases`` queues the phases of the exchange as separate launches of the same kernel (what
        the C++ DDP hook does to defer the waiting phases); the result is the same bytes."""
        st = self.bucket_state(index, grads)
        st.epoch += 1
        st.calls += 1
        st.compressed_calls += int(compressed)
        r1, r2, f1, f2 = st.layout
        measure = self._probe_due(st)
        gather = compressed and 2 <= self.world <= self.gather_max_world
        # While the gain is 0 nothing reads the history except a probe: it is written on the two calls before a
        # probe and the two after it (until the controller has seen the probe's statistics) and left alone otherwise.
        skip_history = (self.skip_history and compressed and st.pred_gain == 0.0 and st.extra.get("pred_gain_per_rank") is None
                        and not measure and st.calls + 2 < st.next_probe and st.calls > st.last_probe + 2)
        if split_phases and self.world > 1:
            masks = [1, 2] if gather else [1, 2, 4]
        else:
            masks = [0]
        self.launches += len(masks)
        args = dict(
            grad=grads, prev=st.prev, curr=st.curr, ef=st.ef, ef2=st.ef2, stats=st.stats, status=self.status,
            region_ptrs=st.region.ptrs, recv1_off=r1, recv2_off=r2, flag1_off=f1, flag2_off=f2,
            rank0=0 if self.loopback else self.rank, chunk_elems=st.chunk, mode=0 if compressed else 1,
            stochastic=self.stochastic, measure=measure, epoch=st.epoch, seed=self.seed, step=step, bucket_id=index,
            mu=self.momentum, pred_gain=self._gains(st), timeout_s=self.timeout_s, grid_x=self._grid(st),
            uniform_gain=st.extra.get("pred_gain_per_rank") is None,
            gather=gather, skip_history=skip_history,
        )
        if self.nvtx:
            torch.cuda.nvtx.range_push(f"nangila.bucket{index}.{'int4' if compressed else 'exact'}")
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                for m in masks:
                    self._timed_launch(index, dict(args, phase_mask=m))
        else:
            for m in masks:
                self._timed_launch(index, dict(args, phase_mask=m))
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        st.swap()
        return st

    def _timed_launch(self, index: int, args: dict) -> None:
        if not self.timing:
            self._glue.predres_launch(**args)
            return
        ev = self._events.get(index)
        if ev is None:
            ev = self._events[index] = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        ev[0].record()
        self._glue.predres_launch(**args)
        ev[1].record()

    def kernel_times_ms(self) -> Dict[int, float]:
        """Device time of the most recent launch of every bucket (``NANGILA_TIMING=1``); buckets whose
        last launch has not finished yet are left out. Nothing is synchronised."""
        out = {}
        for idx, (e0, e1) in self._events.items():
            if e1.query():
                out[idx] = e0.elapsed_time(e1)
        return out

    def _probe_due(self, st: BucketState) -> bool:
        """While the gain is 0 the kernel looks at the history only on probe calls. Probes that keep finding
        nothing to predict are spaced out (every 8th call, then 16th, ... up to 64th); a probe that finds
        something resets the spacing."""
        if st.probe_every == 0:
            st.probe_every = self.probe_every
            st.next_probe = st.probe_every
        if st.calls < st.next_probe:
            return False
        st.last_probe = st.calls
        st.next_probe = st.calls + st.probe_every
        return True

    def _gains(self, st: BucketState) -> List[float]:
        g = st.extra.get("pred_gain_per_rank")
        return list(g) if g is not None else [st.pred_gain] * self.nvr

    # ------------------------------------------------------------------------------------------
    def end_step(self) -> None:
        """Call once per training step after the last bucket was queued. Reads the statistics of the
        PREVIOUS step (already on the host, so nothing blocks), adapts every bucket's prediction gain,
        then queues the copy of this step's statistics.

        Gain control: the kernel subtracts kappa * g_hat. The best kappa for a step is the
        least-squares shrinkage <g + ef, g_hat> / <g_hat, g_hat> clipped to [0, 1]: 1 when the
        momentum predictor tracks the gradient, near 0 when consecutive gradients are dominated by
        mini-batch noise (subtracting a full-size prediction there would make the residual larger
        than the gradient and, through error feedback, amplify the predictor's own quantization
        noise). Both inner products come from the kernel; the value of the previous step is used
        (smoothed). The statistics are summed over the process group before they are read, so every
        rank derives the same gain and the kernel is told so (``uniform_gain``); when a caller sets
        different gains per rank the kernel applies their mean, carried in the chunk trailers. A
        run-away error-feedback memory switches prediction off for a while.
        """
        if self._stats_event is not None:
            self._stats_event.synchronize()
            host = self._stats_host
            for st in self.buckets.values():
                # emulated ranks: one controller for all of them, fed with the sum of their rows
                row = host[st.slot * self.nvr:(st.slot + 1) * self.nvr].sum(0).tolist()
                e2, g2, xp, pp, f2 = row[0], row[1], row[2], row[3], row[4]
                if g2 <= 0.0:
                    continue
                for k, v in enumerate((e2, g2, xp, pp)):
                    st.totals[k] += v
                st.miss_ema = e2 / g2 if st.miss_ema is None else 0.7 * st.miss_ema + 0.3 * e2 / g2
                if not self.adaptive_gain:
                    continue
                if st.cooldown > 0:
                    st.cooldown -= 1
                    continue
                if f2 > 2.0 * g2:
                    st.pred_gain, st.cooldown = 0.0, 20
                    continue
                if pp <= 0.0:
                    continue  # not a probe step: the kernel did not look at the history
                best = min(max(xp / pp, 0.0), 1.0)
                gain = 0.5 * st.pred_gain + 0.5 * best
                st.pred_gain = gain if gain >= 0.2 else 0.0  # below 0.2 (< 4 % less residual energy) the history loads cost more than they save
                if st.probe_every:
                    st.probe_every = self.probe_every if st.pred_gain > 0.0 else min(2 * st.probe_every, max(64, self.probe_every))
        stream = self.stream if self.stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.stream(stream):
            if self.world > 1 and not self.loopback and self.adaptive_gain:
                # every rank must derive the same gains: sum the statistics over the group first
                dist.all_reduce(self.stats_table, group=getattr(self.arena, "group", None))
            self._stats_host.copy_(self.stats_table, non_blocking=True)
            self.stats_table.zero_()
            ev = torch.cuda.Event()
            ev.record(stream)
        self._stats_event = ev

    def check_status(self) -> None:
        """Synchronise the exchange stream and raise if a kernel gave up waiting."""
        if self.stream is not None:
            self.stream.synchronize()
        else:
            torch.cuda.synchronize(self.device)
        if os.environ.get("NANGILA_CHECKED", "0") == "1" and hasattr(self.arena, "check_canaries"):
            self.arena.check_canaries()
        for vr, s in enumerate(self.status):
            w = s.cpu().tolist()
            if w[0] != 0:
                s.zero_()
                raise RuntimeError(
                    f"nangila: fused exchange failed on rank {w[1]} ({STATUS_MESSAGES.get(w[0], 'code %d' % w[0])}); "
                    f"waiting for rank {w[2]}, epoch {w[3]} (last seen {w[4]}), phase {w[5]}, chunk {w[6]}")

    def resync(self) -> None:
        """Recovery after a failed exchange (``check_status`` raised on some rank, or a rank skipped a
        call): every rank must call this at the same point. The ranks agree on the highest epoch any of
        them reached for each bucket (one small MAX all-reduce through the process group), so the next
        launch uses the same, fresh epoch everywhere and no flag left over from the failed exchange can
        satisfy it; the status blocks are cleared. The caller should make the next call on every bucket
        an uncompressed one, which re-seeds the history on all ranks (what the DDP hook does)."""
        if self.stream is not None:
            self.stream.synchronize()
        for s_ in self.status:
            s_.zero_()
        if self.loopback or self.world == 1 or not self.buckets:
            return
        keys = sorted(self.buckets)
        ep = torch.tensor([self.buckets[k].epoch + 1 for k in keys], dtype=torch.int64, device=self.device)
        dist.all_reduce(ep, op=dist.ReduceOp.MAX, group=getattr(self.arena, "group", None))
        for k, e in zip(keys, ep.tolist()):
            self.buckets[k].epoch = int(e)

    def prediction_error(self, index: int) -> float:
        """sqrt(sum e^2 / sum g^2) accumulated over the compressed calls of a bucket (rank 0's view)."""
        st = self.buckets[index]
        a, b = st.stats[0][:2].tolist()
        a += st.totals[0]
        b += st.totals[1]
        return (a / b) ** 0.5 if b > 0 else 0.0

    def wire_bytes(self, st: BucketState, compressed: bool) -> int:
        """Bytes this rank stores into *other* ranks' memory for one call on this bucket."""
        w = self.world
        per_elem = (0.5 + 2.0 / 64.0) if compressed else st.grad_dtype.itemsize
        return int(2 * st.n * per_elem * (w - 1) / w)

    def state_dict(self) -> dict:
        out = {}
        for idx, st in self.buckets.items():
            out[idx] = {
                "n": st.n, "epoch": st.epoch, "prev": st.prev[0].clone(), "curr": st.curr[0].clone(),
                "ef": None if st.ef[0] is None else st.ef[0].clone(),
                "ef2": None if st.ef2[0] is None else st.ef2[0].clone(),
            }
        return out

    def load_state_dict(self, sd: dict) -> None:
        for idx, d in sd.items():
            st = self.buckets.get(idx)
            if st is None or st.n != d["n"]:
                continue
            st.prev[0].copy_(d["prev"])
            st.curr[0].copy_(d["curr"])
            if st.ef[0] is not None and d.get("ef") is not None:
                st.ef[0].copy_(d["ef"])
            if st.ef2[0] is not None and d.get("ef2") is not None:
                st.ef2[0].copy_(d["ef2"])
