"""Compressed collectives for fully-sharded data parallelism (FSDP2 ``fully_shard``).

* :class:`NangilaReduceScatter` — the gradient reduce-scatter as one fused kernel: every rank
  block-INT4 quantizes the whole unsharded gradient (stochastic rounding, optional error feedback),
  stores each shard's chunks straight into the owning rank's slots over NVLink, and the owner
  dequantize-accumulates its shard. Each rank receives only its shard: (W-1)/W * 0.53 bytes per
  element cross the links instead of (W-1)/W * 2.
* :class:`NangilaAllGather` — the parameter all-gather with INT8 (or INT4) block quantization fused in:
  shards are quantized once, pushed to every rank, and dequantized straight into the unsharded
  buffer.

``apply_nangila_fsdp(module)`` installs both on every ``FSDPModule`` under ``module``.

The reference's experimental FSDP1 hook (python/nangila/fsdp.py:80-236) instead all-gathers the full
INT4 gradient of every rank, reconstructs all W copies on every rank and slices out the shard, and
leaves the parameter all-gather alone.

By default the momentum predictor is not used here: the sender must know the prediction to subtract
it, so the history of the averaged gradient would have to live, full size, on every rank, which is
the memory FSDP exists to avoid (``predictor=True`` buys the reference's behaviour at that price).
Error feedback is optional for the same reason (off by default; stochastic rounding keeps the
quantizer unbiased). All state is per FSDP unit.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .predres_engine import STATUS_MESSAGES, _glue
from .symm import LoopbackArena, SymmArena

try:
    from torch.distributed.fsdp._fully_shard._fsdp_api import AllGather, ReduceScatter
except Exception:  # pragma: no cover - older torch
    AllGather = object  # type: ignore
    ReduceScatter = object  # type: ignore


def _chunk_for(shard: int, per_shard: int = 1024, cap: int = 131072) -> int:
    """Chunk size for a shard: the power of two at or above shard / per_shard in [4096, cap] (every chunk
    costs a flag round trip), halved while the shard would give fewer than 4 chunks, never below 2048."""
    env = os.environ.get("NANGILA_CHUNK")
    if env:
        return int(env)
    c = 4096
    while c < cap and c * per_shard < shard:
        c *= 2
    while c > 2048 and shard < 4 * c:
        c //= 2
    return c


class _Base:
    def __init__(self, arena=None, group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
                 timeout_s: Optional[float] = None):
        self._arena = arena
        self._group = group
        self._device = device
        self.timeout_s = float(os.environ.get("NANGILA_WAIT_TIMEOUT_MS", "2000")) / 1e3 if timeout_s is None else timeout_s
        self._regions: Dict[tuple, dict] = {}
        self._status: Optional[List[torch.Tensor]] = None
        self.launches = 0
        self.fallbacks = 0
        self._glue = None
        # CTAs per launch (NANGILA_FSDP_CTAS; 0: as many as there are chunks, clamped by the launcher to what the device
        # holds at once). The collectives overlap with the layers' compute, so a cap trades their own speed for the SMs
        # they take from it.
        self.ctas = int(os.environ.get("NANGILA_FSDP_CTAS", "0"))

    def _ensure(self, device: torch.device, group: Optional[dist.ProcessGroup]):
        if self._glue is None:
            self._glue = _glue()
        if self._arena is None:
            self._arena = SymmArena(group if group is not None else self._group, device)
        arena = self._arena
        self.world = arena.world
        self.rank = arena.rank
        self.loopback = isinstance(arena, LoopbackArena)
        self.nvr = self.world if self.loopback else 1
        if self._status is None:
            self._status = [torch.zeros(8, dtype=torch.int32, device=device) for _ in range(self.nvr)]
        return arena

    def allocate(self, size: Sequence[int], *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return torch.empty(*size, dtype=dtype, device=device)

    def check_status(self) -> None:
        torch.cuda.synchronize()
        for s in self._status or []:
            w = s.cpu().tolist()
            if w[0] != 0:
                s.zero_()
                raise RuntimeError(f"nangila: fused FSDP collective failed on rank {w[1]} "
                                   f"({STATUS_MESSAGES.get(w[0], 'code %d' % w[0])}); waiting for rank {w[2]}")

    @staticmethod
    def _work_or_none(async_op: bool, tensor: torch.Tensor):
        if not async_op:
            return None
        fut: torch.futures.Future = torch.futures.Future(devices=[tensor.device])
        fut.set_result(tensor)
        return torch._C._distributed_c10d._create_work_from_future(fut)


class _RsUnit:
    """State of one FSDP unit (one sharded parameter group): its own error memory, its own rounding
    counter and, in predictor mode, its own bucket (history, gain controller) in the engine."""

    __slots__ = ("index", "calls", "ef")

    def __init__(self, index: int):
        self.index = index
        self.calls = 0
        self.ef: Optional[List[Optional[torch.Tensor]]] = None


class NangilaReduceScatter(_Base, ReduceScatter):
    """``module.set_custom_reduce_scatter(NangilaReduceScatter())``

    State is kept per FSDP *unit*, never per tensor size: the identical transformer blocks of a model all
    have the same flat size, and sharing an error memory among them would add block i's quantization error
    to block i+1's gradient. A unit is named either explicitly (``for_unit(uid)``, which is what
    :func:`apply_nangila_fsdp` installs on every FSDP module) or by its position among the calls of a
    step, with ``end_step()`` marking the step boundary (the FSDP1 hook's state object does that, as the
    reference's ``step_counter`` did: python/nangila/fsdp.py:50-53). Only the exchange region (symmetric
    memory, a function of the size alone) is shared. The key of the stochastic rounding is
    ``(seed, step + calls of the unit, unit index, rank)``, so it changes every time a unit is reduced
    whether or not anybody advances ``step``.

    ``predictor=True`` selects the prediction-residual form of the reference's FSDP hook
    (python/nangila/fsdp.py:107-236): every rank keeps the two-step history of the unit's *averaged full*
    gradient, subtracts the momentum prediction before quantizing and reconstructs the full mean, of
    which it keeps its shard. That is the fused all-reduce kernel of the DDP path followed by a slice; it
    costs two full-size history buffers per unit on every rank (the memory FSDP otherwise saves) and sends
    twice the bytes of the plain compressed reduce-scatter, so it is off by default.
    """

    def __init__(self, *args, error_feedback: bool = False, stochastic: Optional[bool] = None, seed: int = 42,
                 predictor: bool = False, momentum: float = 0.9, warmup_calls: int = 2, **kw):
        super().__init__(*args, **kw)
        self.error_feedback = error_feedback
        # round to nearest when an error memory removes the bias, stochastic (unbiased) rounding otherwise
        self.stochastic = (not error_feedback) if stochastic is None else stochastic
        self.seed = seed
        self.predictor = predictor
        self.momentum = momentum
        self.warmup_calls = warmup_calls  # predictor mode: exact exchanges per unit that seed the history
        self.step = 0
        self._units: Dict[object, _RsUnit] = {}
        self._cursor: Dict[tuple, int] = {}  # auto-named units: occurrences of each size since the step began
        self._first_uid: object = None
        self._engine = None

    @property
    def units_seen(self) -> int:
        return len(self._units)

    def for_unit(self, uid) -> "_RsUnitView":
        """A reduce-scatter object bound to one FSDP unit (any hashable name)."""
        return _RsUnitView(self, uid)

    def end_step(self) -> None:
        """Marks the end of an optimizer step for callers that name units by call order (FSDP1 hook,
        direct use). Not needed for units named with ``for_unit``."""
        self._cursor.clear()
        self._advance_step()

    def _advance_step(self) -> None:
        self.step += 1
        if self._engine is not None:
            self._engine.end_step()

    def _unit(self, uid, n: int, dtype: torch.dtype) -> _RsUnit:
        if uid is None:
            key = (n, dtype)
            k = self._cursor.get(key, 0)
            self._cursor[key] = k + 1
            if k >= 4096 and (self.error_feedback or self.predictor):
                raise RuntimeError("nangila: NangilaReduceScatter names FSDP units by call order within a step; call "
                                   "end_step() once per optimizer step (NangilaFSDPState.step() does), or install it "
                                   "with apply_nangila_fsdp(), which names the units itself")
            uid = ("auto", n, dtype, k)
        elif self._first_uid is None:
            self._first_uid = uid
        elif uid == self._first_uid:
            self._advance_step()  # the first unit of a backward pass is back: a new step has begun
        unit = self._units.get(uid)
        if unit is None:
            unit = self._units[uid] = _RsUnit(len(self._units))
        return unit

    def reduce(self, outputs: List[torch.Tensor], inputs: List[torch.Tensor], scale: float, unit=None) -> None:
        """Core call: one tensor per emulated rank (one in a real group)."""
        n = inputs[0].numel()
        arena = self._ensure(inputs[0].device, None)
        u = self._unit(unit, n, inputs[0].dtype)
        u.calls += 1
        if self.predictor:
            return self._reduce_predicted(u, outputs, inputs, scale)
        key = (n, inputs[0].dtype)
        st = self._regions.get(key)
        if st is None:
            # Phase 2 has one task per chunk of this rank's shard: the chunk size is chosen so that those tasks fill
            # the CTAs the device holds at once in whole waves (256 chunks of 64 K elements per shard left more than
            # half of them idle in that phase)
            env = os.environ.get("NANGILA_CHUNK")
            resident = max(1, int(self._glue.predres_resident_ctas()) // self.nvr)
            chunk = int(env) if env else int(self._glue.predres_chunk_elems(n // self.world, resident))
            total, r1, f1, nchunks = self._glue.rs_region_layout(n, self.world, chunk)
            st = dict(region=arena.allocate(int(total)), r1=r1, f1=f1, nchunks=nchunks, chunk=chunk, epoch=0)
            self._regions[key] = st
        if self.error_feedback and u.ef is None:
            u.ef = [torch.zeros(n, dtype=torch.bfloat16, device=inputs[0].device) for _ in range(self.nvr)]
        ef = u.ef if u.ef is not None else [None] * self.nvr
        st["epoch"] += 1
        self.launches += 1
        cps = st["nchunks"] // self.world
        self._glue.rs_launch(inputs, outputs, ef, self._status, st["region"].ptrs, st["r1"], st["f1"], st["nchunks"],
                             0 if self.loopback else self.rank, st["chunk"], self.stochastic, st["epoch"], self.seed,
                             self.step + u.calls, u.index, scale, self.timeout_s,
                             max(1, min(cps * self.world, self.ctas) if self.ctas > 0 else cps * self.world))

    def _reduce_predicted(self, u: _RsUnit, outputs: List[torch.Tensor], inputs: List[torch.Tensor], scale: float) -> None:
        from .predres_engine import PredResEngine

        if self._engine is None:
            self._engine = PredResEngine(self._arena, inputs[0].device, momentum=self.momentum,
                                         error_feedback=self.error_feedback, stochastic=self.stochastic, seed=self.seed,
                                         timeout_s=self.timeout_s, use_side_stream=False)
            self._engine.status = self._status  # one status block for every kernel of this object
        self._engine.reduce(u.index, inputs, compressed=u.calls > self.warmup_calls, step=self.step + u.calls)
        self.launches += 1
        shard = inputs[0].numel() // self.world
        mul = scale * self.world  # the engine leaves the mean in `inputs`
        for v, out in enumerate(outputs):
            r = v if self.loopback else self.rank
            piece = inputs[v].view(-1)[r * shard:(r + 1) * shard].view_as(out)
            if mul == 1.0:
                out.copy_(piece)
            else:
                torch.mul(piece, mul, out=out)

    def _call(self, uid, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group: dist.ProcessGroup, op,
              async_op: bool = False):
        self._ensure(input_tensor.device, group)
        n = input_tensor.numel()
        shard = n // self.world
        op_name = str(op).upper()
        usable = (input_tensor.is_cuda and input_tensor.is_contiguous() and output_tensor.is_contiguous()
                  and n % self.world == 0 and shard % 8 == 0 and output_tensor.dtype == input_tensor.dtype
                  and input_tensor.dtype in (torch.float32, torch.bfloat16, torch.float16)
                  and ("AVG" in op_name or "SUM" in op_name) and "PREMUL" not in op_name
                  and input_tensor.data_ptr() % 16 == 0 and output_tensor.data_ptr() % 16 == 0)
        if not usable:
            self.fallbacks += 1
            return dist.reduce_scatter_tensor(output_tensor, input_tensor, op=op, group=group, async_op=async_op)
        scale = 1.0 / self.world if "AVG" in op_name else 1.0
        self.reduce([output_tensor], [input_tensor.view(-1)], scale, unit=uid)
        return self._work_or_none(async_op, output_tensor)

    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group: dist.ProcessGroup, op,
                 async_op: bool = False):
        return self._call(None, output_tensor, input_tensor, group, op, async_op)


class _RsUnitView(ReduceScatter):
    """What FSDP2 calls for one module: forwards to the shared :class:`NangilaReduceScatter` with the
    unit's name, so that the unit gets its own error memory, rounding counter and predictor state."""

    def __init__(self, parent: NangilaReduceScatter, uid):
        self.parent = parent
        self.uid = uid

    def allocate(self, size: Sequence[int], *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return self.parent.allocate(size, dtype=dtype, device=device)

    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group: dist.ProcessGroup, op,
                 async_op: bool = False):
        return self.parent._call(self.uid, output_tensor, input_tensor, group, op, async_op)


class NangilaAllGather(_Base, AllGather):
    """``module.set_custom_all_gather(NangilaAllGather(bits=8))``"""

    def __init__(self, *args, bits: int = 8, **kw):
        super().__init__(*args, **kw)
        if bits not in (4, 8):
            raise ValueError("quantize_bits for the parameter all-gather must be 8 or 4")
        self.bits = bits

    def gather(self, outputs: List[torch.Tensor], inputs: List[torch.Tensor]) -> None:
        shard = inputs[0].numel()
        arena = self._ensure(inputs[0].device, None)
        key = (shard, inputs[0].dtype)
        st = self._regions.get(key)
        if st is None:
            chunk = _chunk_for(shard)
            total, r, f = self._glue.ag_region_layout(shard, self.world, chunk, self.bits)
            st = dict(region=arena.allocate(int(total)), r=r, f=f, chunk=chunk, epoch=0)
            self._regions[key] = st
        st["epoch"] += 1
        self.launches += 1
        cps = (shard + st["chunk"] - 1) // st["chunk"]
        self._glue.ag_launch(inputs, outputs, self._status, st["region"].ptrs, st["r"], st["f"],
                             0 if self.loopback else self.rank, st["chunk"], self.bits, st["epoch"], self.timeout_s,
                             max(1, min(cps * (self.world + 1), self.ctas) if self.ctas > 0 else cps * (self.world + 1)))

    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group: dist.ProcessGroup,
                 async_op: bool = False):
        self._ensure(input_tensor.device, group)
        shard = input_tensor.numel()
        usable = (input_tensor.is_cuda and input_tensor.is_contiguous() and output_tensor.is_contiguous()
                  and shard % 8 == 0 and output_tensor.numel() == shard * self.world
                  and output_tensor.dtype == input_tensor.dtype
                  and input_tensor.dtype in (torch.float32, torch.bfloat16, torch.float16)
                  and input_tensor.data_ptr() % 16 == 0 and output_tensor.data_ptr() % 16 == 0)
        if not usable:
            self.fallbacks += 1
            return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)
        self.gather([output_tensor.view(-1)], [input_tensor.view(-1)])
        return self._work_or_none(async_op, output_tensor)


def apply_nangila_fsdp(module: torch.nn.Module, *, compress_gradients: bool = True, quantize_parameters: bool = True,
                       parameter_bits: int = 8, error_feedback: bool = False, predictor: bool = False):
    """Install the fused collectives on every FSDP2 module below ``module``. Returns
    ``(reduce_scatter, all_gather)`` (either may be ``None``). One object of each kind serves all modules
    (shared exchange regions, counters and status); every module gets its own view of the reduce-scatter,
    so error memory, rounding counter and predictor state are per FSDP unit."""
    from torch.distributed.fsdp import FSDPModule

    rs = NangilaReduceScatter(error_feedback=error_feedback, predictor=predictor) if compress_gradients else None
    ag = NangilaAllGather(bits=parameter_bits) if quantize_parameters else None
    for uid, m in enumerate(mm for mm in module.modules() if isinstance(mm, FSDPModule)):
        if isinstance(m, FSDPModule):
            if rs is not None:
                m.set_custom_reduce_scatter(rs.for_unit(uid))
            if ag is not None:
                m.set_custom_all_gather(ag)
    return rs, ag
