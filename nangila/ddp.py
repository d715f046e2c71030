"""Nangila DDP communication hook.

Usage (same as the reference, python/nangila/ddp.py:15-33)::

    from nangila.ddp import register_nangila_hook
    model = DDP(model, device_ids=[local_rank])
    hook = register_nangila_hook(model, threshold=0.95, warmup_steps=100)
    for batch in loader:
        loss = model(batch); loss.backward(); optimizer.step()
        hook.step()

What happens per gradient bucket:

* CUDA buckets: one fused sm_100a kernel launch on a side stream does predict-subtract, error
  feedback, block-INT4 quantization, the exchange over NVLink peer memory, dequantize-accumulate and
  the history update (``nangila.parallel.predres_engine``). During the first ``warmup_steps`` steps
  the same kernel runs in its uncompressed mode (exact mean). DGC and PowerSGD buckets take their own
  fused kernels (``nangila.parallel.dgc_engine`` / ``powersgd_engine``).
* CPU buckets (gloo): the C++ core compresses to packets, packets are all-gathered, every rank
  reconstructs and averages (the reference's transport, ddp.py:286-347), with the warm-up
  all-reduce done as SUM + divide because gloo has no AVG.

Differences from the reference that a user can observe: the keyword arguments really reach the
core (the reference built a config and then dropped it, ddp.py:142-151); compression starts at
``warmup_steps`` (the reference's core kept its own 1000+100-step warm-up); bucket state is keyed by
``bucket.index()`` instead of a call counter (ddp.py:180-181); the predictor-hash exchange carries
the 64-bit hash as two 32-bit halves (ddp.py:392 overflowed a signed 64-bit tensor).
"""


import os
import warnings
from typing import Any, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

from ._C import CompressorType, MetricsCollector, NangilaConfig, NangilaHook, SyncMode  # noqa: F401  (CompressorType is re-exported)
from .utils.liveness import LivenessMixin

NANGILA_AVAILABLE = True

try:
    from torch.distributed import GradBucket
except ImportError:  # pragma: no cover
    GradBucket = Any

try:  # the C++ comm-hook class lives in the torch glue
    from ._cuda import NangilaDDPHook as _CppHookBase  # type: ignore
    CPP_HOOK_AVAILABLE = True
except Exception:  # pragma: no cover - glue not built
    _CppHookBase = None
    CPP_HOOK_AVAILABLE = False


if CPP_HOOK_AVAILABLE:

    class NangilaCppHook(_CppHookBase):
        """The C++ DDP hook as a comm-hook callable: ``ddp.register_comm_hook(None, NangilaCppHook(n, warmup))``.

        All per-bucket work (state lookup, stream hand-over, the fused kernel launch, the future) is
        C++; this subclass only supplies the annotated ``__call__`` DDP insists on and the symmetric
        memory the first time a bucket is seen. Same constructor as the reference's
        ``NangilaCppHook(num_layers, warmup_steps)`` (nangila_ddp/src/bindings.cpp:18-60); it handles
        the prediction-residual compressor on CUDA buckets.
        """

        def __init__(self, num_layers: int = 1000, warmup_steps: int = 100, process_group: Optional[Any] = None, *,
                     momentum: float = 0.9, error_feedback: bool = True, stochastic: Optional[bool] = None, seed: int = 42,
                     reserve_bytes: Optional[int] = None):
            super().__init__(int(num_layers), int(warmup_steps))
            if stochastic is None:  # round to nearest when the error memory is there to remove the bias
                stochastic = not error_feedback
            self.configure(momentum=momentum, error_feedback=error_feedback, stochastic=stochastic, seed=seed)
            self.process_group = process_group
            self._reserve_bytes = reserve_bytes
            self._arena = None
            self._regions: List[Any] = []
            self.__name__ = "nangila_cpp_hook"
            self.__qualname__ = "nangila_cpp_hook"

        def _attach(self, device: torch.device) -> None:
            from .parallel.symm import SymmArena

            group = self.process_group or dist.distributed_c10d._get_default_group()
            self._arena = SymmArena(group, device)
            if self._reserve_bytes:
                self._arena.reserve(int(self._reserve_bytes))

            def allocate(nbytes: int) -> List[int]:
                region = self._arena.allocate(int(nbytes))
                self._regions.append(region)  # keeps the mapping alive
                return [int(p) for p in region.ptrs]

            self.attach(self._arena.rank, self._arena.world, allocate)

        def __call__(self, state: Any, bucket: GradBucket) -> torch.futures.Future[torch.Tensor]:
            if self._arena is None:
                self._attach(bucket.buffer().device)
            return self.run(bucket)

        def step(self) -> None:
            """Call once per optimizer step. The kernels' per-bucket statistics are summed over the process
            group (on the exchange stream, off the critical path) before the gain controller reads them, so
            every rank derives the same prediction gains; the kernel is told that the gains are uniform and
            applies its own value in the reconstruction, which is only right if they are."""
            stats = self.stats_tensor()
            if stats is not None and self._arena is not None and self._arena.world > 1:
                with torch.cuda.stream(torch.cuda.ExternalStream(self.stream_ptr(), device=stats.device)):
                    dist.all_reduce(stats, group=self._arena.group)
            super().step()

else:  # pragma: no cover
    NangilaCppHook = None

_LOG = os.environ.get("NANGILA_LOG", "warn").lower()


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _log(msg: str) -> None:
    if _LOG in ("info", "debug") and (not dist.is_initialized() or dist.get_rank() == 0):
        print(f"[nangila] {msg}", flush=True)


def _warn_if_advanced_ddp_options(compressor_type: int, dgc_sparsity: float, power_sgd_rank: int) -> None:
    if int(compressor_type) != 0 or dgc_sparsity != 0.999 or power_sgd_rank != 1:
        warnings.warn(
            "Non-default DDP compressor tuning options are available for compatibility but are "
            "excluded from the Nangila v0.1 stable support contract.",
            stacklevel=3,
        )


def _validate_sync_mode(sync_mode: Any) -> int:
    try:
        m = int(sync_mode)
    except Exception:
        raise ValueError(f"Invalid sync_mode {sync_mode!r}. Use SyncMode.ASYNC (0), ALWAYS (1), or PERIODIC (2)")
    if m not in (0, 1, 2):
        raise ValueError(f"Invalid sync_mode {sync_mode!r}. Use SyncMode.ASYNC (0), ALWAYS (1), or PERIODIC (2)")
    return m


class NangilaDDPHook(LivenessMixin):
    """DDP communication hook (``ddp_model.register_comm_hook(None, hook)``).

    Args mirror the reference (ddp.py:100-112). ``num_layers`` is only the size of the all-Driver
    mask of the host-side state machine; device state is created per bucket on first use.
    Extra keyword-only knobs: ``momentum``, ``error_feedback``, ``stochastic`` (rounding of the INT4 codes;
    default: round to nearest with error feedback, stochastic without), ``dgc_momentum`` (momentum correction factor of the DGC path).
    """

    def __init__(
        self,
        process_group: Optional[Any] = None,
        threshold: float = 0.95,
        warmup_steps: int = 100,
        num_layers: int = 1000,
        sync_mode: int = 2,
        enable_gpu_native: bool = False,
        *,
        compressor_type: int = 0,
        dgc_sparsity: float = 0.999,
        power_sgd_rank: int = 1,
        momentum: float = 0.9,
        error_feedback: bool = True,
        stochastic: Optional[bool] = None,
        dgc_momentum: float = 0.9,
        total_numel: Optional[int] = None,
        mask: Any = None,
    ):
        _warn_if_advanced_ddp_options(compressor_type, dgc_sparsity, power_sgd_rank)
        self.process_group = process_group or dist.distributed_c10d._get_default_group()
        self.threshold = threshold
        self.warmup_steps = int(warmup_steps)
        self.step_count = 0
        self.sync_mode = _validate_sync_mode(sync_mode)
        self.enable_gpu_native = enable_gpu_native
        self.compressor_type = int(compressor_type)
        self.dgc_sparsity = float(dgc_sparsity)
        self.power_sgd_rank = int(power_sgd_rank)
        self.momentum = float(momentum)
        self.error_feedback = error_feedback
        # Rounding of the INT4 codes: with error feedback the default is round-to-nearest (half the noise power;
        # the error memory removes the bias), without it stochastic rounding (unbiased). NANGILA_STOCHASTIC=0/1 overrides.
        if stochastic is None:
            stochastic = not error_feedback
        self.stochastic = bool(int(os.environ.get("NANGILA_STOCHASTIC", int(bool(stochastic)))))
        self.dgc_momentum = float(dgc_momentum)
        self.config = NangilaConfig(
            momentum=momentum, threshold=threshold, warmup_steps=self.warmup_steps, shadow_run_steps=0,
            compressor_type=self.compressor_type, dgc_sparsity=dgc_sparsity, power_sgd_rank=power_sgd_rank,
        )
        self.__name__ = "nangila_hook"
        self.__qualname__ = "nangila_hook"
        # Topology mask (Sculptor output): Passenger parameters are not exchanged at all; their averaged gradient is
        # synthesised from their Driver's as alpha * g_driver + beta (nangila-core/src/reconstructor.rs:96-152).
        # Layer ids are positions in ``ddp_model.parameters()``.
        mask_bytes, self._passengers = self._parse_mask(mask)
        self._masked_values: Dict[int, torch.Tensor] = {}   # reconstructed Driver gradients of this iteration
        self._masked_todo: List[tuple] = []                 # (passenger view, source id, alpha, beta)
        self._masked_futures: List[tuple] = []              # (future, tensor) completed after the synthesis
        self.passenger_elements = 0                         # elements synthesised instead of exchanged (per iteration)
        self.hook = (NangilaHook(mask_bytes, self.config) if self._passengers
                     else NangilaHook.all_drivers(max(int(num_layers), 1), self.config))
        self.layer_counter = 0
        self.total_original_bytes = 0
        self.total_compressed_bytes = 0
        self.world_size = dist.get_world_size(self.process_group)
        self.rank = dist.get_rank(self.process_group)
        self._total_numel = total_numel
        self._engine = None          # PredResEngine, created on the first CUDA bucket
        self._dgc_engine = None
        self._psgd_engine = None
        self._bucket_calls = 0
        self._force_uncompressed = False
        self.prefer_cpp = False      # set by register_nangila_hook(prefer_cpp=True)
        self.recovered_failures = 0  # buckets that fell back to an exact all-reduce after a rejected packet
        self._exact_until_step = 0   # buckets go through a plain all-reduce before this step (after a resume)
        self._pending_state: Dict[int, dict] = {}  # restored device state, applied when its bucket appears
        self._packet_filter = None   # tests: callable(step, layer_id, src_rank, bytes) -> bytes
        self._cpp = None             # NangilaCppHook once the first CUDA bucket went through it
        self._native = False         # the C++ hook sits on DDP's reducer itself: __call__ is never reached
        self._param_ids: Dict[int, int] = {}
        # production counters (Prometheus text / JSON): fed once per step from the byte counters of whichever
        # path handled the buckets (reference: nangila-core/src/metrics.rs:12-232)
        self._metrics = MetricsCollector()
        self._metrics_bytes = (0, 0)
        self._metrics_failures = 0
        _log(f"DDP hook: sync_mode={SyncMode(self.sync_mode)!r} compressor={self.compressor_type} "
             f"warmup={self.warmup_steps} world={self.world_size}")

    # ------------------------------------------------------------------------------------------
    def __call__(self, state: Any, bucket: GradBucket) -> torch.futures.Future[torch.Tensor]:
        self.layer_counter += 1
        tensor = bucket.buffer()
        try:
            index = int(bucket.index())
        except Exception:
            index = self.layer_counter - 1
        if self.step_count < self._exact_until_step:
            return self._run_plain_allreduce(tensor)
        if self._passengers:
            return self._run_masked(bucket, tensor, index)
        if tensor.is_cuda:
            if self.prefer_cpp and CPP_HOOK_AVAILABLE and self.compressor_type == 0:
                return self._run_cpp(bucket, tensor)
            return self._run_cuda(bucket, tensor, index)
        return self._run_cpu(bucket, tensor, index)

    def _run_plain_allreduce(self, tensor: torch.Tensor) -> torch.futures.Future:
        """Exact mean through the process group, touching no compressor state. Used for the first step
        after a resume: a new DDP instance lays its buckets out in construction order for one
        iteration and only then switches to the gradient-ready order the saved state belongs to."""
        world = self.world_size
        nbytes = tensor.numel() * tensor.element_size()
        self.total_original_bytes += nbytes
        self.total_compressed_bytes += nbytes
        work = dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.process_group, async_op=True)
        return work.get_future().then(lambda f: f.value()[0].div_(world))

    def _apply_pending(self, index: int, target: dict) -> None:
        """Copy a restored bucket state (history, error memory) into freshly created device state."""
        saved = self._pending_state.pop(index, None)
        if saved is None or int(saved.get("n", -1)) != int(target["n"]):
            return
        for k in ("prev", "curr", "ef", "ef2"):
            src, dst = saved.get(k), target.get(k)
            if isinstance(src, torch.Tensor) and isinstance(dst, torch.Tensor) and src.numel() == dst.numel():
                dst.copy_(src.to(dst.dtype))

    def _make_cpp(self) -> "NangilaCppHook":
        cpp = self._cpp = NangilaCppHook(
            1, self.warmup_steps, self.process_group, momentum=self.momentum, error_feedback=self.error_feedback,
            stochastic=self.stochastic,
            reserve_bytes=(int(self._total_numel * 1.02) + (8 << 20)) if self._total_numel else None)
        cpp.fast_forward(self.step_count)
        self.hook.set_gpu_mode(True)
        return cpp

    def install_native(self, ddp_model: DDP) -> None:
        """Put the C++ hook on DDP's reducer as a C++ communication hook: every bucket then goes from the reducer
        to the fused kernel launch without entering the interpreter (``__call__`` of this object is never reached).
        What this class does per bucket in Python moves to ``step()``: the pause flag of Safe Mode / recovery is
        handed over once per step, and the device status is checked once per step (``sync_mode`` ALWAYS) or every
        16th step (PERIODIC). Only for the prediction-residual compressor on CUDA parameters without a topology mask."""
        device = next(p for p in ddp_model.parameters() if p.requires_grad).device
        cpp = self._make_cpp()
        cpp._attach(device)
        cpp.register_native(ddp_model.reducer)
        self._native = True

    def _run_cpp(self, bucket: GradBucket, tensor: torch.Tensor) -> torch.futures.Future:
        """Prediction-residual compressor through the C++ hook: everything per bucket is native."""
        cpp = self._cpp
        if cpp is None:
            cpp = self._make_cpp()
        cpp.set_paused(self._force_uncompressed or self.hook.is_paused())
        if self._pending_state:
            index = int(bucket.index())
            if index in self._pending_state:
                if cpp._arena is None:
                    cpp._attach(tensor.device)
                cpp.ensure_bucket(bucket)
                self._apply_pending(index, cpp.bucket_state(index))
        fut = cpp(None, bucket)
        self._bucket_calls += 1
        if self.sync_mode == 1 or (self.sync_mode == 2 and self._bucket_calls % 100 == 0):
            self._check_device_status()
        return fut

    @staticmethod
    def _parse_mask(mask: Any) -> tuple:
        if mask is None:
            return None, {}
        mask_bytes = bytes(mask.to_bytes()) if hasattr(mask, "to_bytes") else bytes(mask)
        from ._C import TopologyMask

        passengers = {int(lid): (int(source), float(alpha), float(beta))
                      for lid, source, alpha, beta in TopologyMask.from_bytes(mask_bytes).passengers()}
        return mask_bytes, passengers

    def set_mask(self, mask: Any) -> int:
        """Apply a topology mask (``TopologyMask`` or its bytes) to a hook that is already registered, e.g. at the end
        of a Sculptor calibration that ran during warm-up. Call it between steps, on every rank, before compression
        starts: the host-side predictor state of the old mask is dropped. Returns the number of Passengers."""
        mask_bytes, passengers = self._parse_mask(mask)
        self._passengers = passengers
        if passengers:
            new = NangilaHook(mask_bytes, self.config)
            while new.current_step() < self.hook.current_step():
                new.step()
            new.set_gpu_mode(self.hook.gpu_mode())
            self.hook = new
        return len(passengers)

    # ---- buckets under a topology mask ---------------------------------------------------------------
    def _run_masked(self, bucket: GradBucket, tensor: torch.Tensor, index: int) -> torch.futures.Future:
        """A bucket whose parameters may be Passengers. Driver parameters are exchanged as usual: on CUDA every
        maximal run of consecutive Driver parameters goes through the fused kernel as a bucket of its own
        (own history and error memory), on CPU every Driver parameter goes through the packet path.
        Passenger parameters cost nothing on the wire. Their Driver may sit in a bucket that is reduced
        later, so the synthesis is queued when the last bucket of the iteration arrives, and every bucket's
        future completes after it."""
        grads = bucket.gradients()
        params = bucket.parameters()
        base = tensor.storage_offset()
        esize = tensor.element_size()
        segs = []   # (layer id, first element, elements, gradient view)
        for prm, g in zip(params, grads):
            lid = self._param_ids.get(id(prm), -1)
            segs.append((lid, g.storage_offset() - base, g.numel(), g))
        is_cuda = tensor.is_cuda
        compressing = self.compressing
        if is_cuda:
            engine = self._ensure_engine(tensor.device)
            run_no = 0
            i = 0
            while i < len(segs):
                lid, off, numel, g = segs[i]
                if lid in self._passengers and numel > 0:
                    i += 1
                    continue
                # a run of Drivers; a Passenger whose successor would start misaligned is carried along as a Driver
                j, end = i, off + numel
                while j + 1 < len(segs):
                    nlid, noff, nnum, _ = segs[j + 1]
                    if nlid in self._passengers:
                        after = noff + nnum
                        stop_ok = (tensor.data_ptr() + after * esize) % 16 == 0 or j + 2 >= len(segs)
                        if stop_ok:
                            break
                    j += 1
                    end = noff + nnum
                if (tensor.data_ptr() + off * esize) % 16 != 0:   # cannot start a kernel range here: exact all-reduce
                    piece = tensor[off:end]
                    dist.all_reduce(piece, group=self.process_group)
                    piece.div_(self.world_size)
                else:
                    engine.reduce(20_000_000 + index * 4096 + run_no, [tensor[off:end]], compressed=compressing and self.compressor_type == 0,
                                  step=self.step_count)
                nb = (end - off) * esize
                self.total_original_bytes += nb
                self.total_compressed_bytes += int((end - off) * (0.5 + 2.0 / 64.0)) if compressing else nb
                for k in range(i, j + 1):
                    self._masked_values[segs[k][0]] = segs[k][3]
                run_no += 1
                i = j + 1
        else:
            for lid, off, numel, g in segs:
                if lid in self._passengers:
                    continue
                if self.step_count < self.warmup_steps or self.hook.is_paused():
                    dist.all_reduce(g, group=self.process_group)
                    g.div_(self.world_size)
                    if self.step_count + 2 >= self.warmup_steps:
                        self.hook.update(lid, g.detach().float().contiguous().numpy().reshape(-1))
                    nb = g.numel() * g.element_size()
                    self.total_original_bytes += nb
                    self.total_compressed_bytes += nb
                else:
                    flat = g.detach().float().contiguous().numpy().reshape(-1)
                    averaged = self._exchange_cpu(lid, flat, g.device)
                    g.copy_(torch.from_numpy(averaged).view_as(g).to(g.dtype))
                self._masked_values[lid] = g
        for lid, off, numel, g in segs:
            if lid in self._passengers and lid not in self._masked_values:
                source, alpha, beta = self._passengers[lid]
                self._masked_todo.append((g, source, alpha, beta))
                self.total_original_bytes += numel * esize
        stream = self._engine.stream if (is_cuda and self._engine is not None) else None
        fut: torch.futures.Future = torch.futures.Future(devices=[tensor.device]) if is_cuda else torch.futures.Future()
        self._masked_futures.append((fut, tensor))
        if bucket.is_last():
            ctx = torch.cuda.stream(stream) if stream is not None else _NullContext()
            with ctx:
                count = 0
                for g, source, alpha, beta in self._masked_todo:
                    src = self._masked_values.get(source)
                    if src is None or src.numel() != g.numel():
                        raise RuntimeError(f"nangila: Passenger gradient needs Driver {source}, which was not reduced in this iteration")
                    torch.mul(src.view_as(g), alpha, out=g)
                    if abs(beta) > 1e-8:
                        g.add_(beta)
                    count += g.numel()
                self.passenger_elements = count
                for f, t in self._masked_futures:
                    f.set_result(t)
            self._masked_todo.clear()
            self._masked_futures.clear()
            self._masked_values.clear()
        self._bucket_calls += 1
        if is_cuda and (self.sync_mode == 1 or (self.sync_mode == 2 and self._bucket_calls % 100 == 0)):
            self._check_device_status()
        return fut

    @property
    def compressing(self) -> bool:
        return (self.step_count >= self.warmup_steps and not self._force_uncompressed
                and not self.hook.is_paused())

    # ---- CUDA path -----------------------------------------------------------------------------
    def _ensure_engine(self, device: torch.device):
        if self._engine is None:
            from .parallel.predres_engine import PredResEngine
            from .parallel.symm import SymmArena

            arena = SymmArena(self.process_group, device)
            if self._total_numel:
                # room for every bucket's exchange region plus flags and alignment slack
                arena.reserve(int(self._total_numel * 1.02) + (8 << 20))
            self._engine = PredResEngine(arena, device, momentum=self.momentum, error_feedback=self.error_feedback,
                                         stochastic=self.stochastic)
            self.hook.set_gpu_mode(True)
        return self._engine

    def _run_cuda(self, bucket: GradBucket, tensor: torch.Tensor, index: int) -> torch.futures.Future:
        engine = self._ensure_engine(tensor.device)
        compressing = self.compressing
        ctype = self.compressor_type
        if compressing and ctype == 1:
            fut = self._run_cuda_dgc(bucket, tensor, index)
        elif compressing and ctype == 2:
            fut = self._run_cuda_powersgd(bucket, tensor, index)
        else:
            if index in self._pending_state:
                bs = engine.bucket_state(index, [tensor])
                self._apply_pending(index, {"n": bs.n, "prev": bs.prev[0], "curr": bs.curr[0], "ef": bs.ef[0], "ef2": bs.ef2[0]})
            st = engine.reduce(index, [tensor], compressed=compressing and ctype == 0, step=self.step_count)
            nbytes = tensor.numel() * tensor.element_size()
            self.total_original_bytes += nbytes
            self.total_compressed_bytes += (int(tensor.numel() * (0.5 + 2.0 / 64.0)) if compressing else nbytes)
            fut = self._stream_future(engine.stream, tensor)
        self._bucket_calls += 1
        if self.sync_mode == 1 or (self.sync_mode == 2 and self._bucket_calls % 100 == 0):
            self._check_device_status()
        return fut

    @staticmethod
    def _stream_future(stream: Optional[torch.cuda.Stream], tensor: torch.Tensor) -> torch.futures.Future:
        # Completing the future while the exchange stream is current records the dependency, so
        # whoever waits on it (DDP's finalize) orders its stream after the kernel without a host sync.
        fut: torch.futures.Future = torch.futures.Future(devices=[tensor.device])
        if stream is not None:
            with torch.cuda.stream(stream):
                fut.set_result(tensor)
        else:
            fut.set_result(tensor)
        return fut

    def _run_cuda_dgc(self, bucket, tensor, index):
        if self._dgc_engine is None:
            from .parallel.dgc_engine import DGCEngine

            self._dgc_engine = DGCEngine(self._engine.arena, tensor.device, sparsity=self.dgc_sparsity,
                                         momentum=self.dgc_momentum, stream=self._engine.stream)
        k = self._dgc_engine.reduce(index, tensor)
        self.total_original_bytes += tensor.numel() * tensor.element_size()
        self.total_compressed_bytes += k * 8
        return self._stream_future(self._engine.stream, tensor)

    def _run_cuda_powersgd(self, bucket, tensor, index):
        if self._psgd_engine is None:
            from .parallel.powersgd_engine import PowerSGDEngine

            self._psgd_engine = PowerSGDEngine(self._engine.arena, tensor.device, rank=self.power_sgd_rank,
                                               stream=self._engine.stream, group=self.process_group,
                                               exact_engine=self._engine)
        sent = self._psgd_engine.reduce(index, bucket, tensor)
        self.total_original_bytes += tensor.numel() * tensor.element_size()
        self.total_compressed_bytes += sent
        return self._stream_future(self._engine.stream, tensor)

    def _check_device_status(self) -> None:
        if self._engine is None and self._cpp is None:
            return
        try:
            if self._cpp is not None:
                self._cpp.check_status()
            if self._engine is not None:
                self._engine.check_status()
        except RuntimeError:
            # leave the hook usable: the next buckets go through the uncompressed mode and re-seed
            # the history on every rank (FORCE_SYNC semantics of the packet protocol)
            self._force_uncompressed = True
            self._metrics.record_fallback()
            for lid in range(min(10, self.hook.get_stats()["num_drivers"])):
                self.hook.trigger_recovery(lid)
            raise

    # ---- CPU path (gloo) -------------------------------------------------------------------------
    def _run_cpu(self, bucket: GradBucket, tensor: torch.Tensor, index: int) -> torch.futures.Future:
        world = self.world_size
        layer_id = index
        if self.step_count < self.warmup_steps or self.hook.is_paused():
            work = dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.process_group, async_op=True)
            result: torch.futures.Future = torch.futures.Future()
            seed_history = self.step_count + 2 >= self.warmup_steps

            def _done(_):
                tensor.div_(world)
                if seed_history:
                    self.hook.update(layer_id, tensor.detach().float().contiguous().numpy().reshape(-1))
                result.set_result(tensor)

            work.get_future().then(_done)
            nbytes = tensor.numel() * tensor.element_size()
            self.total_original_bytes += nbytes
            self.total_compressed_bytes += nbytes
            return result

        if self.compressor_type == 2:
            return self._run_cpu_per_parameter(bucket, tensor, index)
        flat = tensor.detach().float().contiguous().numpy().reshape(-1)
        averaged = self._exchange_cpu(layer_id % max(self.hook.get_stats()["num_drivers"], 1), flat, tensor.device)
        tensor.copy_(torch.from_numpy(averaged).to(tensor.dtype).view_as(tensor))
        fut: torch.futures.Future = torch.futures.Future()
        fut.set_result(tensor)
        return fut

    def _exchange_cpu(self, layer_id: int, flat: np.ndarray, device: torch.device) -> np.ndarray:
        """Compress -> all-gather packets -> reconstruct every rank's gradient -> mean -> feed the
        mean back to the predictor. ``flat`` may carry a matrix shape; the result is 1-D."""
        world = self.world_size
        self.total_original_bytes += flat.nbytes
        packet = bytes(self.hook.compress(layer_id, flat))
        self.total_compressed_bytes += len(packet)
        local_size = torch.tensor([len(packet)], dtype=torch.long, device=device)
        sizes = [torch.empty_like(local_size) for _ in range(world)]
        dist.all_gather(sizes, local_size, group=self.process_group)
        sizes_i = [int(s.item()) for s in sizes]
        max_size = max(sizes_i)
        padded = torch.zeros(max_size, dtype=torch.uint8, device=device)
        padded[:len(packet)] = torch.frombuffer(bytearray(packet), dtype=torch.uint8)
        gathered = [torch.empty(max_size, dtype=torch.uint8, device=device) for _ in range(world)]
        dist.all_gather(gathered, padded, group=self.process_group)
        filt = self._packet_filter
        acc = np.zeros(flat.size, dtype=np.float64)
        failure: Optional[str] = None
        crc0 = self.hook.crc_failure_count(layer_id)
        for r in range(world):
            data = bytes(gathered[r][:sizes_i[r]].cpu().numpy())
            if filt is not None:  # host-side fault injection (tests): may corrupt, truncate or replace a packet
                data = filt(self.step_count, layer_id, r, data)
            try:
                rec = self.hook.decompress_gathered(layer_id, data)
                if rec.shape[0] != flat.size:
                    raise RuntimeError(f"rank {r} sent {rec.shape[0]} elements, expected {flat.size}")
                if self.hook.crc_failure_count(layer_id) > crc0:
                    # the core substituted its prediction for the damaged payload; that is not this
                    # rank's gradient, so the bucket is exchanged again exactly
                    raise RuntimeError("checksum mismatch")
                acc += rec
            except Exception as exc:  # CRC mismatch, truncated packet, step / layer mismatch, size mismatch
                failure = f"packet of rank {r} for layer {layer_id} rejected: {exc}"
                break
        # A packet may be unreadable on some ranks only (a desynchronised replica): agree on the outcome
        # before choosing the collective that follows.
        bad = torch.tensor([1 if failure else 0], dtype=torch.int32, device=device)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX, group=self.process_group)
        if int(bad.item()):
            # Recovery (FORCE_SYNC semantics of the packet protocol): this bucket is averaged exactly,
            # the averaged gradient re-seeds the predictor on every rank, and the next packet of the
            # layer is sent uncompressed with the FORCE_SYNC flag.
            self.recovered_failures += 1
            warnings.warn(f"nangila: {failure or 'a peer rejected a packet'}; exact all-reduce for this bucket "
                          f"(step {self.step_count})")
            t = torch.from_numpy(np.ascontiguousarray(flat.reshape(-1), dtype=np.float32)).to(device)
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.process_group)
            averaged = (t / world).cpu().numpy().astype(np.float32)
            self.hook.trigger_recovery(layer_id)
            self.hook.update(layer_id, averaged)
            return averaged
        averaged = (acc / world).astype(np.float32)
        self.hook.update(layer_id, averaged)
        return averaged

    def _run_cpu_per_parameter(self, bucket: GradBucket, tensor: torch.Tensor, index: int) -> torch.futures.Future:
        """PowerSGD needs matrix-shaped gradients: every parameter of the bucket with two or more
        dimensions goes through the compressor with its own shape (layer id = position of the
        parameter in the model); the remaining small / 1-D gradients are averaged uncompressed."""
        grads = bucket.gradients()
        try:
            params = bucket.parameters()
        except Exception:
            params = [None] * len(grads)
        nlayers = max(self.hook.get_stats()["num_drivers"], 1)
        raw: List[torch.Tensor] = []
        for pos, g in enumerate(grads):
            if g.dim() >= 2 and g.numel() >= 256:
                prm = params[pos]
                lid = self._param_ids.get(id(prm), (index * 4096 + pos)) % nlayers
                arr = g.detach().float().contiguous().numpy()
                averaged = self._exchange_cpu(lid, arr, g.device)
                g.copy_(torch.from_numpy(averaged).view_as(g).to(g.dtype))
            else:
                raw.append(g)
        if raw:
            flat = torch.cat([g.reshape(-1) for g in raw])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.process_group)
            flat.div_(self.world_size)
            off = 0
            for g in raw:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
            self.total_original_bytes += flat.numel() * flat.element_size()
            self.total_compressed_bytes += flat.numel() * flat.element_size()
        fut: torch.futures.Future = torch.futures.Future()
        fut.set_result(tensor)
        return fut

    # ------------------------------------------------------------------------------------------
    def step(self) -> None:
        """Call after each optimizer step."""
        self._feed_metrics(self._cpp.is_compression_enabled() if self._native else self.compressing)
        self.step_count += 1
        self.layer_counter = 0
        self.hook.step()
        if self._engine is not None:
            self._engine.end_step()
        failure: Optional[BaseException] = None
        if self._native:
            # the step that just ran was the uncompressed one a failure asked for (if any)
            self._force_uncompressed = False
        if self._cpp is not None:
            self._cpp.step()  # sums the kernels' statistics over the group, then adapts the gains
            if self._native and (self.sync_mode == 1 or (self.sync_mode == 2 and self.step_count % 16 == 0)):
                try:
                    self._check_device_status()   # sets _force_uncompressed when a kernel gave up waiting
                except RuntimeError as exc:
                    failure = exc
        if self._force_uncompressed and not self._native:
            self._force_uncompressed = False  # one uncompressed step re-seeded the history everywhere
        if self.step_count % 10 == 0 and self.step_count > self.warmup_steps and _LOG in ("info", "debug"):
            ratio = self.compression_ratio
            if ratio > 1.0:
                _log(f"[Step {self.step_count}] Compression: {self.total_original_bytes / 1e6:.1f} MB -> "
                     f"{self.total_compressed_bytes / 1e6:.1f} MB ({ratio:.1f}x)")
        if self.step_count % 100 == 0 and self.step_count > 0:
            self._verify_predictor_hash()
        if self._native:
            # whatever pauses compression for the coming step (Safe Mode, recovery after a failed exchange, a
            # predictor-hash mismatch) is handed to the reducer-level hook here, once per step
            self._cpp.set_paused(self._force_uncompressed or self.hook.is_paused())
        if failure is not None:
            raise failure
        self.check_peers()   # last: the bookkeeping of the finished step is complete when a missing peer ends the run

    def _byte_counters(self) -> tuple:
        """(bytes the buckets held, bytes that would cross the wire per peer) so far, whichever path ran."""
        if self._cpp is not None:
            native = self._cpp.get_stats()
            return int(native["total_original_bytes"]), int(native["total_compressed_bytes"])
        return int(self.total_original_bytes), int(self.total_compressed_bytes)

    def _feed_metrics(self, compressed: bool) -> None:
        orig, comp = self._byte_counters()
        d_orig, d_comp = orig - self._metrics_bytes[0], comp - self._metrics_bytes[1]
        self._metrics_bytes = (orig, comp)
        if d_orig > 0 or d_comp > 0:
            self._metrics.record_bytes(max(d_orig, 0), max(d_comp, 0))
        self._metrics.record_step(bool(compressed))
        while self._metrics_failures < self.recovered_failures:
            self._metrics.record_fallback()
            self._metrics_failures += 1

    def metrics(self) -> "MetricsCollector":
        """The hook's metrics collector: ``.to_prometheus()`` gives the text exposition format
        (``nangila_compression_ratio``, ``nangila_bytes_saved``, ``nangila_steps_compressed``, ...),
        ``.to_json()`` the same figures as JSON, ``.snapshot()`` a dict."""
        return self._metrics

    def get_stats(self) -> dict:
        stats = dict(self.hook.get_stats())
        stats["step"] = self.step_count
        stats["compression_enabled"] = self.compressing
        stats["total_original_bytes"] = self.total_original_bytes
        stats["total_compressed_bytes"] = self.total_compressed_bytes
        stats["recovered_failures"] = self.recovered_failures
        if self.total_original_bytes > 0:
            stats["overall_compression_ratio"] = self.total_original_bytes / max(self.total_compressed_bytes, 1)
        if self._cpp is not None:
            native = self._cpp.get_stats()
            stats["kernel_launches"] = native["kernel_launches"]
            stats["total_original_bytes"] = native["total_original_bytes"]
            stats["total_compressed_bytes"] = native["total_compressed_bytes"]
            stats["overall_compression_ratio"] = native["compression_ratio"]
            stats["pred_gain_per_bucket"] = dict(native["prediction_gain"])
            stats["cpp_hook"] = True
            if "bucket_kernel_ms" in native:
                stats["bucket_kernel_ms"] = dict(native["bucket_kernel_ms"])
        if self._engine is not None:
            stats["kernel_launches"] = self._engine.launches
            if self._engine.timing:
                stats["bucket_kernel_ms"] = self._engine.kernel_times_ms()
            errs = {}
            for idx, st in self._engine.buckets.items():
                if st.compressed_calls:
                    errs[idx] = self._engine.prediction_error(idx)
            stats["prediction_error_per_bucket"] = errs
            stats["pred_gain_per_bucket"] = {idx: st.pred_gain for idx, st in self._engine.buckets.items()}
        return stats

    def fast_forward(self, to_step: int) -> None:
        """Advance the step counters to ``to_step`` without exchanging anything (all ranks must call
        it at the same point). Used to leave the warm-up early once the history is seeded; the
        reference's examples do the same by stepping the hook in a loop (examples/train_llm.py:29-34,
        nangila_ddp/src/ddp_hook.cpp:60-63)."""
        while self.hook.current_step() < to_step:
            self.hook.step()
        self.step_count = max(self.step_count, int(to_step))
        if self._cpp is not None:
            self._cpp.fast_forward(int(to_step))

    def get_kernel_launches(self) -> int:
        """Number of fused-kernel launches queued by this hook so far on this rank."""
        n = self._cpp.get_kernel_launches() if self._cpp is not None else 0
        for eng in (self._engine, self._dgc_engine, self._psgd_engine):
            if eng is not None:
                n += eng.launches
        return n

    @property
    def compression_ratio(self) -> float:
        if self._cpp is not None:
            return float(self._cpp.get_stats()["compression_ratio"])
        if self.total_compressed_bytes == 0:
            return 1.0
        return self.total_original_bytes / self.total_compressed_bytes

    def state_hash(self) -> int:
        """64-bit hash of the predictor state on this rank (host core, or a device reduction of the
        bucket histories when the CUDA path is active)."""
        if self._cpp is not None and self._cpp.get_stats()["num_buckets"]:
            from .ops.reductions import state_hash as device_hash

            tensors = []
            for idx in sorted(self._cpp.get_stats()["prediction_gain"]):
                st = self._cpp.bucket_state(idx)
                tensors += [st["curr"], st["prev"]]
            return device_hash(tensors, seed=self.step_count)
        if self._engine is not None and self._engine.buckets:
            from .ops.reductions import state_hash as device_hash

            tensors = []
            for idx in sorted(self._engine.buckets):
                st = self._engine.buckets[idx]
                tensors += [st.curr[0], st.prev[0]]
            return device_hash(tensors, seed=self.step_count)
        return int(self.hook.predictor_hash())

    def _verify_predictor_hash(self) -> bool:
        """All ranks must hold the same predictor state; on a mismatch the next step runs
        uncompressed, which re-seeds the history everywhere."""
        try:
            h = self.state_hash()
            dev = "cpu"
            if self._engine is not None:
                dev = self._engine.device
            elif self._cpp is not None:
                dev = self._cpp._arena.device
            t = torch.tensor([h & 0xFFFFFFFF, (h >> 32) & 0xFFFFFFFF], dtype=torch.int64, device=dev)
            gathered = [torch.zeros_like(t) for _ in range(self.world_size)]
            dist.all_gather(gathered, t, group=self.process_group)
            vals = [(int(g[0].item()) | (int(g[1].item()) << 32)) for g in gathered]
            if all(v == vals[0] for v in vals):
                return True
            warnings.warn(f"nangila: predictor state hash mismatch at step {self.step_count}: {vals}")
            self._force_uncompressed = True
            self.hook.verify_hash(vals[0] ^ 1 if vals[0] == h else vals[0])
            return False
        except Exception as exc:  # pragma: no cover
            warnings.warn(f"nangila: hash verification failed: {exc!r}")
            return True

    # ---- checkpoint ------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        sd = {"step_count": self.step_count, "total_original_bytes": self.total_original_bytes,
              "total_compressed_bytes": self.total_compressed_bytes,
              "core": bytes(self.hook.make_checkpoint().to_bytes())}
        if self._engine is not None:
            sd["predres"] = self._engine.state_dict()
        if self._cpp is not None:
            out = {}
            for idx in self._cpp.get_stats()["prediction_gain"]:
                st = self._cpp.bucket_state(idx)
                out[idx] = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in st.items()}
            sd["predres"] = out
        return sd

    def load_state_dict(self, sd: dict) -> None:
        from ._C import NangilaCheckpoint

        self.step_count = int(sd["step_count"])
        self.total_original_bytes = int(sd.get("total_original_bytes", 0))
        self.total_compressed_bytes = int(sd.get("total_compressed_bytes", 0))
        self.hook.restore_checkpoint(NangilaCheckpoint.from_bytes(sd["core"]))
        # Device state is applied lazily, bucket by bucket, once DDP has settled on its bucket layout;
        # until then (one step) gradients are averaged exactly.
        self._pending_state = {int(k): v for k, v in (sd.get("predres") or {}).items()}
        self._exact_until_step = self.step_count + 1
        if self._cpp is not None:
            self._cpp.fast_forward(self.step_count)
        if self._native:
            # the reducer-level hook does the same in C++: one uncompressed step, then saved state per bucket
            self._cpp.set_exact_until(self._exact_until_step)
            for idx, st in self._pending_state.items():
                if isinstance(st.get("prev"), torch.Tensor) and isinstance(st.get("curr"), torch.Tensor):
                    self._cpp.restore_bucket(idx, st["prev"], st["curr"], st.get("ef") if isinstance(st.get("ef"), torch.Tensor) else None)
            self._pending_state = {}

    def enable_safe_mode(self, config=None) -> None:
        from ._C import SafeModeConfig

        self.hook.enable_safe_mode(config or SafeModeConfig())

    def report_validation_loss(self, loss: float):
        return self.hook.report_validation_loss(float(loss))


def register_nangila_hook(
    ddp_model: DDP,
    threshold: float = 0.95,
    warmup_steps: int = 100,
    prefer_cpp: bool = True,
    sync_mode: int = 2,
    enable_gpu_native: bool = False,
    *,
    compressor_type: int = 0,
    dgc_sparsity: float = 0.999,
    power_sgd_rank: int = 1,
    mask: Any = None,
    mask_path: Optional[str] = None,
    liveness_timeout: Optional[float] = None,
    **extra: Any,
) -> "NangilaDDPHook":
    """Register the Nangila compression hook on a DDP model and return it (call ``.step()`` after
    every optimizer step). Signature and defaults as the reference (ddp.py:415-426).

    ``mask`` (a ``TopologyMask``, or its bytes as ``Sculptor.generate_mask()`` returns them) or ``mask_path`` (a
    file holding those bytes) applies a calibrated topology: Passenger parameters (layer id = position in
    ``ddp_model.parameters()``) are not exchanged; their averaged gradient is ``alpha * g_driver + beta``. The
    reference accepted no mask here and treated every layer as a Driver (ddp.py:151).

    ``liveness_timeout`` (seconds) turns on rank heartbeats through the process group's store: ``hook.step()`` then
    raises ``RankFailure`` naming a peer that left or fell silent (see ``NangilaDDPHook.enable_liveness``)."""
    if not isinstance(ddp_model, DDP):
        raise TypeError(f"Expected DistributedDataParallel, got {type(ddp_model)}")
    _warn_if_advanced_ddp_options(compressor_type, dgc_sparsity, power_sgd_rank)
    sync_mode = _validate_sync_mode(sync_mode)
    if mask is None and mask_path is not None:
        with open(mask_path, "rb") as fh:
            mask = fh.read()
    params = [p for p in ddp_model.parameters() if p.requires_grad]
    num_layers = len(list(ddp_model.parameters()))
    # bytes of symmetric memory the bucket regions will need: two areas per bucket, each holding the
    # larger of the raw and the packed form of every element
    total = sum(p.numel() * (8 if p.element_size() >= 4 else 4) for p in params)
    hook = NangilaDDPHook(
        process_group=ddp_model.process_group, threshold=threshold, warmup_steps=warmup_steps,
        num_layers=num_layers, sync_mode=sync_mode, enable_gpu_native=enable_gpu_native,
        compressor_type=compressor_type, dgc_sparsity=dgc_sparsity, power_sgd_rank=power_sgd_rank,
        total_numel=total, mask=mask, **extra,
    )
    # NANGILA_PREFER_CPP=0/1 overrides the argument (to compare the two hook implementations)
    hook.prefer_cpp = bool(int(os.environ.get("NANGILA_PREFER_CPP", int(bool(prefer_cpp)))))
    hook._param_ids = {id(p): i for i, p in enumerate(ddp_model.parameters())}
    native = (hook.prefer_cpp and CPP_HOOK_AVAILABLE and int(compressor_type) == 0 and not hook._passengers
              and bool(params) and all(p.is_cuda for p in params) and os.environ.get("NANGILA_NATIVE_HOOK", "1") != "0")
    if native:
        hook.install_native(ddp_model)   # C++ hook on the reducer: no Python per bucket
    else:
        ddp_model.register_comm_hook(state=None, hook=hook)
    if liveness_timeout is not None:
        hook.enable_liveness(interval=min(0.5, float(liveness_timeout) / 4.0), timeout=float(liveness_timeout))
    return hook


__all__ = ["NangilaDDPHook", "register_nangila_hook", "CPP_HOOK_AVAILABLE", "NangilaCppHook"]
