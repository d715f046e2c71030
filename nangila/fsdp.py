"""FSDP integration.

Two entry points:

* ``apply_nangila_fsdp(module)`` (re-exported from ``nangila.parallel.fsdp_collectives``) for FSDP2
  ``fully_shard``: a true compressed reduce-scatter and a quantizing parameter all-gather, each one
  fused kernel over NVLink peer memory.
* ``NangilaFSDPState`` / ``nangila_fsdp_hook`` with the reference's signatures
  (python/nangila/fsdp.py:9-78, :80-236) for FSDP1 ``register_comm_hook``. The hook receives the
  unsharded flat gradient and must leave this rank's shard in ``output``; it runs the same fused
  reduce-scatter kernel (the reference all-gathers every rank's full INT4 gradient instead and
  slices). When the kernel cannot be used (CPU tensors, odd shard sizes) it falls back to the
  process group's reduce-scatter.
"""
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ._C import NangilaConfig
from .ddp import _validate_sync_mode
from .parallel.fsdp_collectives import NangilaAllGather, NangilaReduceScatter, apply_nangila_fsdp  # noqa: F401
from .utils.liveness import LivenessMixin


class NangilaFSDPState(LivenessMixin):
    """State object for ``fsdp_model.register_comm_hook(state, nangila_fsdp_hook)``."""

    def __init__(self, process_group: Optional[dist.ProcessGroup], config: Optional[NangilaConfig] = None,
                 sync_mode: int = 2, *, predictor: bool = False, error_feedback: bool = False):
        self.process_group = process_group if process_group is not None else dist.group.WORLD
        self.config = config if config is not None else NangilaConfig()
        self.sync_mode = _validate_sync_mode(sync_mode)
        self.world_size = dist.get_world_size(self.process_group)
        self.rank = dist.get_rank(self.process_group)
        # predictor=True: the reference's prediction-residual data flow (full-size history of the averaged gradient
        # per unit on every rank); default: block-INT4 reduce-scatter without history
        self.predictor = predictor
        self.error_feedback = error_feedback
        self._step = 0
        self._calls = 0
        self.stream: Optional[torch.cuda.Stream] = None
        self.managed_params: Dict[int, torch.nn.Parameter] = {}
        self.history: Dict[int, Any] = {}
        self._rs: Optional[NangilaReduceScatter] = None

    def step_counter(self) -> int:
        return self._step

    def step(self) -> None:
        """Advance the step; call once per optimizer step. The FSDP units reduced by the hook are told apart by
        their position among the calls of a step (as the reference's ``layer_counter`` did,
        python/nangila/fsdp.py:50-53,86-87), so this is also what keeps their states apart."""
        self._step += 1
        if self._rs is not None:
            self._rs.end_step()
        self.check_peers()   # rank heartbeats, when enable_liveness() was called (nangila/utils/liveness.py)

    def get_history(self, key: int):
        return self.history.get(key)

    @staticmethod
    def compute_gamma(residual: torch.Tensor) -> float:
        """max |r| / 7 (python/nangila/fsdp.py:71-78); kept for callers of the old API."""
        return max(float(residual.abs().max()) / 7.0, 1e-8)

    def reduce_scatter(self) -> NangilaReduceScatter:
        if self._rs is None:
            self._rs = NangilaReduceScatter(group=self.process_group, predictor=self.predictor,
                                            error_feedback=self.error_feedback, momentum=float(self.config.momentum))
        return self._rs


def nangila_fsdp_hook(state: NangilaFSDPState, grad: torch.Tensor, *args) -> None:
    """FSDP1 communication hook. ``args`` is ``(output,)`` for sharded strategies (the hook fills it
    with this rank's reduced shard) and empty for NO_SHARD (the gradient is all-reduced in place)."""
    state._calls += 1
    world = state.world_size
    if not args:
        dist.all_reduce(grad, group=state.process_group)
        grad.div_(world)
        return
    output = args[0]
    rs = state.reduce_scatter()
    if grad.is_cuda and grad.is_contiguous() and output.is_contiguous():
        rs(output, grad, state.process_group, dist.ReduceOp.AVG)
        if state.sync_mode == 1 or (state.sync_mode == 2 and state._calls % 100 == 0):
            rs.check_status()
    else:
        try:
            dist.reduce_scatter_tensor(output, grad, group=state.process_group)
            output.div_(world)
        except (RuntimeError, NotImplementedError):
            # backends without reduce-scatter (gloo): all-reduce and keep this rank's shard
            full = grad.detach().clone()
            dist.all_reduce(full, group=state.process_group)
            shard = output.numel()
            output.copy_(full.reshape(-1)[state.rank * shard:(state.rank + 1) * shard].view_as(output)).div_(world)
