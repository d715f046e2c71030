"""Sculptor calibration with the statistics computed on the device.

``DeviceSculptor`` has the interface of ``nangila.Sculptor`` (record / end_step / generate_mask /
num_samples / num_layers / reset) but takes CUDA tensors and never copies gradients to the host:
layer norms, the element-wise streaming pair statistics and their reduction to correlation and
coupling run in the kernels of ``csrc/kernels/sculptor_stats.cu``; the pair schedule and the greedy
Driver / Passenger assignment stay in the C++ core (``nangila._C.Sculptor``), which receives only
scalars (reference: nangila-core/src/sculptor.rs:238-550, all on the host there).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .._C import Sculptor as _CoreSculptor


class DeviceSculptor:
    def __init__(self, threshold: float = 0.95, strategy: str = "full", param: int = 0):
        from ..parallel.predres_engine import _glue

        self._glue = _glue()
        self.core = _CoreSculptor(threshold)
        if strategy != "full":
            self.core.set_sampling_strategy(strategy, param)
        self.threshold = threshold
        self._current: Dict[int, torch.Tensor] = {}
        self._pair_state: Dict[Tuple[int, int], torch.Tensor] = {}
        self._pair_count: Dict[Tuple[int, int], int] = {}
        self._steps = 0

    def record(self, layer_id: int, gradient: torch.Tensor) -> None:
        """Register this step's gradient of a layer (a CUDA tensor; it is read at ``end_step``, so it
        must stay unchanged until then). A layer id seen twice closes the open step first."""
        if layer_id in self._current:
            self.end_step()
        self._current[int(layer_id)] = gradient.detach().contiguous().view(-1)

    def end_step(self) -> None:
        if not self._current:
            return
        ids = sorted(self._current)
        tensors = [self._current[i] for i in ids]
        sumsq = self._glue.sculptor_layer_sumsq(tensors).sqrt().tolist()
        for i, norm in zip(ids, sumsq):
            self.core.record_norm(i, norm, self._current[i].numel())
        pairs = self.core.scheduled_pairs(ids)
        if pairs:
            xi, xj, st, cnt = [], [], [], []
            for a, b in pairs:
                key = (min(a, b), max(a, b))
                if key not in self._pair_state:
                    n = self._current[key[0]].numel()
                    self._pair_state[key] = torch.zeros(5 * n, dtype=torch.float32, device=tensors[0].device)
                    self._pair_count[key] = 0
                self._pair_count[key] += 1
                xi.append(self._current[key[0]])
                xj.append(self._current[key[1]])
                st.append(self._pair_state[key])
                cnt.append(self._pair_count[key])
            # a pair scheduled twice in one step (kNN does that) must be applied in order
            seen: Dict[Tuple[int, int], int] = {}
            batches: List[List[int]] = []
            for k, (a, b) in enumerate(pairs):
                key = (min(a, b), max(a, b))
                lvl = seen.get(key, 0)
                seen[key] = lvl + 1
                while len(batches) <= lvl:
                    batches.append([])
                batches[lvl].append(k)
            for batch in batches:
                self._glue.sculptor_pair_update([xi[k] for k in batch], [xj[k] for k in batch], [st[k] for k in batch],
                                                [cnt[k] for k in batch])
        self.core.note_step()
        self._steps += 1
        self._current.clear()

    def _finalize(self) -> None:
        keys = [k for k, c in self._pair_count.items() if c >= 2]
        if not keys:
            return
        out = self._glue.sculptor_pair_finalize([self._pair_state[k] for k in keys], [self._pair_count[k] for k in keys])
        rows = out.tolist()
        for key, r in zip(keys, rows):
            s_corr, v_corr, sa_ij, sb_ij, v_ij, sa_ji, sb_ji, v_ji = r
            if v_corr <= 0:
                continue
            corr = s_corr / v_corr
            a_ij, b_ij = (sa_ij / v_ij, sb_ij / v_ij) if v_ij > 0 else (0.0, 0.0)
            a_ji, b_ji = (sa_ji / v_ji, sb_ji / v_ji) if v_ji > 0 else (0.0, 0.0)
            self.core.set_pair_result(key[0], key[1], self._pair_count[key], corr, a_ij, b_ij, a_ji, b_ji)

    def generate_mask(self) -> bytes:
        if self._current:
            self.end_step()
        self._finalize()
        return self.core.generate_mask()

    def correlation(self, a: int, b: int):
        self._finalize()
        return self.core.correlation(a, b)

    def coupling(self, driver: int, passenger: int):
        self._finalize()
        return self.core.coupling(driver, passenger)

    def num_samples(self) -> int:
        return self.core.num_samples()

    def num_layers(self) -> int:
        return self.core.num_layers()

    def reset(self) -> None:
        self.core.reset()
        self._current.clear()
        self._pair_state.clear()
        self._pair_count.clear()
        self._steps = 0
