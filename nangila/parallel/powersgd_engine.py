"""Host driver of the PowerSGD path: per-parameter matrix state (error memory, warm-start Q), the
two tcgen05 GEMMs, the two cross-rank factor exchanges and the reconstruction, for every matrix-shaped
gradient of a DDP bucket; the remaining small / 1-D gradients of the bucket are averaged exactly by
the prediction-residual engine's uncompressed mode.

The six launches per matrix (prep, GEMM, exchange, GEMM, exchange, reconstruct) of all matrices of a
DDP bucket are recorded once into a CUDA graph and replayed with one launch per bucket afterwards: a
ResNet-50 step has 53 matrices, and 300-odd small dependent kernels queued one behind the other leave
the GPU mostly idle; in the graph the chains of different matrices run side by side (a few branch streams). The exchange kernels read their epoch from a device word that the graph increments, so a replay
is a new exchange; everything else in the recorded launches (buffers, tensor maps) is fixed for the life
of the bucket. ``NANGILA_PSGD_GRAPH=0`` launches the kernels one by one instead.

Replaces PowerSGDCompressor (nangila-core/src/power_sgd.rs:20-193). Unlike the reference, which ships
every rank's own P and Q and averages W dense reconstructions, P and Q' are averaged across ranks
(standard PowerSGD), so the wire carries (m + n) r floats per matrix per rank.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .predres_engine import STATUS_MESSAGES, _glue
from .symm import LoopbackArena, Region


def eligible(shape: torch.Size, numel_min: int = 4096) -> bool:
    """Matrix view (m = shape[0], n = prod(shape[1:])) usable by the TMA-fed GEMMs."""
    if len(shape) < 2:
        return False
    m = shape[0]
    n = 1
    for d in shape[1:]:
        n *= d
    return m % 8 == 0 and n % 8 == 0 and m >= 16 and n >= 16 and m * n >= numel_min


@dataclass
class MatrixState:
    m: int
    n: int
    r: int
    mef: List[torch.Tensor]      # bf16 [m, n]: gradient + error memory of the current step
    ef: List[torch.Tensor]       # bf16 [m, n]: error memory
    qt: List[torch.Tensor]       # bf16 [16, n]: warm-start Q, transposed, orthonormal rows
    pt: List[torch.Tensor]       # bf16 [16, m]
    p_local: List[torch.Tensor]  # fp32 [m, 16]
    q_local: List[torch.Tensor]  # fp32 [n, 16]
    p_full: List[torch.Tensor]   # p_local plus the tile counters of the GEMM's epilogue push, cleared together
    q_full: List[torch.Tensor]
    p_cnt: List[torch.Tensor]    # int32 view of the counters
    q_cnt: List[torch.Tensor]
    p_mean: List[torch.Tensor]
    q_mean: List[torch.Tensor]
    scratch: List[torch.Tensor]  # fp32 [max(m, n), 16]
    region_p: Region
    region_q: Region
    lay_p: tuple
    lay_q: tuple
    epoch: int = 0


def initial_qt(n: int, r: int, device) -> torch.Tensor:
    """The reference's deterministic warm start Q[i][j] = ((i + j) mod 100) / 100, orthonormalised by
    column Gram-Schmidt (power_sgd.rs:110-125), returned transposed and padded to 16 rows."""
    i = torch.arange(n, device=device, dtype=torch.float64)[:, None]
    j = torch.arange(r, device=device, dtype=torch.float64)[None, :]
    q = ((i + j) % 100) / 100.0
    for c in range(r):
        for k in range(c):
            q[:, c] -= (q[:, c] @ q[:, k]) * q[:, k]
        nrm = q[:, c].norm()
        if nrm > 1e-10:
            q[:, c] /= nrm
    out = torch.zeros(16, n, device=device, dtype=torch.bfloat16)
    out[:r] = q.t().to(torch.bfloat16)
    return out


class PowerSGDEngine:
    def __init__(self, arena, device: torch.device, rank: int = 1, stream: Optional[torch.cuda.Stream] = None,
                 group=None, timeout_s: Optional[float] = None, exact_engine=None):
        if not 1 <= rank <= 16:
            raise ValueError("power_sgd_rank must be in [1, 16] on the device path")
        self.arena = arena
        self.device = torch.device(device)
        self.world = arena.world
        self.rank = arena.rank
        self.loopback = isinstance(arena, LoopbackArena)
        self.nvr = self.world if self.loopback else 1
        self.r = rank
        self.stream = stream
        self.group = group
        self.exact_engine = exact_engine
        self.timeout_s = float(os.environ.get("NANGILA_WAIT_TIMEOUT_MS", "2000")) / 1e3 if timeout_s is None else timeout_s
        self.states: Dict[tuple, MatrixState] = {}
        self.use_graphs = os.environ.get("NANGILA_PSGD_GRAPH", "1") != "0"
        self.push_from_gemm = os.environ.get("NANGILA_PSGD_PUSH", "1") != "0"
        self._graphs: Dict[int, tuple] = {}   # bucket index -> (key, CUDAGraph, epoch word, launches recorded)
        self.graph_replays = 0
        self._capture_stream: Optional[torch.cuda.Stream] = None
        # parallel chains in a bucket's graph: at most this many exchange kernels (8 CTAs each) wait for peers at once
        self.graph_branches = max(1, int(os.environ.get("NANGILA_PSGD_BRANCHES", "8")))
        self._branches: List[torch.cuda.Stream] = []
        self.status = [torch.zeros(8, dtype=torch.int32, device=self.device) for _ in range(self.nvr)]
        self.launches = 0
        self._glue = _glue()

    def _state(self, key: tuple, m: int, n: int) -> MatrixState:
        st = self.states.get(key)
        if st is not None and st.m == m and st.n == n:
            return st
        r = min(self.r, m, n)
        dev = self.device
        z = lambda *s, dt=torch.float32: [torch.zeros(*s, dtype=dt, device=dev) for _ in range(self.nvr)]  # noqa: E731
        tot_p, rp, fp = self._glue.psgd_exchange_layout(m, r, self.world)
        tot_q, rq, fq = self._glue.psgd_exchange_layout(n, r, self.world)
        q0 = initial_qt(n, r, dev)
        # accumulators of the two projections, each followed by its tile counters (tiles + 1 words, padded)
        pt_words, qt_words = (m + 127) // 128 + 1, (n + 127) // 128 + 1
        p_full = z(m * 16 + (pt_words + 3) // 4 * 4)
        q_full = z(n * 16 + (qt_words + 3) // 4 * 4)
        st = MatrixState(m=m, n=n, r=r, mef=z(m, n, dt=torch.bfloat16), ef=z(m, n, dt=torch.bfloat16),
                         qt=[q0.clone() for _ in range(self.nvr)], pt=z(16, m, dt=torch.bfloat16),
                         p_local=[t[:m * 16].view(m, 16) for t in p_full], q_local=[t[:n * 16].view(n, 16) for t in q_full],
                         p_full=p_full, q_full=q_full,
                         p_cnt=[t[m * 16:].view(torch.int32) for t in p_full], q_cnt=[t[n * 16:].view(torch.int32) for t in q_full],
                         p_mean=z(m, 16), q_mean=z(n, 16),
                         scratch=z(max(m, n), 16), region_p=self.arena.allocate(int(tot_p)),
                         region_q=self.arena.allocate(int(tot_q)), lay_p=(rp, fp), lay_q=(rq, fq))
        self.states[key] = st
        return st

    def compress_matrix(self, key: tuple, grads: List[torch.Tensor], epoch_word: Optional[torch.Tensor] = None) -> int:
        """Run the whole PowerSGD step for one matrix; ``grads`` (one per emulated rank, any shape with
        >= 2 dims) is replaced by the rank-r approximation of the mean. Returns bytes sent per rank.
        With ``epoch_word`` (an int32 device word) the exchanges take their epoch from it, which is what a
        recorded launch needs; otherwise from the matrix's own host-side counter."""
        g0 = grads[0]
        m = g0.shape[0]
        n = g0.numel() // m
        st = self._state(key, m, n)
        st.epoch += 1
        G = self._glue
        rank0 = 0 if self.loopback else self.rank
        flat = [g.reshape(m, n) for g in grads]
        # The GEMMs start the exchange of their result from the epilogue: the CTA that completes a 128-row tile stores
        # it into every rank's slot over NVLink, the one that completes the last tile releases the flags; the exchange
        # kernel then only waits, averages and orthonormalises (NANGILA_PSGD_PUSH=0: it also does the stores).
        push = self.push_from_gemm
        for v in range(self.nvr):
            G.psgd_prep(flat[v], st.ef[v], st.mef[v], st.p_full[v], st.q_full[v])  # also clears accumulators and counters
            G.psgd_gemm(st.mef[v], st.qt[v], False, st.p_local[v], self.status[v], self.timeout_s, False,
                        **(dict(counters=st.p_cnt[v], push_region_ptrs=st.region_p.ptrs, push_recv_off=st.lay_p[0],
                                push_flag_off=st.lay_p[1], push_me=rank0 + v, push_rank=st.r, push_epoch=st.epoch,
                                push_epoch_word=epoch_word) if push else {}))
        G.psgd_exchange(st.p_local, st.p_mean, [s[:m] for s in st.scratch], st.pt, self.status, st.region_p.ptrs,
                        st.lay_p[0], st.lay_p[1], m, st.r, rank0, True, st.epoch, self.timeout_s, epoch_word, push)
        for v in range(self.nvr):
            G.psgd_gemm(st.mef[v], st.pt[v], True, st.q_local[v], self.status[v], self.timeout_s, False,
                        **(dict(counters=st.q_cnt[v], push_region_ptrs=st.region_q.ptrs, push_recv_off=st.lay_q[0],
                                push_flag_off=st.lay_q[1], push_me=rank0 + v, push_rank=st.r, push_epoch=st.epoch,
                                push_epoch_word=epoch_word) if push else {}))
        G.psgd_exchange(st.q_local, st.q_mean, [s[:n] for s in st.scratch], st.qt, self.status, st.region_q.ptrs,
                        st.lay_q[0], st.lay_q[1], n, st.r, rank0, False, st.epoch, self.timeout_s, epoch_word, push)
        for v in range(self.nvr):
            G.psgd_reconstruct(flat[v], st.ef[v], st.mef[v], st.p_mean[v], st.q_mean[v], m, n, st.r)
        self.launches += 3 * self.nvr + 2 + self.nvr
        return (m + n) * st.r * 4 * max(self.world - 1, 0)

    def reduce(self, index: int, bucket, tensor: torch.Tensor) -> int:
        """DDP entry: compress every eligible gradient of the bucket, average the rest exactly."""
        grads = bucket.gradients()
        sent = 0
        small: List[torch.Tensor] = []

        matrices = [(pos, g) for pos, g in enumerate(grads) if eligible(g.shape) and g.is_contiguous()]
        taken = {pos for pos, _ in matrices}
        small = [g for pos, g in enumerate(grads) if pos not in taken]

        def run_matrices(epoch_word=None) -> int:
            return sum(self.compress_matrix((index, pos), [g], epoch_word) for pos, g in matrices)

        def body():
            nonlocal sent
            if matrices and self.use_graphs:
                sent += self._replay_bucket(index, matrices, run_matrices)
            else:
                sent += run_matrices()
            if small:
                flat = torch.cat([g.reshape(-1) for g in small])
                self.exact_engine.reduce(1_000_000 + index, [flat], compressed=False)
                # the exact engine queues on its own stream; wait for it before scattering back
                if self.exact_engine.stream is not None:
                    torch.cuda.current_stream(self.device).wait_stream(self.exact_engine.stream)
                off = 0
                for g in small:
                    g.copy_(flat[off:off + g.numel()].view_as(g))
                    off += g.numel()
                sent += flat.numel() * flat.element_size()

        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                body()
        else:
            body()
        return sent

    def _replay_bucket(self, index: int, matrices, run_matrices) -> int:
        """One graph launch for all matrices of a bucket. The graph is recorded the first time the bucket
        is seen with this set of gradient addresses (DDP's bucket views keep theirs) and recorded again if
        they change. Called with the engine's stream current."""
        key = tuple((g.data_ptr(), tuple(g.shape), g.dtype) for _, g in matrices)
        entry = self._graphs.get(index)
        if entry is None or entry[0] != key:
            for pos, g in matrices:  # state buffers are created outside the recording
                self._state((index, pos), g.shape[0], g.numel() // g.shape[0])
            if entry is not None:
                epoch_word = entry[2]  # keep counting: the peers' flags hold the old epochs
            else:
                epoch_word = torch.zeros(1, dtype=torch.int32, device=self.device)
            before = self.launches
            graph = torch.cuda.CUDAGraph()
            if self._capture_stream is None:  # recording needs a non-default stream; replays run on the caller's
                self._capture_stream = torch.cuda.Stream(device=self.device)
            torch.cuda.current_stream(self.device).synchronize()
            if not self._branches:
                self._branches = [torch.cuda.Stream(device=self.device) for _ in range(self.graph_branches)]
            with torch.cuda.graph(graph, stream=self._capture_stream, capture_error_mode="thread_local"):
                epoch_word.add_(1)
                # The matrices are independent of one another: each one's chain of six kernels is recorded on one
                # of a few branch streams, so the graph has that many parallel chains and the small kernels of
                # different matrices overlap instead of queueing behind one another.
                main = torch.cuda.current_stream(self.device)
                sent = 0
                for i, (pos, g) in enumerate(matrices):
                    branch = self._branches[i % len(self._branches)]
                    if i < len(self._branches):
                        branch.wait_stream(main)
                    with torch.cuda.stream(branch):
                        sent += self.compress_matrix((index, pos), [g], epoch_word)
                for branch in self._branches[:len(matrices)]:
                    main.wait_stream(branch)
            entry = self._graphs[index] = (key, graph, epoch_word, self.launches - before, sent)
            self.launches = before
        entry[1].replay()
        self.graph_replays += 1
        self.launches += 1
        return entry[4]

    def check_status(self) -> None:
        (self.stream.synchronize() if self.stream is not None else torch.cuda.synchronize(self.device))
        for s in self.status:
            w = s.cpu().tolist()
            if w[0] != 0:
                s.zero_()
                raise RuntimeError(f"nangila: PowerSGD kernel failed ({STATUS_MESSAGES.get(w[0], 'code %d' % w[0])}), "
                                   f"phase {w[5]}, tile {w[6]}")
