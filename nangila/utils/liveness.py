"""Which ranks are still there: heartbeats through the process group's store.

A rank that leaves a job (crash, kill, exception) does so between two collectives at best; the others find out when
their next collective fails or times out, and the error names no rank. ``RankMonitor`` gives them the name: every rank
bumps a counter in the c10d store from a daemon thread; a peer whose counter has not moved for ``timeout`` seconds (or
that said goodbye through ``leave()``) is reported by ``dead_ranks()`` / ``check()``. Everything here runs on the host
and touches no device, so it works the same under gloo and NCCL; nothing waits on a GPU.

The reference has no rank-failure handling at all (no time-outs, no heartbeats; nangila-hook/src/hook.rs handles
corrupted packets and desynchronised predictors only).

    monitor = RankMonitor.for_group(process_group)       # or hook.enable_liveness()
    ...
    try:
        loss.backward()                                  # a collective fails because rank 2 is gone
    except RuntimeError:
        monitor.check(wait=2.0)                          # raises RankFailure([2]) once the silence is long enough
        raise
"""
from __future__ import annotations

import threading
import time
from typing import Iterable, List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    """One or more ranks stopped sending heartbeats (``.ranks``), or the store itself went away (``.store_lost``)."""

    def __init__(self, ranks: Iterable[int], store_lost: bool = False):
        self.ranks = sorted(ranks)
        self.store_lost = store_lost
        what = "the rendezvous store is unreachable (the rank that hosts it is gone)" if store_lost and not self.ranks \
            else f"rank(s) {', '.join(map(str, self.ranks))} stopped responding"
        super().__init__(f"nangila: {what}")


def _own_store_client(store):
    """A second connection to the TCP store behind ``store``. The heartbeat thread calls the store while the main thread
    may be inside a collective set-up that uses it too, and one client connection is not meant for two threads. Falls
    back to the given store (file / hash stores, or a server that cannot be reached a second time)."""
    import datetime

    inner = store
    while hasattr(inner, "underlying_store"):
        inner = inner.underlying_store
    try:
        if isinstance(inner, dist.TCPStore):
            return dist.TCPStore(inner.host, inner.port, is_master=False, wait_for_workers=False, timeout=datetime.timedelta(seconds=30))
    except Exception:
        pass
    return store


class RankMonitor:
    """Heartbeat writer and reader over a c10d ``Store``.

    ``interval``: seconds between this rank's heartbeats. ``timeout``: a peer silent for longer is considered gone
    (keep it a few intervals long: the thread shares the interpreter with the training loop).
    """

    def __init__(self, store, rank: int, world_size: int, interval: float = 0.5, timeout: float = 5.0, prefix: str = "nangila/hb"):
        if timeout <= interval:
            raise ValueError("timeout must be longer than the heartbeat interval")
        self.store, self.rank, self.world_size = store, int(rank), int(world_size)
        self.interval, self.timeout, self.prefix = float(interval), float(timeout), prefix
        self._last_value = [-1] * self.world_size     # last counter read per rank
        self._last_change = [time.monotonic()] * self.world_size
        self._left: set = set()
        self._stop = threading.Event()
        self._store_error: Optional[BaseException] = None
        self._lock = threading.Lock()
        self._io = threading.Lock()   # one store call at a time from this object (writer thread and reader share the client)
        self._beat()
        self._thread = threading.Thread(target=self._run, name="nangila-heartbeat", daemon=True)
        self._thread.start()

    @classmethod
    def for_group(cls, process_group=None, **kwargs) -> "RankMonitor":
        """Monitor over the store the default process group was created with."""
        from torch.distributed import distributed_c10d as c10d

        group = process_group if process_group is not None else dist.group.WORLD
        return cls(_own_store_client(c10d._get_default_store()), dist.get_rank(group), dist.get_world_size(group), **kwargs)

    # ---- writer ---------------------------------------------------------------------------------------------------
    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _beat(self) -> None:
        try:
            with self._io:
                self.store.add(self._key(self.rank), 1)
        except Exception as exc:  # the store lives in rank 0's process: when that goes, every call fails
            self._store_error = exc

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            self._beat()

    def leave(self) -> None:
        """Says goodbye (peers report this rank at once, without waiting for the silence) and stops the heartbeat."""
        self._stop.set()
        try:
            with self._io:
                self.store.add(f"{self.prefix}/left/{self.rank}", 1)
        except Exception:
            pass

    def close(self) -> None:
        """Stops the heartbeat thread without a goodbye (the job is over for everybody)."""
        self._stop.set()

    # ---- reader ---------------------------------------------------------------------------------------------------
    def poll(self) -> None:
        """Reads every peer's counter once (``add(key, 0)`` never blocks)."""
        now = time.monotonic()
        with self._lock:
            for r in range(self.world_size):
                if r == self.rank:
                    continue
                try:
                    with self._io:
                        value = int(self.store.add(self._key(r), 0))
                        left = int(self.store.add(f"{self.prefix}/left/{r}", 0))
                except Exception as exc:
                    self._store_error = exc
                    return
                if left:
                    self._left.add(r)
                if value != self._last_value[r]:
                    self._last_value[r] = value
                    self._last_change[r] = now

    def dead_ranks(self) -> List[int]:
        """Peers that said goodbye or whose heartbeat has been silent for longer than ``timeout``."""
        self.poll()
        now = time.monotonic()
        with self._lock:
            silent = {r for r in range(self.world_size) if r != self.rank and now - self._last_change[r] > self.timeout}
            return sorted(silent | self._left)

    def check(self, wait: float = 0.0) -> None:
        """Raises ``RankFailure`` if a peer is gone. ``wait``: keep looking for up to that many seconds (after a failed
        collective the culprit's heartbeat is only just going quiet; ``timeout`` has to pass before it shows)."""
        deadline = time.monotonic() + max(0.0, wait)
        while True:
            dead = self.dead_ranks()
            if dead or self._store_error is not None:
                raise RankFailure(dead, store_lost=self._store_error is not None)
            if time.monotonic() >= deadline:
                return
            time.sleep(min(self.interval, 0.1))


class LivenessMixin:
    """``enable_liveness`` / ``check_peers`` / ``leave`` for an object that has a ``process_group`` and a ``step()`` that
    ends with ``self.check_peers()`` (the DDP hook and the FSDP state)."""

    liveness: Optional[RankMonitor] = None

    def enable_liveness(self, interval: float = 0.5, timeout: float = 5.0) -> RankMonitor:
        """Starts heartbeats through the process group's store and returns the ``RankMonitor``. From then on ``step()``
        raises ``RankFailure`` as soon as a peer has said goodbye or has been silent for ``timeout`` seconds, i.e. before
        this rank launches into another exchange with a rank that is not there; after a failed collective,
        ``check_peers(wait=...)`` names the rank that went away."""
        if self.liveness is None:
            self.liveness = RankMonitor.for_group(getattr(self, "process_group", None), interval=interval, timeout=timeout)
        return self.liveness

    def check_peers(self, wait: float = 0.0) -> None:
        """Raises ``RankFailure`` if a peer is gone (no-op unless ``enable_liveness`` was called)."""
        if self.liveness is not None:
            self.liveness.check(wait)

    def leave(self) -> None:
        """Announces that this rank is about to leave the job, so that the others stop at their next ``step()``
        instead of waiting for it in a collective."""
        if self.liveness is not None:
            self.liveness.leave()
