"""A rank leaves a running job between two steps (host-side failure, gloo ranks on CPU; no device is involved):
the others learn which rank it was, either from its goodbye before they start another exchange, or from the heartbeats
after their next collective failed."""
import json
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _port() -> str:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return str(p)


def _run(tmp_path, mode):
    port, world = _port(), 3
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "_liveness_worker.py"), str(r), str(world), port, mode, str(tmp_path)],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
             for r in range(world)]
    errs = [p.communicate(timeout=120)[1] for p in procs]
    reports = {}
    for r in range(world - 1):
        path = tmp_path / f"report_{r}.json"
        assert path.exists(), errs[r][-2000:]
        reports[r] = json.loads(path.read_text())
    return reports


@pytest.mark.timeout(300)
def test_crashed_rank_is_named_after_the_failed_collective(tmp_path):
    reports = _run(tmp_path, "crash")
    for r, rep in reports.items():
        assert rep["steps"] in (4, 5), rep                  # five steps with everybody (the fifth's step() may already see the silence)
        assert rep["ranks"] == [2] and not rep["store_lost"], rep
        assert rep["how"] in ("collective error", "liveness")
        if rep["how"] == "collective error":
            assert rep["seconds_to_name"] < 4.5, rep         # heartbeat time-out 1.5 s, not the group's 8 s


@pytest.mark.timeout(300)
def test_rank_that_says_goodbye_stops_the_others_before_their_next_exchange(tmp_path):
    reports = _run(tmp_path, "goodbye")
    for r, rep in reports.items():
        # stopped by the goodbye alone: at the end of the fifth step() if the leaver was quicker, else at the health check
        assert rep["how"] == "liveness" and rep["ranks"] == [2] and not rep["store_lost"] and rep["steps"] in (4, 5), rep


def test_monitor_on_a_shared_store_reports_silence_and_goodbyes():
    import time

    import torch.distributed as dist

    from nangila.utils.liveness import RankFailure, RankMonitor

    store = dist.HashStore()
    mons = [RankMonitor(store, r, 3, interval=0.05, timeout=0.4) for r in range(3)]
    try:
        time.sleep(0.3)
        assert mons[0].dead_ranks() == [] and mons[1].dead_ranks() == []
        mons[0].check()                      # nobody missing: returns
        mons[2].close()                      # rank 2 falls silent without a word
        t0 = time.monotonic()
        with pytest.raises(RankFailure) as err:
            mons[0].check(wait=3.0)
        assert err.value.ranks == [2] and not err.value.store_lost and 0.2 < time.monotonic() - t0 < 2.0
        mons[1].leave()                      # rank 1 says goodbye: known at once
        assert mons[0].dead_ranks() == [1, 2]
        assert "rank(s) 1, 2 stopped responding" in str(RankFailure([2, 1]))
        with pytest.raises(ValueError):
            RankMonitor(store, 0, 2, interval=1.0, timeout=0.5)
    finally:
        for m in mons:
            m.close()
