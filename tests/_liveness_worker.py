"""One gloo rank of the rank-failure tests: trains a small DDP model with the hook, and either leaves (crash or goodbye)
or reports how it learned that a peer left. Usage: _liveness_worker.py RANK WORLD PORT MODE OUTDIR"""
import datetime
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nangila.ddp import register_nangila_hook  # noqa: E402
from nangila.utils.liveness import RankFailure  # noqa: E402


def main() -> int:
    rank, world, port, mode, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    torch.manual_seed(0)
    ddp = DDP(nn.Sequential(nn.Linear(32, 16), nn.ReLU(), nn.Linear(16, 4)))
    hook = register_nangila_hook(ddp, warmup_steps=2, liveness_timeout=1.5)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
    gen = torch.Generator().manual_seed(100 + rank)
    leaver = world - 1
    report = {"rank": rank, "steps": 0}
    t_fail = None
    try:
        for step in range(12):
            x, y = torch.randn(8, 32, generator=gen), torch.randint(0, 4, (8,), generator=gen)
            nn.functional.cross_entropy(ddp(x), y).backward()
            opt.step()
            opt.zero_grad()
            hook.step()
            report["steps"] = step + 1
            if step == 4:
                if rank == leaver and mode == "crash":
                    os._exit(0)            # no goodbye, nothing in flight: between two steps
                if rank == leaver and mode == "goodbye":
                    hook.leave()
                    time.sleep(0.5)        # stays around a moment: the others must stop because of the goodbye alone
                    os._exit(0)
                if mode == "goodbye":
                    hook.check_peers(wait=3.0)   # a health check between steps
    except RankFailure as exc:
        report.update(how="liveness", ranks=exc.ranks, store_lost=exc.store_lost)
        if exc.store_lost:
            report["store_error"] = repr(hook.liveness._store_error)[:300]
    except Exception as exc:  # the collective with the missing rank failed or timed out
        t_fail = time.monotonic()
        report.update(how="collective error", error=type(exc).__name__)
        try:
            hook.check_peers(wait=4.0)
        except RankFailure as named:
            report.update(ranks=named.ranks, store_lost=named.store_lost, seconds_to_name=round(time.monotonic() - t_fail, 2))
    with open(os.path.join(out, f"report_{rank}.json"), "w") as f:
        json.dump(report, f)
    if rank == 0:
        time.sleep(3.0)   # rank 0 hosts the store: it stays until the others have had time to read it
    os._exit(0)   # the group cannot be torn down collectively any more


if __name__ == "__main__":
    sys.exit(main())
