"""Process-group bring-up for one-process-per-GPU jobs started by ``torch.distributed.run``."""
from __future__ import annotations

import os
import random
from typing import Tuple

import torch
import torch.distributed as dist


def local_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    return torch.device("cpu")


def init_distributed(backend: str | None = None) -> Tuple[int, int, torch.device]:
    """Initialise the default group from RANK / WORLD_SIZE / MASTER_* (a single process becomes a group of
    one on 127.0.0.1). Returns (rank, world, device)."""
    dev = local_device()
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        backend = backend or ("nccl" if dev.type == "cuda" else "gloo")
        kw = {"device_id": dev} if dev.type == "cuda" else {}
        dist.init_process_group(backend, **kw)
    return dist.get_rank(), dist.get_world_size(), dev


def seed_everything(seed: int) -> None:
    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
