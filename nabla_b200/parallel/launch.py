"""Process-group bring-up for one-process-per-GPU runs (torchrun sets RANK / LOCAL_RANK /
WORLD_SIZE / MASTER_ADDR / MASTER_PORT)."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def is_distributed() -> bool:
    return world_size() > 1


def init_distributed(backend: str | None = None, timeout_s: float = 600.0) -> tuple[int, int]:
    """Initialise torch.distributed from the torchrun environment (no-op for a single
    process). Binds this process to ``cuda:LOCAL_RANK`` and makes it the default device."""
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    if ws <= 1:
        if torch.cuda.is_available():
            torch.cuda.set_device(0)
        return 0, 1
    if not dist.is_initialized():
        use_cuda = torch.cuda.is_available()
        if backend is None:
            backend = "nccl" if use_cuda else "gloo"
        if use_cuda:
            torch.cuda.set_device(local_rank())
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = {}
        if use_cuda and backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank())
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    if torch.cuda.is_available():
        from ..core.common.context import set_default_device
        from ..types import Accelerator

        set_default_device(Accelerator(local_rank()))
    return dist.get_rank(), dist.get_world_size()
