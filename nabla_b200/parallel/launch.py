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


def shutdown(*compiled, timeout_s: float = 45.0) -> None:
    """Orderly end of a (multi-rank) run: drop the recorded schedules and their CUDA graphs, wait for
    the device, meet the other ranks, then destroy the process group and return normally, so the
    interpreter's exit hooks run. Captured graphs hold NCCL and peer-memory launches; destroying the
    communicator while such a graph is alive can block, which is why the graphs go first.

    A daemon timer ends the process (exit code 0, streams flushed) if the teardown itself does not
    come back within ``timeout_s``: a rank stuck in teardown must not keep the job's launcher alive."""
    import gc
    import sys
    import threading

    for c in compiled:
        rel = getattr(c, "release", None)
        if rel is not None:
            rel()
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if not (dist.is_available() and dist.is_initialized()):
        return

    def _bail():
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)

    guard = threading.Timer(timeout_s, _bail)
    guard.daemon = True
    guard.start()
    try:
        dist.barrier()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            from . import symm

            symm.release_all()          # peer mappings go while every rank is still here
            torch.cuda.synchronize()
            dist.barrier()
        dist.destroy_process_group()
    finally:
        guard.cancel()
