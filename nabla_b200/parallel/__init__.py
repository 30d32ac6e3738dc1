"""Multi-GPU runtime: process-group setup, collective backend, symmetric memory and the fused
compute+collective kernels."""
from .launch import init_distributed, is_distributed, local_rank, rank, shutdown, world_size  # noqa: F401
from .health import PeerLostError, announce_exit, beat, check_peers  # noqa: F401
