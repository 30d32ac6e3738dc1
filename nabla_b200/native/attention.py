"""Attention kernels wrapper. Until the tcgen05 flash-attention library is loaded the
wrappers report "unsupported" and callers use their composed implementation."""
from __future__ import annotations

import torch

launch_count = 0


def supported(q, k, v, mask, dropout_p) -> bool:
    return False


def bwd_available() -> bool:
    return False


def sdpa_fwd(q, k, v, *, causal, scale):
    raise NotImplementedError


def sdpa_bwd(do, q, k, v, o, lse, *, causal, scale):
    raise NotImplementedError
