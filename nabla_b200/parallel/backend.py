"""Collective backend for *distributed* meshes (one process per GPU).

Default implementation: ``torch.distributed`` (NCCL over NVLink/NVSwitch on GPUs, gloo on
CPU). When ``nabla_b200.parallel.symm`` has been initialised, sum all-reduce / all-gather /
reduce-scatter of CUDA tensors run through the hand-written peer-memory kernels instead
(``csrc/peer_collectives.cu``); NCCL stays the baseline and handles ``ppermute`` send/recv.

All functions take the local shard buffer and the mesh axes that span the group.
"""
from __future__ import annotations

import os
from typing import Sequence

import torch
import torch.distributed as dist

_REDUCE = {"sum": "SUM", "max": "MAX", "min": "MIN", "prod": "PRODUCT"}
stats = {"nccl_calls": 0, "native_calls": 0}


def _group(mesh, axes):
    pg, ranks = mesh.process_group(tuple(axes))
    return pg, ranks


def _native():
    if os.environ.get("NABLA_B200_COMM", "native") == "nccl":
        return None
    try:
        from . import symm

        return symm if symm.is_ready() else None
    except Exception:
        return None


def _local_only() -> bool:
    from . import symm

    return symm.local_only()


def all_reduce(buf: torch.Tensor, mesh, axes: Sequence[str], op: str = "sum") -> torch.Tensor:
    pg, ranks = _group(mesh, axes)
    if len(ranks) == 1 or _local_only():
        return buf
    nat = _native()
    if nat is not None and op == "sum" and nat.supports(buf):
        stats["native_calls"] += 1
        return nat.all_reduce(buf, mesh, tuple(axes))
    out = buf.clone() if buf.is_contiguous() else buf.contiguous()
    stats["nccl_calls"] += 1
    dist.all_reduce(out, op=getattr(dist.ReduceOp, _REDUCE[op]), group=pg)
    return out


def all_gather(buf: torch.Tensor, mesh, axes: Sequence[str], dim: int, sizes: Sequence[int] | None = None) -> torch.Tensor:
    """Concatenate the group's shards along ``dim``. ``sizes`` gives every member's extent
    along ``dim`` when shards are uneven."""
    pg, ranks = _group(mesh, axes)
    n = len(ranks)
    if n == 1:
        return buf
    buf = buf.contiguous()
    even = sizes is None or len(set(sizes)) == 1
    if _local_only():
        return torch.cat([buf] * n, dim=dim)
    nat = _native()
    if nat is not None and even and dim == 0 and nat.supports(buf) and (buf.numel() * buf.element_size()) % 16 == 0 \
            and buf.numel() * buf.element_size() * n + 4096 <= nat.DEFAULT_BYTES - 65536:
        stats["native_calls"] += 1
        return nat.all_gather_dim0(buf, mesh, tuple(axes))
    stats["nccl_calls"] += 1
    if even:
        if dim == 0:
            out = torch.empty((n * buf.shape[0],) + tuple(buf.shape[1:]), dtype=buf.dtype, device=buf.device)
            dist.all_gather_into_tensor(out, buf, group=pg)
            return out
        parts = [torch.empty_like(buf) for _ in range(n)]
        dist.all_gather(parts, buf, group=pg)
        return torch.cat(parts, dim=dim)
    mx = max(sizes)
    pad_shape = list(buf.shape)
    pad_shape[dim] = mx
    padded = torch.zeros(pad_shape, dtype=buf.dtype, device=buf.device)
    padded.narrow(dim, 0, buf.shape[dim]).copy_(buf)
    parts = [torch.empty_like(padded) for _ in range(n)]
    dist.all_gather(parts, padded, group=pg)
    return torch.cat([p.narrow(dim, 0, s) for p, s in zip(parts, sizes)], dim=dim)


def reduce_scatter(buf: torch.Tensor, mesh, axes: Sequence[str], dim: int) -> torch.Tensor | None:
    """Sum over the group and keep this rank's chunk of ``dim`` (even split only; returns
    ``None`` when the extent does not divide, the caller then falls back)."""
    pg, ranks = _group(mesh, axes)
    n = len(ranks)
    if n == 1:
        return buf
    if buf.shape[dim] % n != 0:
        return None
    x = buf.movedim(dim, 0).contiguous() if dim != 0 else buf.contiguous()
    if _local_only():
        c = x.shape[0] // n
        out = x[ranks.index(dist.get_rank()) * c:][:c].clone()
        return out.movedim(0, dim) if dim != 0 else out
    nat = _native()
    if nat is not None and nat.supports(x) and (x.numel() // n * x.element_size()) % 16 == 0:
        stats["native_calls"] += 1
        out = nat.reduce_scatter_dim0(x, mesh, tuple(axes))
        return out.movedim(0, dim) if dim != 0 else out
    out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    stats["nccl_calls"] += 1
    dist.reduce_scatter_tensor(out, x, group=pg)
    return out.movedim(0, dim) if dim != 0 else out


def permute(buf: torch.Tensor, mesh, perm: Sequence[tuple[int, int]]) -> torch.Tensor:
    """Point-to-point shift: rank ``src`` sends its shard to ``dst`` for every pair; ranks
    nobody sends to receive zeros. One peer-memory kernel per call (``symm.permute``); grouped NCCL
    send/recv when the native path is off or the payload does not fit it."""
    me = mesh.rank
    if _local_only():
        return buf.clone()
    nat = _native()
    if nat is not None and os.environ.get("NABLA_B200_PERMUTE", "native") != "nccl" and nat.permute_supported(buf, mesh, perm):
        # one peer-memory kernel on every rank of the mesh instead of a grouped NCCL send / recv
        stats["native_calls"] += 1
        stats["native_permute"] = stats.get("native_permute", 0) + 1
        return nat.permute(buf, mesh, perm)
    ops = []
    out = torch.zeros_like(buf)
    send_to = [d for s, d in perm if s == me]
    recv_from = [s for s, d in perm if d == me]
    src_buf = buf.contiguous()
    for d in send_to:
        if d == me:
            out.copy_(src_buf)
        else:
            ops.append(dist.P2POp(dist.isend, src_buf, d))
    for s in recv_from:
        if s != me:
            ops.append(dist.P2POp(dist.irecv, out, s))
    if ops:
        stats["nccl_calls"] += 1
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return out


def broadcast(buf: torch.Tensor, mesh, root: int = 0) -> torch.Tensor:
    out = buf.clone()
    if _local_only():
        return out
    stats["nccl_calls"] += 1
    dist.broadcast(out, src=root)
    return out
