"""gather / take and scatter along an axis (reference: nabla/ops/view/indexing.py:27-504).

``gather(x, indices, axis)`` replaces dimension ``axis`` of ``x`` by the shape of ``indices``
(numpy ``take``). ``scatter(x, indices, updates, axis)`` writes ``updates`` at those positions
(last write wins); its transpose, scatter-add, is the VJP of gather (embedding backward).
"""
from __future__ import annotations

import torch

from ...core.sharding.propagation import OpShardingRule
from ...core.tensor.api import Tensor
from ...types import DType
from ..base import Operation, _norm_axis, ensure_tensor


def _take(x: torch.Tensor, idx: torch.Tensor, axis: int, bd: int) -> torch.Tensor:
    """x: [B..., d0..dn], idx: [B..., i0..ik] (batch dims shared) or unbatched idx."""
    if bd == 0 or idx.dim() < bd or tuple(idx.shape[:bd]) != tuple(x.shape[:bd]):
        flat = torch.index_select(x, axis, idx.reshape(-1).long())
        return flat.reshape(*x.shape[:axis], *idx.shape, *x.shape[axis + 1:])
    # batched indices: loop-free via flattening batch into the gather
    xb = x.reshape(-1, *x.shape[bd:])
    ib = idx.reshape(-1, *idx.shape[bd:])
    outs = [_take(xb[i], ib[i], axis - bd, 0) for i in range(xb.shape[0])]
    out = torch.stack(outs, 0)
    return out.reshape(*x.shape[:bd], *out.shape[1:])


class GatherOp(Operation):
    partial_policy = "first"

    def adapt_kwargs(self, args, kwargs, batch_dims):
        x, idx = args[0], args[1]
        rank = len(x._impl.global_shape)
        return {"axis": _norm_axis(int(kwargs.get("axis", 0)), rank) + x._impl.batch_dims,
                "bd": min(x._impl.batch_dims, idx._impl.batch_dims)}

    def kernel(self, x, idx, *, axis: int, bd: int = 0):
        from ... import native

        if (bd == 0 and axis == 0 and x.dim() == 2 and native.use_native(x)):
            from ...native import kernels

            if kernels.has("embedding") and x.dtype in (torch.bfloat16, torch.float32):
                return kernels.embedding_gather(x, idx)
        return _take(x, idx, axis, bd)

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, bd: int = 0, **kw):
        xs, is_ = input_shapes
        mx = {i: [f"d{i}"] if i != axis else [f"bcast_g{i}"] for i in range(len(xs))}
        # batch dims of indices line up with x's; the remaining index dims are new factors
        mi = {i: [f"d{i}"] if i < bd else [f"i{i}"] for i in range(len(is_))}
        outs, j = {}, 0
        for i in range(len(xs)):
            if i == axis:
                for k in range(bd, len(is_)):
                    outs[j] = [f"i{k}"]
                    j += 1
            else:
                outs[j] = [f"d{i}"]
                j += 1
        return OpShardingRule([mx, mi], [outs])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from ..creation import zeros_like

        x, idx = primals
        return (scatter_add(zeros_like(x), idx, cot, axis=kwargs.get("axis", 0)), None)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return gather(tangents[0], primals[1], axis=kwargs.get("axis", 0))


class ScatterOp(Operation):
    """``mode='set'``: out = x with out[idx] = updates. ``mode='add'``: out[idx] += updates."""

    def adapt_kwargs(self, args, kwargs, batch_dims):
        x, idx = args[0], args[1]
        rank = len(x._impl.global_shape)
        return {"axis": _norm_axis(int(kwargs.get("axis", 0)), rank) + x._impl.batch_dims,
                "mode": kwargs.get("mode", "set"), "bd": min(x._impl.batch_dims, idx._impl.batch_dims)}

    def kernel(self, x, idx, upd, *, axis: int, mode: str = "set", bd: int = 0):
        from ... import native

        if (mode == "add" and bd == 0 and axis == 0 and x.dim() == 2 and native.use_native(x)
                and x.dtype in (torch.bfloat16, torch.float32)):
            from ...native import kernels

            if kernels.has("embedding"):
                return kernels.embedding_scatter_add(x, idx, upd)
        if bd:
            xb = x.reshape(-1, *x.shape[bd:])
            ib = idx.reshape(-1, *idx.shape[bd:])
            ub = upd.reshape(-1, *upd.shape[bd:])
            outs = [self.kernel(xb[i], ib[i], ub[i], axis=axis - bd, mode=mode, bd=0) for i in range(xb.shape[0])]
            return torch.stack(outs, 0).reshape(x.shape)
        if x.numel() == 0 or upd.numel() == 0:
            return x.clone()            # an empty shard (uneven split): nothing to write
        xm = torch.movedim(x, axis, 0).clone()
        k = idx.dim()
        um = upd
        # updates: x.shape[:axis] + idx.shape + x.shape[axis+1:]  -> move the index block first
        perm = list(range(axis, axis + k)) + list(range(0, axis)) + list(range(axis + k, um.dim()))
        um = um.permute(perm).reshape(-1, *xm.shape[1:])
        flat = idx.reshape(-1).long()
        if mode == "add":
            xm.index_add_(0, flat, um.to(xm.dtype))
        else:
            xm[flat] = um.to(xm.dtype)
        return torch.movedim(xm, 0, axis)

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, **kw):
        xs, is_, us = input_shapes
        mx = {i: [f"d{i}"] if i != axis else [f"bcast_s{i}"] for i in range(len(xs))}
        mi = {i: [f"bcast_i{i}"] for i in range(len(is_))}
        mu = {}
        k = len(is_)
        for i in range(len(us)):
            if i < axis:
                mu[i] = [f"d{i}"]
            elif i < axis + k:
                mu[i] = [f"bcast_u{i}"]
            else:
                mu[i] = [f"d{i - k + 1}"]
        return OpShardingRule([mx, mi, mu], [dict(mx)])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from ..creation import zeros_like

        x, idx, upd = primals
        ax = kwargs.get("axis", 0)
        if kwargs.get("mode", "set") == "add":
            return (cot, None, gather(cot, idx, axis=ax))
        return (scatter(cot, idx, zeros_like(upd), axis=ax), None, gather(cot, idx, axis=ax))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _scatter(tangents[0], primals[1], tangents[2], axis=kwargs.get("axis", 0),
                        mode=kwargs.get("mode", "set"))


_gather, _scatter = GatherOp(), ScatterOp()


def gather(x, indices=None, axis: int = 0) -> Tensor:
    """``numpy.take`` along ``axis``; without ``indices`` it collects the shards of a distributed
    tensor into a replicated one (reference: nabla/ops/view/indexing.py:454-470)."""
    x = ensure_tensor(x)
    if indices is None:
        from ..communication import gather_all_axes

        return gather_all_axes(x)
    indices = ensure_tensor(indices)
    return _gather(x, indices, axis=int(axis))


take = gather


def scatter(x, indices, updates, axis: int = 0) -> Tensor:
    x = ensure_tensor(x)
    return _scatter(x, ensure_tensor(indices), ensure_tensor(updates, x), axis=int(axis), mode="set")


def scatter_add(x, indices, updates, axis: int = 0) -> Tensor:
    x = ensure_tensor(x)
    return _scatter(x, ensure_tensor(indices), ensure_tensor(updates, x), axis=int(axis), mode="add")
