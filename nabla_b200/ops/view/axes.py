"""Axis-manipulating view ops (reference: nabla/ops/view/axes.py:43-868): unsqueeze, squeeze,
swap_axes/transpose, moveaxis, flip, permute, and ``*_physical`` variants whose axes index the
physical shape (vmap batch dims included)."""
from __future__ import annotations

import torch

from ...core.sharding.propagation import OpShardingRule
from ...core.tensor.api import Tensor
from ..base import AxisOp, Operation, _norm_axis, ensure_tensor


def _perm_rule(rank: int, perm) -> OpShardingRule:
    return OpShardingRule([{i: [f"d{i}"] for i in range(rank)}], [{j: [f"d{p}"] for j, p in enumerate(perm)}])


class UnsqueezeOp(AxisOp):
    partial_policy = "any"
    axis_offset_for_insert = True

    def logical_rank_for_axis(self, rank, kwargs):
        return rank + 1

    def kernel(self, x, *, axis: int):
        return x.unsqueeze(axis)

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, **kw):
        rank = len(input_shapes[0])
        outs, j = {}, 0
        for i in range(rank + 1):
            if i == axis:
                outs[i] = [f"new{i}"]
            else:
                outs[i] = [f"d{j}"]
                j += 1
        return OpShardingRule([{i: [f"d{i}"] for i in range(rank)}], [outs])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (squeeze(cot, axis=kwargs["axis"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return unsqueeze(tangents[0], axis=kwargs["axis"])


class SqueezeOp(AxisOp):
    partial_policy = "any"

    def kernel(self, x, *, axis: int):
        if x.shape[axis] != 1:
            raise ValueError(f"cannot squeeze axis {axis} of extent {x.shape[axis]}")
        return x.squeeze(axis)

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, **kw):
        rank = len(input_shapes[0])
        outs, j = {}, 0
        for i in range(rank):
            if i != axis:
                outs[j] = [f"d{i}"]
                j += 1
        return OpShardingRule([{i: [f"d{i}"] for i in range(rank)}], [outs])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (unsqueeze(cot, axis=_pos_axis(kwargs["axis"], primals[0])),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return squeeze(tangents[0], axis=kwargs["axis"])


def _pos_axis(axis: int, x: Tensor) -> int:
    rank = len(x._impl.global_shape)
    return axis + rank if axis < 0 else axis


class SwapAxesOp(AxisOp):
    partial_policy = "any"
    axis_keys = ("axis1", "axis2")

    def kernel(self, x, *, axis1: int, axis2: int):
        return x.transpose(axis1, axis2)

    def sharding_rule(self, input_shapes, output_shapes, *, axis1: int, axis2: int, **kw):
        rank = len(input_shapes[0])
        perm = list(range(rank))
        perm[axis1], perm[axis2] = perm[axis2], perm[axis1]
        return _perm_rule(rank, perm)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (swap_axes(cot, kwargs["axis1"], kwargs["axis2"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return swap_axes(tangents[0], kwargs["axis1"], kwargs["axis2"])


class PermuteOp(Operation):
    partial_policy = "any"

    def adapt_kwargs(self, args, kwargs, batch_dims):
        x = args[0]
        bd = max(batch_dims, x._impl.batch_dims)
        rank = len(x._impl.global_shape)
        order = [_norm_axis(int(a), rank) for a in kwargs["order"]]
        if sorted(order) != list(range(rank)):
            raise ValueError(f"invalid permutation {kwargs['order']} for rank {rank}")
        return {"order": tuple(range(bd)) + tuple(a + bd for a in order)}

    def kernel(self, x, *, order):
        return x.permute(order)

    def sharding_rule(self, input_shapes, output_shapes, *, order, **kw):
        return _perm_rule(len(input_shapes[0]), order)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        rank = len(primals[0]._impl.global_shape)
        order = [a + rank if a < 0 else a for a in kwargs["order"]]
        inv = [0] * rank
        for i, p in enumerate(order):
            inv[p] = i
        return (permute(cot, tuple(inv)),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return permute(tangents[0], kwargs["order"])


class MoveaxisOp(AxisOp):
    partial_policy = "any"
    axis_keys = ("source", "destination")

    def kernel(self, x, *, source: int, destination: int):
        return torch.movedim(x, source, destination)

    def sharding_rule(self, input_shapes, output_shapes, *, source: int, destination: int, **kw):
        rank = len(input_shapes[0])
        perm = [i for i in range(rank) if i != source]
        perm.insert(destination, source)
        return _perm_rule(rank, perm)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (moveaxis(cot, kwargs["destination"], kwargs["source"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return moveaxis(tangents[0], kwargs["source"], kwargs["destination"])


class FlipOp(AxisOp):
    partial_policy = "any"

    def kernel(self, x, *, axis):
        return torch.flip(x, dims=tuple(axis) if isinstance(axis, (tuple, list)) else (axis,))

    def sharding_rule(self, input_shapes, output_shapes, *, axis, **kw):
        rank = len(input_shapes[0])
        ax = set(axis) if isinstance(axis, (tuple, list)) else {axis}
        m = {i: [f"bcast_flip{i}"] if i in ax else [f"d{i}"] for i in range(rank)}
        return OpShardingRule([dict(m)], [dict(m)])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (flip(cot, kwargs["axis"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return flip(tangents[0], kwargs["axis"])


# ---- physical variants -------------------------------------------------------------------
class _Physical:
    """Axes are physical; the number of batch dims changes when a batch axis is added/removed."""

    def adapt_kwargs(self, args, kwargs, batch_dims):
        x = args[0]
        rank = len(x._impl._shape) + (1 if isinstance(self, UnsqueezeOp) else 0)
        a = int(kwargs["axis"])
        return {**kwargs, "axis": a + rank if a < 0 else a}


class UnsqueezePhysicalOp(_Physical, UnsqueezeOp):
    _name = "unsqueeze_physical"

    def output_batch_dims(self, batch_dims, kwargs):
        return batch_dims + 1 if kwargs["axis"] < batch_dims else batch_dims

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (squeeze_physical(cot, axis=kwargs["axis"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return unsqueeze_physical(tangents[0], axis=kwargs["axis"])


class SqueezePhysicalOp(_Physical, SqueezeOp):
    _name = "squeeze_physical"

    def output_batch_dims(self, batch_dims, kwargs):
        return batch_dims - 1 if kwargs["axis"] < batch_dims else batch_dims

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (unsqueeze_physical(cot, axis=kwargs["axis"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return squeeze_physical(tangents[0], axis=kwargs["axis"])


_unsqueeze, _squeeze, _swap, _permute, _moveaxis, _flip = (UnsqueezeOp(), SqueezeOp(), SwapAxesOp(), PermuteOp(),
                                                          MoveaxisOp(), FlipOp())
_unsqueeze_p, _squeeze_p = UnsqueezePhysicalOp(), SqueezePhysicalOp()


def unsqueeze(x, axis: int = 0) -> Tensor:
    x = ensure_tensor(x)
    if isinstance(axis, (tuple, list)):
        rank = len(x._impl.global_shape) + len(axis)
        for a in sorted(int(v) + rank if int(v) < 0 else int(v) for v in axis):
            x = _unsqueeze(x, axis=a)
        return x
    return _unsqueeze(x, axis=int(axis))


def squeeze(x, axis=0) -> Tensor:
    """Remove the size-1 dimension at ``axis`` (default 0, as in the reference,
    nabla/ops/view/axes.py:413); a tuple removes several, ``None`` every size-1 dimension."""
    x = ensure_tensor(x)
    rank = len(x._impl.global_shape)
    if axis is None:
        axis = tuple(i for i, d in enumerate(x._impl.global_shape) if d == 1)
    if isinstance(axis, (tuple, list)):
        for a in sorted((int(v) + rank if int(v) < 0 else int(v) for v in axis), reverse=True):
            x = _squeeze(x, axis=a)
        return x
    return _squeeze(x, axis=int(axis))


def swap_axes(x, axis1: int, axis2: int) -> Tensor:
    return _swap(ensure_tensor(x), axis1=int(axis1), axis2=int(axis2))


transpose = swap_axes


def permute(x, order) -> Tensor:
    return _permute(ensure_tensor(x), order=tuple(int(a) for a in order))


def moveaxis(x, source: int, destination: int) -> Tensor:
    return _moveaxis(ensure_tensor(x), source=int(source), destination=int(destination))


def flip(x, axis) -> Tensor:
    if isinstance(axis, (tuple, list)):
        axis = tuple(int(a) for a in axis)
    else:
        axis = int(axis)
    return _flip(ensure_tensor(x), axis=axis)


def unsqueeze_physical(x, axis: int = 0) -> Tensor:
    return _unsqueeze_p(x, axis=int(axis))


def squeeze_physical(x, axis: int = 0) -> Tensor:
    return _squeeze_p(x, axis=int(axis))

MoveAxisOp = MoveaxisOp      # spelling of the reference (nabla/ops/view/axes.py)
