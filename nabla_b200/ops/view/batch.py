"""vmap plumbing (reference: nabla/ops/view/batch.py:57-447).

``batch_dims`` counts leading physical dimensions that are invisible to the user's function.
These ops move dimensions between the logical and the batch part without touching data
(except ``moveaxis_physical`` / ``broadcast_batch_dims``).
"""
from __future__ import annotations

import torch

from ...core.sharding.propagation import OpShardingRule
from ...core.tensor.api import Tensor
from ..base import Operation, ensure_tensor


class _Identity(Operation):
    partial_policy = "any"
    delta = 0

    def kernel(self, x):
        return x

    def output_batch_dims(self, batch_dims, kwargs):
        return batch_dims + self.delta


class IncrBatchDimsOp(_Identity):
    delta = 1

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (decr_batch_dims(cot),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return incr_batch_dims(tangents[0])


class DecrBatchDimsOp(_Identity):
    delta = -1

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (incr_batch_dims(cot),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return decr_batch_dims(tangents[0])


class MoveaxisPhysicalOp(Operation):
    partial_policy = "any"

    def adapt_kwargs(self, args, kwargs, batch_dims):
        rank = len(args[0]._impl._shape)
        s, d = int(kwargs["source"]), int(kwargs["destination"])
        return {"source": s + rank if s < 0 else s, "destination": d + rank if d < 0 else d}

    def kernel(self, x, *, source: int, destination: int):
        return torch.movedim(x, source, destination)

    def sharding_rule(self, input_shapes, output_shapes, *, source: int, destination: int, **kw):
        rank = len(input_shapes[0])
        perm = [i for i in range(rank) if i != source]
        perm.insert(destination, source)
        return OpShardingRule([{i: [f"d{i}"] for i in range(rank)}], [{j: [f"d{p}"] for j, p in enumerate(perm)}])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (moveaxis_physical(cot, kwargs["destination"], kwargs["source"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return moveaxis_physical(tangents[0], kwargs["source"], kwargs["destination"])


class BroadcastBatchDimsOp(Operation):
    """Prepend missing batch dims (broadcast) so the tensor has ``batch_shape`` in front."""

    partial_policy = "any"

    def kernel(self, x, *, batch_shape, own: int):
        missing = len(batch_shape) - own
        if missing <= 0:
            return x
        x = x.reshape(*([1] * missing), *x.shape)
        return x.expand(*batch_shape[:missing], *x.shape[missing:])

    def output_batch_dims(self, batch_dims, kwargs):
        return len(kwargs["batch_shape"])

    def sharding_rule(self, input_shapes, output_shapes, *, batch_shape, own: int, **kw):
        rank = len(input_shapes[0])
        missing = len(batch_shape) - own
        return OpShardingRule([{i: [f"d{i}"] for i in range(rank)}],
                              [{**{j: [f"nb{j}"] for j in range(missing)},
                                **{i + missing: [f"d{i}"] for i in range(rank)}}])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from ..reduction import reduce_sum_physical

        missing = len(kwargs["batch_shape"]) - kwargs["own"]
        for _ in range(missing):
            cot = reduce_sum_physical(cot, axis=0, keepdims=False)
        return (cot,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return broadcast_batch_dims(tangents[0], kwargs["batch_shape"])


_incr, _decr, _move_p, _bbd = IncrBatchDimsOp(), DecrBatchDimsOp(), MoveaxisPhysicalOp(), BroadcastBatchDimsOp()


def incr_batch_dims(x) -> Tensor:
    return _incr(ensure_tensor(x))


def decr_batch_dims(x) -> Tensor:
    x = ensure_tensor(x)
    if x._impl.batch_dims <= 0:
        raise ValueError("decr_batch_dims on a tensor without batch dims")
    return _decr(x)


def moveaxis_physical(x, source: int, destination: int) -> Tensor:
    x = ensure_tensor(x)
    rank = len(x._impl._shape)
    s = source + rank if source < 0 else source
    d = destination + rank if destination < 0 else destination
    if s == d:
        return x
    return _move_p(x, source=s, destination=d)


def move_axis_to_batch_dims(x, axis: int) -> Tensor:
    """Logical ``axis`` becomes the innermost... outermost batch dim (physical position 0)."""
    x = ensure_tensor(x)
    rank = len(x._impl.global_shape)
    a = axis + rank if axis < 0 else axis
    return incr_batch_dims(moveaxis_physical(x, x._impl.batch_dims + a, 0))


def move_axis_from_batch_dims(x, batch_axis: int = 0, logical_destination: int = 0) -> Tensor:
    x = ensure_tensor(x)
    bd = x._impl.batch_dims
    out_rank = len(x._impl.global_shape) + 1
    dest = logical_destination + out_rank if logical_destination < 0 else logical_destination
    ba = batch_axis + bd if batch_axis < 0 else batch_axis
    # move the chosen batch axis to the end of the batch block, drop it from the batch dims,
    # then place it inside the logical block
    x = moveaxis_physical(x, ba, bd - 1)
    x = decr_batch_dims(x)
    return moveaxis_physical(x, bd - 1, bd - 1 + dest)


def broadcast_batch_dims(x, batch_shape) -> Tensor:
    x = ensure_tensor(x)
    batch_shape = tuple(int(b) for b in batch_shape)
    if x._impl.batch_dims >= len(batch_shape):
        return x
    return _bbd(x, batch_shape=batch_shape, own=x._impl.batch_dims)

MoveAxisPhysicalOp = MoveaxisPhysicalOp      # spelling of the reference (nabla/ops/view/batch.py)
