"""Reductions (reference: nabla/ops/reduction.py:67-955).

Single-axis primitives with ``keepdims``; multi-axis and ``axis=None`` forms chain them.
Reducing over a sharded dimension leaves a pending cross-device reduction: sum stays deferred
(``partial_sum_axes``), max/min are resolved immediately with a max/min collective.
"""
from __future__ import annotations

import torch

from ..core.tensor.api import Tensor
from ..types import DType
from .base import AxisOp, ReduceOperation, UnaryOperation, ensure_tensor


def _empty_reduce(x, axis, keepdims, value):
    shp = list(x.shape)
    if keepdims:
        shp[axis] = 1
    else:
        del shp[axis]
    return torch.full(shp, value, dtype=x.dtype, device=x.device)


class ReduceSumOp(ReduceOperation):
    native_op = "sum"

    def torch_reduce(self, x, axis, keepdims):
        if x.dtype == torch.bool:
            x = x.to(torch.int64)
        return torch.sum(x, dim=axis, keepdim=keepdims)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .. import config
        from .view import broadcast_to, unsqueeze

        x = primals[0]
        if config.debug_stream("PHYS_VJP"):
            for tag, t in (("reduce_sum.vjp primal", x), ("reduce_sum.vjp cotangent", cot)):
                print(f"[NABLA_DEBUG_PHYS_VJP] {tag}: shape={tuple(t._impl.global_shape)} "
                      f"batch_dims={t._impl.batch_dims} phys={tuple(t._impl._shape)}")
        if not kwargs.get("keepdims", False):
            cot = unsqueeze(cot, axis=kwargs["axis"])
        return (broadcast_to(cot, tuple(x._impl.global_shape)),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _reduce_sum(tangents[0], **kwargs)


class _ReduceExt(ReduceOperation):
    def _global_extreme(self, y):
        """The op's own output over a sharded axis is the per-shard extreme (labelled as a
        pending reduction); the derivative needs the extreme over all shards."""
        sp = y._impl.sharding
        if sp is None or not sp.partial_sum_axes:
            return y
        from .communication import all_reduce, relabel_spec

        axes = set(sp.partial_sum_axes)
        plain = sp.clone()
        plain.partial_sum_axes = set()
        return all_reduce(relabel_spec(y, plain), reduce_axes=axes, reduce_op=self.collective_reduce_type)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .comparison import equal
        from .unary import cast
        from .view import broadcast_to, unsqueeze

        x = primals[0]
        y = self._global_extreme(outputs)
        if not kwargs.get("keepdims", False):
            cot = unsqueeze(cot, axis=kwargs["axis"])
            y = unsqueeze(y, axis=kwargs["axis"])
        shape = tuple(x._impl.global_shape)
        mask = cast(equal(x, broadcast_to(y, shape)), x.dtype)
        count = _reduce_sum(mask, axis=kwargs["axis"], keepdims=True)
        return (broadcast_to(cot, shape) * mask / count,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        from .comparison import equal
        from .unary import cast
        from .view import broadcast_to, unsqueeze

        x = primals[0]
        y = self._global_extreme(outputs)
        y = y if kwargs.get("keepdims", False) else unsqueeze(y, axis=kwargs["axis"])
        mask = cast(equal(x, broadcast_to(y, tuple(x._impl.global_shape))), x.dtype)
        count = _reduce_sum(mask, axis=kwargs["axis"], keepdims=True)
        return _reduce_sum(tangents[0] * mask / count, **kwargs)


class ReduceMaxOp(_ReduceExt):
    native_op = "max"
    collective_reduce_type = "max"

    def torch_reduce(self, x, axis, keepdims):
        if x.shape[axis] == 0:   # empty trailing shard: identity of max
            return _empty_reduce(x, axis, keepdims, float("-inf"))
        return torch.amax(x, dim=axis, keepdim=keepdims)


class ReduceMinOp(_ReduceExt):
    native_op = "min"
    collective_reduce_type = "min"

    def torch_reduce(self, x, axis, keepdims):
        if x.shape[axis] == 0:
            return _empty_reduce(x, axis, keepdims, float("inf"))
        return torch.amin(x, dim=axis, keepdim=keepdims)


class _ArgOp(AxisOp):
    fn = None

    native_op = None

    def kernel(self, x, *, axis: int, keepdims: bool = False):
        if self.native_op is not None and x.is_cuda and x.dim() and x.shape[axis] > 0:
            from ..native import kernels

            out = kernels.reduce(x, axis, self.native_op, keepdims)
            if out is not None:
                return out
        return type(self).fn(x, dim=axis, keepdim=keepdims)

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, keepdims: bool = False, **kw):
        # the searched axis must be whole on every shard: give it a factor nobody shards
        from ..core.sharding.propagation import OpShardingRule

        rank = len(input_shapes[0])
        ins = {i: [f"d{i}"] if i != axis else [f"bcast_arg{i}"] for i in range(rank)}
        outs, j = {}, 0
        for i in range(rank):
            if i == axis and not keepdims:
                continue
            outs[j] = [f"d{i}"] if i != axis else [f"one{i}"]
            j += 1
        return OpShardingRule([ins], [outs])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (None,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return None


class ArgmaxOp(_ArgOp):
    fn = staticmethod(torch.argmax)
    native_op = "argmax"


class ArgminOp(_ArgOp):
    fn = staticmethod(torch.argmin)
    native_op = "argmin"


class CumsumOp(AxisOp):
    def kernel(self, x, *, axis: int, exclusive: bool = False, reverse: bool = False):
        if x.is_cuda:
            from ..native import kernels

            out = kernels.cumsum(x, axis, exclusive, reverse)
            if out is not None:
                return out
        if reverse:
            x = torch.flip(x, dims=(axis,))
        y = torch.cumsum(x, dim=axis)
        if exclusive:
            y = y - x
        if reverse:
            y = torch.flip(y, dims=(axis,))
        return y

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, **kw):
        from ..core.sharding.propagation import OpShardingRule

        rank = len(input_shapes[0])
        m = {i: [f"d{i}"] if i != axis else [f"bcast_scan{i}"] for i in range(rank)}
        return OpShardingRule([dict(m)], [dict(m)])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        kw = dict(kwargs)
        kw["reverse"] = not kwargs.get("reverse", False)
        return (_cumsum(cot, **kw),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _cumsum(tangents[0], **kwargs)


_reduce_sum, _reduce_max, _reduce_min = ReduceSumOp(), ReduceMaxOp(), ReduceMinOp()
_argmax, _argmin, _cumsum = ArgmaxOp(), ArgminOp(), CumsumOp()


def _axes(x: Tensor, axis) -> list[int]:
    rank = len(x._impl.global_shape)
    if axis is None:
        return list(range(rank))
    if isinstance(axis, (tuple, list)):
        ax = [int(a) + rank if int(a) < 0 else int(a) for a in axis]
    else:
        ax = [int(axis) + rank if int(axis) < 0 else int(axis)]
    for a in ax:
        if not 0 <= a < max(rank, 1):
            raise ValueError(f"axis {axis} out of range for rank {rank}")
    return sorted(set(ax))


def _chain(op, x: Tensor, axis, keepdims: bool) -> Tensor:
    x = ensure_tensor(x)
    if len(x._impl.global_shape) == 0:
        return x
    axes = _axes(x, axis)
    # reduce from the last axis so earlier indices stay valid when dims are dropped
    for a in reversed(axes):
        x = op(x, axis=a, keepdims=keepdims)
    return x


def reduce_sum(x, *, axis=None, keepdims: bool = False) -> Tensor:
    return _chain(_reduce_sum, x, axis, keepdims)


def reduce_max(x, *, axis=None, keepdims: bool = False) -> Tensor:
    return _chain(_reduce_max, x, axis, keepdims)


def reduce_min(x, *, axis=None, keepdims: bool = False) -> Tensor:
    return _chain(_reduce_min, x, axis, keepdims)


class DivideByCountOp(UnaryOperation):
    """``x / count`` with ``count`` an INTEGER kwarg: the second half of a mean. Kept as an op of its
    own, and not as a product with the float ``1.0 / count``, because ``compile(dynamic_dims=...)``
    re-evaluates integers that follow a dynamic size and cannot do that for a float computed from
    one: a mean over the batch stays on the path that never re-runs Python for a new batch size."""

    partial_policy = "any"
    _name = "divide_by_count"

    def kernel(self, x, *, count: int):
        return x / max(int(count), 1)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (_div_count(cot, **kwargs),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _div_count(tangents[0], **kwargs)


_div_count = DivideByCountOp()


def mean(x, *, axis=None, keepdims: bool = False) -> Tensor:
    x = ensure_tensor(x)
    axes = _axes(x, axis)
    n = 1
    for a in axes:
        n *= x._impl.global_shape[a]
    s = reduce_sum(x, axis=axis, keepdims=keepdims)
    return _div_count(s, count=int(n))


class MeanOp(ReduceSumOp):
    """``mean`` under the reference's op name (nabla/ops/reduction.py). Calling the op gives the
    same composition as ``mean``: a sum (all-reduced when the axis is sharded) scaled by one over the
    GLOBAL extent, so sharded inputs need no rule of their own."""

    _name = "mean"

    def __call__(self, x, *, axis=None, keepdims: bool = False):
        return mean(x, axis=axis, keepdims=keepdims)


class MeanPhysicalOp(MeanOp):
    """``mean_physical`` under the reference's op name: the axis indexes the physical shape."""

    _name = "mean_physical"

    def __call__(self, x, *, axis: int, keepdims: bool = False):
        return mean_physical(x, axis=axis, keepdims=keepdims)


def argmax(x, axis: int = -1, keepdims: bool = False) -> Tensor:
    return _argmax(ensure_tensor(x), axis=axis, keepdims=keepdims)


def argmin(x, axis: int = -1, keepdims: bool = False) -> Tensor:
    return _argmin(ensure_tensor(x), axis=axis, keepdims=keepdims)


def cumsum(x, axis: int = -1, exclusive: bool = False, reverse: bool = False) -> Tensor:
    return _cumsum(ensure_tensor(x), axis=axis, exclusive=exclusive, reverse=reverse)


# ---- physical variants: axes index the physical shape (batch dims included); used by vmap
class _PhysMixin:
    def adapt_kwargs(self, args, kwargs, batch_dims):
        out = dict(kwargs)
        t = args[0]
        rank = len(t._impl._shape)
        a = int(out["axis"])
        out["axis"] = a + rank if a < 0 else a
        return out

    def output_batch_dims(self, batch_dims, kwargs):
        if kwargs["axis"] < batch_dims and not kwargs.get("keepdims", False):
            return batch_dims - 1
        return batch_dims


def _restore_reduced_axis(cot, x, outputs, kwargs):
    """Give the cotangent of a physical reduction its reduced axis back (size 1). When that axis was
    one of ``x``'s vmap dims, it comes back as a vmap dim, so the result lines up with ``x``."""
    from .view.axes import unsqueeze_physical
    from .view.batch import incr_batch_dims

    if kwargs.get("keepdims", False):
        return cot
    lead = cot._impl.batch_dims - outputs._impl.batch_dims      # vmap dims that only the cotangent has
    cot = unsqueeze_physical(cot, axis=kwargs["axis"] + max(lead, 0))
    if kwargs["axis"] < x._impl.batch_dims and cot._impl.batch_dims - max(lead, 0) < x._impl.batch_dims:
        cot = incr_batch_dims(cot)
    return cot


PhysicalReduceOp = _PhysMixin     # what every *_physical reduction derives from (reference: reduction.py:67)


class ReduceSumPhysicalOp(_PhysMixin, ReduceSumOp):
    _name = "reduce_sum_physical"

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .view.shape import broadcast_to_physical

        x = primals[0]
        cot = _restore_reduced_axis(cot, x, outputs, kwargs)
        lead = tuple(cot._impl._shape[:len(cot._impl._shape) - len(x._impl._shape)])
        return (broadcast_to_physical(cot, lead + tuple(x._impl._shape)),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return reduce_sum_physical(tangents[0], **kwargs)


_reduce_sum_physical = ReduceSumPhysicalOp()


def reduce_sum_physical(x, axis: int, keepdims: bool = False) -> Tensor:
    return _reduce_sum_physical(x, axis=axis, keepdims=keepdims)


class _PhysExtremeMixin(_PhysMixin):
    """Derivative rules of max / min over a physical axis: the cotangent (tangent) goes to (comes
    from) the positions that hold the extreme value, shared equally between ties."""

    def _mask(self, x, outputs, kwargs):
        from .comparison import equal
        from .unary import cast
        from .view.axes import unsqueeze_physical
        from .view.shape import broadcast_to_physical

        y = outputs if kwargs.get("keepdims", False) else unsqueeze_physical(outputs, axis=kwargs["axis"])
        shape = tuple(x._impl._shape)
        mask = cast(equal(x, broadcast_to_physical(y, shape)), x.dtype)
        count = reduce_sum_physical(mask, axis=kwargs["axis"], keepdims=True)
        return mask / broadcast_to_physical(count, shape), shape

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .view.axes import unsqueeze_physical
        from .view.shape import broadcast_to_physical

        w, shape = self._mask(primals[0], outputs, kwargs)
        cot = _restore_reduced_axis(cot, primals[0], outputs, kwargs)
        lead = tuple(cot._impl._shape[:len(cot._impl._shape) - len(shape)])
        return (broadcast_to_physical(cot, lead + tuple(shape)) * w,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        w, _ = self._mask(primals[0], outputs, kwargs)
        return reduce_sum_physical(tangents[0] * w, **kwargs)


class ReduceMaxPhysicalOp(_PhysExtremeMixin, ReduceMaxOp):
    _name = "reduce_max_physical"


class ReduceMinPhysicalOp(_PhysExtremeMixin, ReduceMinOp):
    _name = "reduce_min_physical"


_reduce_max_physical, _reduce_min_physical = ReduceMaxPhysicalOp(), ReduceMinPhysicalOp()


def reduce_max_physical(x, axis: int, keepdims: bool = False) -> Tensor:
    """Maximum over a PHYSICAL axis (batch dimensions count; reference: nabla/ops/reduction.py:712)."""
    return _reduce_max_physical(x, axis=axis, keepdims=keepdims)


def reduce_min_physical(x, axis: int, keepdims: bool = False) -> Tensor:
    """Minimum over a PHYSICAL axis (reference: nabla/ops/reduction.py:735)."""
    return _reduce_min_physical(x, axis=axis, keepdims=keepdims)


def mean_physical(x, axis: int, keepdims: bool = False) -> Tensor:
    n = x._impl._shape[axis]
    return _div_count(reduce_sum_physical(x, axis=axis, keepdims=keepdims), count=int(n))
