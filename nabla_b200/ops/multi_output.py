"""Ops with several outputs (reference: nabla/ops/multi_output.py:52-546): split (tuple),
chunk (list, sizes differ by at most one), unbind (tuple), minmax (dict). The split axis must be whole on
every shard, so a sharded split axis is gathered first."""
from __future__ import annotations

import torch

from ..core.sharding.propagation import OpShardingRule
from ..core.tensor.api import Tensor
from .base import AxisOp, ensure_tensor


class _SplitBase(AxisOp):
    partial_policy = "any"

    def _rule(self, rank, axis, n_out, drop=False):
        ins = {i: [f"d{i}"] if i != axis else [f"bcast_sp{i}"] for i in range(rank)}
        outs = []
        for k in range(n_out):
            m, j = {}, 0
            for i in range(rank):
                if i == axis:
                    if drop:
                        continue
                    m[j] = [f"piece{k}"]
                else:
                    m[j] = [f"d{i}"]
                j += 1
            outs.append(m)
        return OpShardingRule([ins], outs)


class SplitOp(_SplitBase):
    def kernel(self, x, *, sizes, axis: int):
        return tuple(torch.split(x, list(sizes), dim=axis))

    def sharding_rule(self, input_shapes, output_shapes, *, sizes, axis: int, **kw):
        return self._rule(len(input_shapes[0]), axis, len(sizes))

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .creation import zeros
        from .view import concatenate

        x = primals[0]
        shp = list(x._impl.global_shape)
        ax = kwargs["axis"] + len(shp) if kwargs["axis"] < 0 else kwargs["axis"]
        cots = []
        for c, n in zip(cot, kwargs["sizes"]):
            if c is None:   # this piece was not used downstream
                c = zeros(tuple(shp[:ax] + [int(n)] + shp[ax + 1:]), dtype=x.dtype, device=x.device)
            cots.append(c)
        return (concatenate(cots, axis=kwargs["axis"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _split(tangents[0], **kwargs)


class UnbindOp(_SplitBase):
    def kernel(self, x, *, axis: int):
        return tuple(torch.unbind(x, dim=axis))

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, **kw):
        return self._rule(len(input_shapes[0]), axis, input_shapes[0][axis], drop=True)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .creation import zeros
        from .view import stack

        x = primals[0]
        shp = list(x._impl.global_shape)
        ax = kwargs["axis"] + len(shp) if kwargs["axis"] < 0 else kwargs["axis"]
        piece = tuple(shp[:ax] + shp[ax + 1:])
        cots = [c if c is not None else zeros(piece, dtype=x.dtype, device=x.device) for c in cot]
        return (stack(cots, axis=kwargs["axis"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _unbind(tangents[0], **kwargs)


class MinMaxOp(AxisOp):
    collective_reduce_type = "max"

    def kernel(self, x, *, axis: int, keepdims: bool = False):
        return {"min": torch.amin(x, dim=axis, keepdim=keepdims), "max": torch.amax(x, dim=axis, keepdim=keepdims)}

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, keepdims: bool = False, **kw):
        rank = len(input_shapes[0])
        ins = {i: [f"d{i}"] if i != axis else [f"bcast_mm{i}"] for i in range(rank)}
        m, j = {}, 0
        for i in range(rank):
            if i == axis and not keepdims:
                continue
            m[j] = [f"d{i}"] if i != axis else ["one"]
            j += 1
        return OpShardingRule([ins], [dict(m), dict(m)])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .reduction import _reduce_max, _reduce_min

        x = primals[0]
        g = None
        for key, op in (("max", _reduce_max), ("min", _reduce_min)):
            c = cot.get(key) if isinstance(cot, dict) else None
            if c is None:
                continue
            (gi,) = op.vjp_rule((x,), c, outputs[key], kwargs)
            g = gi if g is None else g + gi
        return (g,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        from .reduction import _reduce_max, _reduce_min

        return {"max": _reduce_max.jvp_rule(primals, tangents, outputs["max"], kwargs),
                "min": _reduce_min.jvp_rule(primals, tangents, outputs["min"], kwargs)}


class ChunkOp(SplitOp):
    """`split` as issued by `chunk` (sizes differ by at most one); shows as ``chunk`` in a trace."""

    _name = "chunk"

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _chunk(tangents[0], **kwargs)


_split, _unbind, _minmax, _chunk = SplitOp(), UnbindOp(), MinMaxOp(), ChunkOp()


def split(x, num_splits=None, axis: int = 0, *, num_or_sizes=None) -> tuple[Tensor, ...]:
    """Split into ``num_splits`` equal parts (int, the reference's form, nabla/ops/multi_output.py:481)
    or into the given sizes (list)."""
    if num_splits is None:
        num_splits = num_or_sizes
    if num_splits is None:
        raise TypeError("split() needs the number of parts or their sizes")
    num_or_sizes = num_splits
    x = ensure_tensor(x)
    rank = len(x._impl.global_shape)
    n = x._impl.global_shape[axis + rank if axis < 0 else axis]
    if isinstance(num_or_sizes, int):
        if n % num_or_sizes != 0:
            raise ValueError(f"axis of size {n} is not divisible into {num_or_sizes} parts")
        sizes = (n // num_or_sizes,) * num_or_sizes
    else:
        sizes = tuple(int(s) for s in num_or_sizes)
        if sum(sizes) != n:
            raise ValueError(f"split sizes {sizes} do not sum to {n}")
    return tuple(_split(x, sizes=sizes, axis=int(axis)))


def chunk(x, chunks: int, axis: int = 0) -> list[Tensor]:
    """``chunks`` pieces whose sizes differ by at most one, the larger ones first (numpy's
    ``array_split``; reference: nabla/ops/multi_output.py:219-226). Empty pieces are dropped, so an
    axis shorter than ``chunks`` gives one piece per element."""
    x = ensure_tensor(x)
    rank = len(x._impl.global_shape)
    n = x._impl.global_shape[axis + rank if axis < 0 else axis]
    div, rem = divmod(int(n), int(chunks))
    sizes = [div + 1 if i < rem else div for i in range(int(chunks))]
    return list(_chunk(x, sizes=tuple(s for s in sizes if s > 0), axis=int(axis)))


def unbind(x, axis: int = 0) -> tuple[Tensor, ...]:
    return tuple(_unbind(ensure_tensor(x), axis=int(axis)))


def minmax(x, axis: int | None = None, keepdims: bool = False) -> dict[str, Tensor]:
    """``{"min": ..., "max": ...}``. Without ``axis`` both are scalars over the whole tensor (the
    reference's form, nabla/ops/multi_output.py:528-538); with ``axis`` they are taken along it."""
    x = ensure_tensor(x)
    if axis is not None:
        return _minmax(x, axis=int(axis), keepdims=keepdims)
    rank = len(x._impl.global_shape)
    if rank == 0:
        return {"min": x, "max": x}
    out = _minmax(x, axis=rank - 1, keepdims=keepdims)
    lo, hi = out["min"], out["max"]
    from .reduction import reduce_max, reduce_min

    for ax in reversed(range(rank - 1)):
        lo = reduce_min(lo, axis=ax, keepdims=keepdims)
        hi = reduce_max(hi, axis=ax, keepdims=keepdims)
    return {"min": lo, "max": hi}
