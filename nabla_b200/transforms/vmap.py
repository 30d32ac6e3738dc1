"""``vmap`` (reference: nabla/transforms/vmap.py:68-363).

The mapped axis of every input is moved to the front of the physical shape and counted as a
*batch dim*; the user's function then runs unchanged on tensors whose logical shape lacks that
axis (ops translate their axis arguments past the batch dims). Outputs get the batch dim moved
to ``out_axes``. With ``spmd_axis_name`` the batch axis is split over that mesh axis, which is
how pipeline stages are expressed: ``vmap(stage_fn, spmd_axis_name='stage', mesh=mesh)``.
"""
from __future__ import annotations

from typing import Any, Callable

from ..core.common import pytree
from ..core.tensor.api import Tensor


def _broadcast_axes(axes: Any, n: int) -> tuple:
    if isinstance(axes, (list, tuple)) and not isinstance(axes, str):
        if len(axes) != n:
            raise ValueError(f"axes spec of length {len(axes)} for {n} arguments")
        return tuple(axes)
    return (axes,) * n


def _walk_prefix(fn: Callable, tree: Any, axis_spec: Any, *extra) -> Any:
    """Apply ``fn(tensor, axis, *extra)`` with ``axis_spec`` a prefix of ``tree``'s structure."""
    if isinstance(tree, Tensor):
        if isinstance(axis_spec, (list, tuple, dict)):
            raise ValueError("axis spec is deeper than the argument structure")
        return fn(tree, axis_spec, *extra)
    if axis_spec is None or isinstance(axis_spec, int):
        return pytree.tree_map(lambda t: fn(t, axis_spec, *extra) if isinstance(t, Tensor) else t, tree)
    if isinstance(tree, (list, tuple)) and isinstance(axis_spec, (list, tuple)):
        if len(tree) != len(axis_spec):
            raise ValueError("axis spec does not match the argument structure")
        out = [_walk_prefix(fn, t, a, *extra) for t, a in zip(tree, axis_spec)]
        return type(tree)(out) if not hasattr(tree, "_fields") else type(tree)(*out)
    if isinstance(tree, dict) and isinstance(axis_spec, dict):
        return {k: _walk_prefix(fn, v, axis_spec[k], *extra) for k, v in tree.items()}
    leaves_t, td = pytree.tree_flatten(tree)
    spec_leaves = pytree.tree_leaves(axis_spec, is_leaf=lambda x: x is None or isinstance(x, int))
    if len(leaves_t) == len(spec_leaves):
        return pytree.tree_unflatten(td, [fn(t, a, *extra) if isinstance(t, Tensor) else t
                                          for t, a in zip(leaves_t, spec_leaves)])
    raise ValueError("axis spec does not match the argument structure")


def _batch_size(args, in_ax, axis_size) -> int:
    sizes = set()

    def visit(t, ax):
        if ax is not None:
            rank = len(t._impl.global_shape)
            a = ax + rank if ax < 0 else ax
            if not 0 <= a < rank:
                raise ValueError(f"vmap axis {ax} out of range for shape {tuple(t._impl.global_shape)}")
            sizes.add(t._impl.global_shape[a])
        return t

    for arg, ax in zip(args, in_ax):
        _walk_prefix(visit, arg, ax)
    if axis_size is not None:
        sizes.add(int(axis_size))
    if not sizes:
        raise ValueError("vmap needs axis_size when no input is mapped")
    if len(sizes) != 1:
        raise ValueError(f"vmap got inconsistent sizes for the mapped axes: {sorted(sizes)}")
    return sizes.pop()


def _shard_batch_axis(t: Tensor, old_bd: int, axis_name: str, mesh) -> Tensor:
    """Split physical dim ``old_bd`` (the axis about to become a batch dim) over ``axis_name``."""
    from ..core.sharding.spec import DimSpec
    from ..ops.communication import shard

    cur = t._impl.sharding
    rank = len(t._impl._shape)
    specs = [cur.dim_specs[i].clone() if cur is not None and i < len(cur.dim_specs) else DimSpec([]) for i in range(rank)]
    for s in specs:
        if axis_name in s.axes:
            s.axes = [a for a in s.axes if a != axis_name]
    specs[old_bd] = DimSpec([axis_name])
    rep = set(cur.replicated_axes) - {axis_name} if cur is not None else set()
    par = set(cur.partial_sum_axes) - {axis_name} if cur is not None else set()
    return shard(t, mesh, specs, replicated_axes=rep, partial_sum_axes=par)


def _batch_tensor(t: Tensor, axis, size: int, spmd_axis_name, mesh) -> Tensor:
    from ..ops import view as V

    old_bd = t._impl.batch_dims
    if axis is None:
        x = V.unsqueeze(t, axis=0)
        if size != 1:
            x = V.broadcast_to(x, (size,) + tuple(t._impl.global_shape))
    else:
        rank = len(t._impl.global_shape)
        a = axis + rank if axis < 0 else axis
        x = V.moveaxis_physical(t, old_bd + a, old_bd) if a != 0 else t
    if spmd_axis_name is not None and mesh is not None:
        x = _shard_batch_axis(x, old_bd, spmd_axis_name, mesh)
    x = V.incr_batch_dims(x)
    if old_bd > 0:
        x = V.moveaxis_physical(x, old_bd, 0)
    return x


def _unbatch_tensor(t: Tensor, axis, spmd_axis_name=None, mesh=None) -> Tensor:
    from ..ops import view as V

    bd = t._impl.batch_dims
    if bd <= 0:
        raise ValueError("vmap output lost its batch dimension")
    x = V.moveaxis_physical(t, 0, bd - 1) if bd > 1 else t
    x = V.decr_batch_dims(x)
    if axis is None:
        return V.squeeze(V.slice_tensor(x, (0,) * len(x._impl.global_shape),
                                        (1,) + tuple(x._impl.global_shape[1:])), axis=0)
    if axis != 0:
        nbd = x._impl.batch_dims
        rank = len(x._impl.global_shape)
        a = axis + rank if axis < 0 else axis
        x = V.moveaxis_physical(x, nbd, nbd + a)
    return x


def vmap(func: Callable | None = None, in_axes: Any = 0, out_axes: Any = 0, axis_size: int | None = None,
         spmd_axis_name: str | None = None, mesh=None) -> Callable:
    """Vectorise ``func`` over one axis of its inputs (usable as a decorator)."""
    if func is None:
        return lambda f: vmap(f, in_axes=in_axes, out_axes=out_axes, axis_size=axis_size,
                              spmd_axis_name=spmd_axis_name, mesh=mesh)

    def vectorized(*args: Any) -> Any:
        if not args:
            raise ValueError("vmap requires at least one input argument.")
        in_ax = _broadcast_axes(in_axes, len(args))
        size = _batch_size(args, in_ax, axis_size)
        batched = tuple(_walk_prefix(_batch_tensor, a, ax, size, spmd_axis_name, mesh) for a, ax in zip(args, in_ax))
        outputs = func(*batched)
        single = not isinstance(outputs, (list, tuple))
        outs = [outputs] if single else list(outputs)
        out_ax = _broadcast_axes(out_axes, len(outs))

        def unb(t, ax):
            if not isinstance(t, Tensor):
                return t
            if t._impl.batch_dims == 0:
                # an output that does not depend on mapped inputs: broadcast it
                from ..ops import view as V

                if ax is None:
                    return t
                t = V.broadcast_to(V.unsqueeze(t, axis=0), (size,) + tuple(t._impl.global_shape))
                return V.moveaxis(t, 0, ax) if ax != 0 else t
            return _unbatch_tensor(t, ax, spmd_axis_name, mesh)

        res = [_walk_prefix(unb, o, ax) for o, ax in zip(outs, out_ax)]
        return res[0] if single else type(outputs)(res)

    vectorized.__name__ = f"vmap({getattr(func, '__name__', 'fn')})"
    return vectorized
