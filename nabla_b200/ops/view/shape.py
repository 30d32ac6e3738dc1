"""Shape-changing view ops (reference: nabla/ops/view/shape.py:56-1510): broadcast_to, reshape,
slice_tensor, slice_update, concatenate, stack, pad, flatten, rebind, broadcast_to_physical.

Sharding: dimensions an op leaves intact keep their mesh axes. ``reshape`` keeps a sharded
dimension when it survives as the major part of a split or the major member of a merge and
the extents divide evenly (e.g. splitting a tp-sharded hidden dim into heads); otherwise the
touched dimensions are gathered first, as the reference does for every sharded reshape
(nabla/ops/view/shape.py:170-202). Sliced / padded / concatenated dimensions are gathered.
"""
from __future__ import annotations

import math

import torch

from ...core.sharding.propagation import OpShardingRule
from ...core.tensor.api import Tensor
from ..base import AxisOp, Operation, ShapeOp, _norm_axis, ensure_tensor


def _local_out_shape(node, device_id: int, out_index: int = 0):
    from ...core.sharding.spec import compute_local_shape

    o = node.outputs()[out_index]
    if o is None or o.sharding is None:
        return None
    return compute_local_shape(o._shape, o.sharding, device_id)


# ---------------------------------------------------------------- broadcast_to
class BroadcastToOp(ShapeOp):
    def adapt_kwargs(self, args, kwargs, batch_dims):
        x = args[0]
        bd = max(batch_dims, x._impl.batch_dims)
        return {"shape": tuple(x._impl._shape[:bd]) + tuple(int(s) for s in kwargs["shape"])}

    def kernel(self, x, *, shape):
        # insert the new leading logical dims after the batch dims (physical layout)
        extra = len(shape) - x.dim()
        if extra > 0:
            bd = getattr(self, "_bd", 0)
            x = x.reshape(*x.shape[:bd], *([1] * extra), *x.shape[bd:])
        return x.expand(shape)

    def __call__(self, x, **kwargs):
        self._bd = x._impl.batch_dims
        return super().__call__(x, **kwargs)

    def execute(self, node):
        self._bd = node.input_impls()[0].batch_dims
        return super().execute(node)

    def sharding_rule(self, input_shapes, output_shapes, *, shape, **kw):
        in_shape = input_shapes[0]
        out_rank = len(shape)
        bd = getattr(self, "_bd", 0)
        extra = out_rank - len(in_shape)
        ins = {}
        for i, s in enumerate(in_shape):
            j = i if i < bd else i + extra
            ins[i] = [f"d{j}"] if int(s) == int(shape[j]) else [f"bcast_in{i}"]
        return OpShardingRule([ins], [{j: [f"d{j}"] for j in range(out_rank)}])

    def shard_kwargs(self, kwargs, node, shard_idx, device_id):
        loc = _local_out_shape(node, device_id)
        return kwargs if loc is None else {"shape": loc}

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from ..utils import reduce_to_shape

        return (reduce_to_shape(cot, tuple(primals[0]._impl.global_shape)),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return broadcast_to(tangents[0], kwargs["shape"])


class BroadcastToPhysicalOp(BroadcastToOp):
    """Expand to a full PHYSICAL shape (vmap dims included) of the same rank. `broadcast_to_physical`
    inserts any missing dims first, so the op itself only widens size-1 dims."""

    _name = "broadcast_to_physical"

    def adapt_kwargs(self, args, kwargs, batch_dims):
        return {"shape": tuple(int(s) for s in kwargs["shape"])}

    def kernel(self, x, *, shape):
        return x.expand(shape)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from ..reduction import reduce_sum_physical

        x = primals[0]
        # a cotangent with more vmap dims than the primal keeps them in front: align from the right
        off = len(cot._impl._shape) - len(x._impl._shape)
        for i, s in enumerate(x._impl._shape):
            if s == 1 and cot._impl._shape[i + off] != 1:
                cot = reduce_sum_physical(cot, axis=i + off, keepdims=True)
        return (cot,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        t = tangents[0]
        more = t._impl.batch_dims - primals[0]._impl.batch_dims
        shape = tuple(kwargs["shape"])
        if more > 0:      # the tangent is mapped over dims the primal does not have (jacfwd's basis)
            shape = tuple(t._impl._shape[:more]) + shape
        return broadcast_to_physical(t, shape)


# ---------------------------------------------------------------- reshape
def _reshape_groups(in_shape, out_shape):
    """Minimal groups of consecutive (in dims, out dims) with equal products."""
    groups = []
    i = j = 0
    n, m = len(in_shape), len(out_shape)
    while i < n or j < m:
        gi, gj = [], []
        pi = pj = 1
        if i < n:
            gi.append(i); pi *= in_shape[i]; i += 1
        if j < m:
            gj.append(j); pj *= out_shape[j]; j += 1
        while pi != pj:
            if pi < pj and i < n:
                gi.append(i); pi *= in_shape[i]; i += 1
            elif pj < pi and j < m:
                gj.append(j); pj *= out_shape[j]; j += 1
            else:
                break
        # absorb trailing 1s
        while i < n and in_shape[i] == 1 and (j >= m or out_shape[j] != 1):
            gi.append(i); i += 1
        while j < m and out_shape[j] == 1 and (i >= n or in_shape[i] != 1):
            gj.append(j); j += 1
        groups.append((gi, gj))
    return groups


class ReshapeOp(ShapeOp):
    def adapt_kwargs(self, args, kwargs, batch_dims):
        x = args[0]
        bd = max(batch_dims, x._impl.batch_dims)
        shape = [int(s) for s in kwargs["shape"]]
        if -1 in shape:
            known = -math.prod(shape)
            total = math.prod(x._impl.global_shape)
            shape[shape.index(-1)] = total // known if known else 0
        return {"shape": tuple(x._impl._shape[:bd]) + tuple(shape)}

    def kernel(self, x, *, shape):
        return x.reshape(shape)

    def _plan(self, in_shape, out_shape, spec):
        """factor maps + which input dims keep their sharding."""
        ins, outs = {}, {}
        for gi, gj in _reshape_groups(list(in_shape), list(out_shape)):
            # the dimension that can keep a sharding is the first one of extent > 1 on each side
            lead_i = next((d for d in gi if in_shape[d] != 1), gi[0] if gi else None)
            lead_j = next((d for d in gj if out_shape[d] != 1), gj[0] if gj else None)
            for d in gi:
                ins[d] = [f"bcast_r{d}"]
            for d in gj:
                outs[d] = [f"new_r{d}"]
            if lead_i is None or lead_j is None:
                continue
            if len(gi) == 1 and len(gj) == 1:
                ins[lead_i] = [f"g{lead_i}"]
                outs[lead_j] = [f"g{lead_i}"]
                continue
            shards = 1
            if spec is not None and lead_i < len(spec.dim_specs):
                shards = spec.dim_specs[lead_i].get_total_shards(spec.mesh)
            others_sharded = spec is not None and any(spec.dim_specs[d].axes for d in gi
                                                       if d != lead_i and d < len(spec.dim_specs))
            # dims before the leads must be 1 so that the leads stay the major part
            major_ok = all(in_shape[d] == 1 for d in gi if d < lead_i) and all(out_shape[d] == 1 for d in gj if d < lead_j)
            if (not others_sharded and major_ok and in_shape[lead_i] % shards == 0 and out_shape[lead_j] % shards == 0
                    and (in_shape[lead_i] // shards) * math.prod(in_shape[d] for d in gi if d != lead_i)
                    == (out_shape[lead_j] // shards) * math.prod(out_shape[d] for d in gj if d != lead_j)):
                ins[lead_i] = [f"g{lead_i}"]
                outs[lead_j] = [f"g{lead_i}"]
        return ins, outs

    def sharding_rule(self, input_shapes, output_shapes, *, shape, **kw):
        spec = getattr(self, "_spec", None)
        ins, outs = self._plan(input_shapes[0], shape, spec)
        return OpShardingRule([ins], [outs])

    def __call__(self, x, **kwargs):
        self._spec = x._impl.sharding
        try:
            return super().__call__(x, **kwargs)
        finally:
            self._spec = None

    def shard_kwargs(self, kwargs, node, shard_idx, device_id):
        loc = _local_out_shape(node, device_id)
        return kwargs if loc is None else {"shape": loc}

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (reshape(cot, tuple(primals[0]._impl.global_shape)),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return reshape(tangents[0], kwargs["shape"])


# ---------------------------------------------------------------- slicing
class SliceTensorOp(ShapeOp):
    def adapt_kwargs(self, args, kwargs, batch_dims):
        x = args[0]
        bd = max(batch_dims, x._impl.batch_dims)
        return {"start": (0,) * bd + tuple(int(s) for s in kwargs["start"]),
                "size": tuple(x._impl._shape[:bd]) + tuple(int(s) for s in kwargs["size"])}

    def kernel(self, x, *, start, size):
        idx = tuple(slice(s, s + n) for s, n in zip(start, size))
        return x[idx]

    def sharding_rule(self, input_shapes, output_shapes, *, start, size, **kw):
        shp = input_shapes[0]
        m_in, m_out = {}, {}
        for i, s in enumerate(shp):
            whole = start[i] == 0 and int(size[i]) == int(s)
            m_in[i] = [f"d{i}"] if whole else [f"bcast_s{i}"]
            m_out[i] = [f"d{i}"] if whole else [f"sl{i}"]
        return OpShardingRule([m_in], [m_out])

    def shard_kwargs(self, kwargs, node, shard_idx, device_id):
        loc = _local_out_shape(node, device_id)
        return kwargs if loc is None else {"start": kwargs["start"], "size": loc}

    def vjp_rule(self, primals, cot, outputs, kwargs):
        x = primals[0]
        shape = x._impl.global_shape
        paddings = []
        for s, n, full in zip(kwargs["start"], kwargs["size"], shape):
            paddings.append((int(s), int(full) - int(s) - int(n)))
        return (pad(cot, paddings),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return slice_tensor(tangents[0], start=kwargs["start"], size=kwargs["size"])


class SliceUpdateOp(ShapeOp):
    """Functional ``x[start:start+size] = update``."""

    partial_policy = "all"

    def adapt_kwargs(self, args, kwargs, batch_dims):
        x = args[0]
        bd = max(batch_dims, x._impl.batch_dims)
        return {"start": (0,) * bd + tuple(int(s) for s in kwargs["start"]),
                "size": tuple(x._impl._shape[:bd]) + tuple(int(s) for s in kwargs["size"]),
                "use_buffer_ops": bool(kwargs.get("use_buffer_ops", False))}

    def kernel(self, x, u, *, start, size, use_buffer_ops: bool = False):
        # `use_buffer_ops` records which API asked (`x[...] = v` sets it, `x.at[...]` and
        # `slice_update` do not; reference: nabla/ops/view/shape.py:1065-1077). Both write into a
        # copy: the old value may still be needed by a backward pass.
        out = x.clone()
        idx = tuple(slice(s, s + n) for s, n in zip(start, size))
        out[idx] = u.to(out.dtype)
        return out

    def sharding_rule(self, input_shapes, output_shapes, *, start, size, **kw):
        shp = input_shapes[0]
        mx, mu = {}, {}
        for i, s in enumerate(shp):
            whole = start[i] == 0 and int(size[i]) == int(s)
            mx[i] = [f"d{i}"] if whole else [f"bcast_x{i}"]
            mu[i] = [f"d{i}"] if whole else [f"bcast_u{i}"]
        return OpShardingRule([mx, mu], [dict(mx)])

    def shard_kwargs(self, kwargs, node, shard_idx, device_id):
        u = node.input_impls()[1]
        if u.sharding is None:
            return kwargs
        return {**kwargs, "size": tuple(u._buffers[shard_idx].shape)}

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from ..creation import zeros_like

        x, u = primals
        gx = slice_update(cot, zeros_like(u), start=kwargs["start"], size=kwargs["size"])
        gu = slice_tensor(cot, start=kwargs["start"], size=kwargs["size"])
        return (gx, gu)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return slice_update(tangents[0], tangents[1], start=kwargs["start"], size=kwargs["size"])


# ---------------------------------------------------------------- concatenate / stack
class ConcatenateOp(AxisOp):
    partial_policy = "all"

    def kernel(self, xs, *, axis: int):
        return torch.cat(list(xs), dim=axis)

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, **kw):
        ins = [{i: [f"d{i}"] if i != axis else [f"bcast_c{k}"] for i in range(len(s))}
               for k, s in enumerate(input_shapes)]
        rank = len(input_shapes[0])
        return OpShardingRule(ins, [{i: [f"d{i}"] if i != axis else ["cat"] for i in range(rank)}])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        xs = primals[0]
        rank = len(xs[0]._impl.global_shape)
        ax = kwargs["axis"] + rank if kwargs["axis"] < 0 else kwargs["axis"]
        outs, off = [], 0
        full = list(cot._impl.global_shape)
        for x in xs:
            n = x._impl.global_shape[ax]
            start = [0] * rank
            start[ax] = off
            size = list(full)
            size[ax] = n
            outs.append(slice_tensor(cot, start=tuple(start), size=tuple(size)))
            off += n
        return (outs,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return concatenate(list(tangents[0]), axis=kwargs["axis"])


class StackOp(AxisOp):
    partial_policy = "all"

    def logical_rank_for_axis(self, rank, kwargs):
        return rank + 1

    def kernel(self, xs, *, axis: int):
        return torch.stack(list(xs), dim=axis)

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, **kw):
        rank = len(input_shapes[0])
        ins = [{i: [f"d{i}"] for i in range(rank)} for _ in input_shapes]
        outs, j = {}, 0
        for i in range(rank + 1):
            if i == axis:
                outs[i] = ["stk"]
            else:
                outs[i] = [f"d{j}"]
                j += 1
        return OpShardingRule(ins, [outs])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from ..multi_output import unbind

        return (list(unbind(cot, axis=kwargs["axis"])),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return stack(list(tangents[0]), axis=kwargs["axis"])


# ---------------------------------------------------------------- pad
class PadOp(ShapeOp):
    def adapt_kwargs(self, args, kwargs, batch_dims):
        x = args[0]
        bd = max(batch_dims, x._impl.batch_dims)
        return {"paddings": ((0, 0),) * bd + tuple((int(a), int(b)) for a, b in kwargs["paddings"]),
                "value": kwargs.get("value", 0.0)}

    def kernel(self, x, *, paddings, value=0.0):
        flat = []
        for lo, hi in reversed(paddings):
            flat += [lo, hi]
        return torch.nn.functional.pad(x, flat, mode="constant", value=value)

    def sharding_rule(self, input_shapes, output_shapes, *, paddings, **kw):
        m_in, m_out = {}, {}
        for i, (lo, hi) in enumerate(paddings):
            same = lo == 0 and hi == 0
            m_in[i] = [f"d{i}"] if same else [f"bcast_p{i}"]
            m_out[i] = [f"d{i}"] if same else [f"pad{i}"]
        return OpShardingRule([m_in], [m_out])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        x = primals[0]
        start = tuple(int(lo) for lo, _ in kwargs["paddings"])
        return (slice_tensor(cot, start=start, size=tuple(x._impl.global_shape)),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return pad(tangents[0], kwargs["paddings"], value=0.0)


class RebindOp(ShapeOp):
    """Assert/relabel the shape (a no-op on static shapes)."""

    def adapt_kwargs(self, args, kwargs, batch_dims):
        return {}

    def kernel(self, x):
        return x

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (cot,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return tangents[0]


_broadcast_to, _broadcast_to_p, _reshape = BroadcastToOp(), BroadcastToPhysicalOp(), ReshapeOp()
_slice, _slice_update, _concat, _stack, _pad, _rebind = (SliceTensorOp(), SliceUpdateOp(), ConcatenateOp(), StackOp(),
                                                         PadOp(), RebindOp())


def broadcast_to(x, shape) -> Tensor:
    x = ensure_tensor(x)
    shape = tuple(int(s) for s in shape)
    if tuple(x._impl.global_shape) == shape:
        return x
    return _broadcast_to(x, shape=shape)


def broadcast_to_physical(x, shape) -> Tensor:
    """Broadcast to the physical shape ``shape`` (the tensor's vmap dims, then its logical dims).
    Dims that ``shape`` has and ``x`` lacks are new LOGICAL dims, placed right behind the vmap dims,
    so the number of vmap dims never changes (reference: nabla/ops/view/shape.py:1127-1161)."""
    from .axes import unsqueeze_physical

    x = ensure_tensor(x)
    shape = tuple(int(s) for s in shape)
    if tuple(x._impl._shape) == shape:
        return x
    bd = x._impl.batch_dims
    for _ in range(len(shape) - len(x._impl._shape)):
        x = unsqueeze_physical(x, axis=bd)
    return _broadcast_to_p(x, shape=shape)


def reshape(x, shape) -> Tensor:
    x = ensure_tensor(x)
    shape = tuple(int(s) for s in shape)
    if tuple(x._impl.global_shape) == shape:
        return x
    return _reshape(x, shape=shape)


def flatten(x, start_dim: int = 0, end_dim: int = -1) -> Tensor:
    x = ensure_tensor(x)
    shp = list(x._impl.global_shape)
    rank = len(shp)
    if rank == 0:
        return reshape(x, (1,))
    s = start_dim + rank if start_dim < 0 else start_dim
    e = end_dim + rank if end_dim < 0 else end_dim
    return reshape(x, tuple(shp[:s]) + (math.prod(shp[s:e + 1]),) + tuple(shp[e + 1:]))


def slice_tensor(x, start, size) -> Tensor:
    x = ensure_tensor(x)
    start, size = tuple(int(s) for s in start), tuple(int(s) for s in size)
    if all(s == 0 for s in start) and size == tuple(x._impl.global_shape):
        return x
    return _slice(x, start=start, size=size)


def slice_update(x, update, start, size, *, use_buffer_ops: bool = False) -> Tensor:
    x = ensure_tensor(x)
    update = ensure_tensor(update, x)
    if update.dtype is not x.dtype:
        from ..unary import cast

        update = cast(update, x.dtype)
    return _slice_update(x, update, start=tuple(int(s) for s in start), size=tuple(int(s) for s in size),
                         use_buffer_ops=bool(use_buffer_ops))


def slice_update_inplace(x, update, start, size) -> Tensor:
    """`slice_update` as issued by ``x[...] = value``: same result, marked ``use_buffer_ops=True``."""
    return slice_update(x, update, start, size, use_buffer_ops=True)


def concatenate(tensors, axis: int = 0) -> Tensor:
    xs = [ensure_tensor(x) for x in tensors]
    if len(xs) == 1:
        return xs[0]
    if any(x._impl.batch_dims for x in xs):
        from ..base import _align_batch_dims

        xs = _align_batch_dims(xs)
    return _concat(xs, axis=int(axis))


def stack(tensors, axis: int = 0) -> Tensor:
    xs = [ensure_tensor(x) for x in tensors]
    if any(x._impl.batch_dims for x in xs):
        from ..base import _align_batch_dims

        xs = _align_batch_dims(xs)
    return _stack(xs, axis=int(axis))


def pad(x, paddings=None, mode: str = "constant", value: float = 0.0, **kwargs) -> Tensor:
    """Pad every logical dimension by ``(before, after)`` with ``value`` (``pad_width`` is accepted as
    an alias of ``paddings``; only ``mode="constant"`` exists, as in the reference,
    nabla/ops/view/shape.py:1472-1495)."""
    if paddings is None:
        paddings = kwargs.get("pad_width")
    if paddings is None:
        raise ValueError("pad() requires paddings or pad_width")
    if mode != "constant":
        raise NotImplementedError(f"pad mode {mode!r} is not supported (only 'constant')")
    x = ensure_tensor(x)
    paddings = tuple((int(a), int(b)) for a, b in paddings)
    if all(a == 0 and b == 0 for a, b in paddings):
        return x
    return _pad(x, paddings=paddings, value=value)


def rebind(x, shape=None, **kw) -> Tensor:
    return _rebind(ensure_tensor(x))
