"""Communication ops (reference: nabla/ops/communication/*.py, 3027 lines over 12 files).

Every op works in two execution modes decided by the mesh: *simulated* (this process holds
all shards; collectives are list computations, the reference's simulation branch) and
*distributed* (one process per GPU; ``nabla_b200.parallel.backend`` runs NCCL or the
peer-memory kernels). Reductions honour ``reduce_axes``: they run inside the sub-groups of
the mesh spanned by those axes, on real hardware too.

Global-view semantics: ``shard`` / ``all_gather`` / ``gather_all_axes`` / ``all_to_all`` /
``reshard`` change the layout of a tensor, not its value, so their VJP is "lay the cotangent
out like the input". ``all_reduce`` resolves pending partial sums; applied to values that are
not marked partial it sums the per-device values (psum), as the reference does.
"""
from __future__ import annotations

import math
from typing import Any, Iterable, Sequence

import torch

from ...core.common import pytree
from ...core.sharding.spec import (DeviceMesh, DimSpec, ShardingSpec, compute_local_shape, compute_local_slices,
                                   needs_reshard, shard_index)
from ...core.sharding.spmd import replicated_spec
from ...core.tensor.api import Tensor
from ...types import CPU, Accelerator, Device, as_device
from ..base import CollectiveOperation, Operation, ensure_tensor


def _spec_of(x: Tensor, mesh: DeviceMesh | None = None) -> ShardingSpec:
    if x._impl.sharding is not None:
        return x._impl.sharding
    return replicated_spec(mesh, len(x._impl._shape))


def _reduce_bufs(bufs: list[torch.Tensor], op: str) -> torch.Tensor:
    acc = bufs[0]
    if len(bufs) == 1:
        return acc
    if op == "sum":
        acc32 = acc.float() if acc.dtype in (torch.bfloat16, torch.float16) else acc.clone()
        for b in bufs[1:]:
            acc32 = acc32 + b
        return acc32.to(acc.dtype)
    for b in bufs[1:]:
        acc = {"max": torch.maximum, "min": torch.minimum, "prod": torch.mul}[op](acc, b)
    return acc


class _LayoutOp(CollectiveOperation):
    """Common plumbing: the op computes its own output spec; the kernel used for shape
    inference is the identity on the *global* shape unless overridden."""

    def kernel(self, x, **kwargs):
        return x

    def out_spec(self, x: Tensor, mesh: DeviceMesh, kwargs: dict) -> ShardingSpec:
        raise NotImplementedError

    def plan_layouts(self, args, mesh, kwargs):
        """Hook of `spmd.prepare`: ``(operands as they are, output specs, nothing to reduce first)``."""
        x = args[0]
        spec = self.out_spec(x, mesh, kwargs)
        return args, (lambda shapes: [spec for _ in shapes]), set()

    def infer_sharding_spec(self, args, mesh, kwargs=None):
        """``(output spec, the operands' specs, no pre-reduction)``: a collective decides its own output
        layout (reference: nabla/ops/communication/base.py:124-160)."""
        x = args[0]
        return self.out_spec(x, mesh, kwargs or {}), [t._impl.sharding for t in args if isinstance(t, Tensor)], set()

    def _mesh(self, node) -> DeviceMesh:
        m = node.kwargs.get("mesh")
        if m is not None:
            return m
        for im in node.input_impls():
            if im.sharding is not None:
                return im.sharding.mesh
        o = node.outputs()[0]
        return o.sharding.mesh

    @staticmethod
    def _shards(impl, mesh: DeviceMesh) -> list[torch.Tensor]:
        """Per-local-shard buffers, replicating an unsharded tensor's single buffer."""
        bufs = impl._buffers
        n = mesh.num_local
        return list(bufs) if len(bufs) == n else [bufs[0]] * n

    def _reshard_cot(self, cot: Tensor, x: Tensor) -> Tensor:
        sp = x._impl.sharding
        if sp is None:
            return cot.gather() if cot._impl.sharding is not None else cot
        want = sp.clone()
        want.partial_sum_axes = set()
        return reshard_to_spec(cot, want)


# ---------------------------------------------------------------- shard (slice to a layout)
class ShardOp(_LayoutOp):
    """Slice a tensor that is replicated along the dims being split (no communication)."""

    def out_spec(self, x, mesh, kwargs):
        return ShardingSpec(mesh, [DimSpec.from_raw(d).clone() for d in kwargs["dim_specs"]],
                            replicated_axes=set(kwargs.get("replicated_axes") or ()),
                            partial_sum_axes=set(kwargs.get("partial_sum_axes") or ()))

    def execute(self, node):
        mesh = self._mesh(node)
        x = node.input_impls()[0]
        out = node.outputs()[0]
        spec = out.sharding
        src = x.sharding
        bufs = self._shards(x, mesh)
        res = []
        for s, dev in enumerate(mesh.local_ids):
            b = bufs[s]
            idx = []
            for d, ds in enumerate(spec.dim_specs):
                already = src is not None and src.dim_specs[d].axes == ds.axes
                if not ds.axes or already:
                    idx.append(slice(None))
                else:
                    if src is not None and src.dim_specs[d].axes:
                        raise RuntimeError("shard: input dim must be replicated before it is re-split")
                    i, tot = shard_index(spec, d, dev)
                    from ...core.sharding.spec import local_slice

                    st, ln = local_slice(out._shape[d], i, tot)
                    idx.append(slice(st, st + ln))
            piece = b[tuple(idx)]
            res.append(piece if piece.is_contiguous() else piece.contiguous())
        return [res]

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (self._reshard_cot(cot, primals[0]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _shard_op(tangents[0], **kwargs)


# ---------------------------------------------------------------- all_gather
class AllGatherOp(_LayoutOp):
    """Make physical dim ``dim`` whole on every device of its sharding group."""

    @classmethod
    def estimate_cost(cls, size_bytes: int, mesh, axes, input_specs=None, output_specs=None) -> float:
        return CollectiveOperation._ring_cost(size_bytes, mesh, axes, factor=1.0)

    def out_spec(self, x, mesh, kwargs):
        sp = _spec_of(x, mesh).clone()
        sp.dim_specs[kwargs["dim"]] = DimSpec([])
        return sp

    def execute(self, node):
        mesh = self._mesh(node)
        x = node.input_impls()[0]
        dim = node.kwargs["dim"]
        axes = list(x.sharding.dim_specs[dim].axes) if x.sharding is not None else []
        bufs = self._shards(x, mesh)
        if not axes:
            return [bufs]
        if mesh.is_distributed:
            from ...parallel import backend

            g = mesh.group_of(mesh.rank, axes)
            sizes = [compute_local_shape(x._shape, x.sharding, d)[dim] for d in g]
            return [[backend.all_gather(bufs[0], mesh, axes, dim, sizes)]]
        out: list[Any] = [None] * mesh.size
        for g in mesh.groups(axes):
            full = torch.cat([bufs[i] for i in g], dim=dim)
            for i in g:
                out[i] = full
        return [out]

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (self._reshard_cot(cot, primals[0]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _all_gather_op(tangents[0], **kwargs)


class GatherAllAxesOp(_LayoutOp):
    """Replicate fully: every sharded dim is gathered."""

    def out_spec(self, x, mesh, kwargs):
        sp = _spec_of(x, mesh)
        return ShardingSpec(mesh, [DimSpec([]) for _ in sp.dim_specs], partial_sum_axes=set(sp.partial_sum_axes))

    def execute(self, node):
        mesh = self._mesh(node)
        x = node.input_impls()[0]
        bufs = self._shards(x, mesh)
        spec = x.sharding
        for dim, ds in enumerate(spec.dim_specs):
            if not ds.axes:
                continue
            axes = list(ds.axes)
            if mesh.is_distributed:
                from ...parallel import backend

                g = mesh.group_of(mesh.rank, axes)
                sizes = [compute_local_shape(x._shape, spec, d)[dim] for d in g]
                bufs = [backend.all_gather(bufs[0], mesh, axes, dim, sizes)]
            else:
                new: list[Any] = [None] * mesh.size
                for g in mesh.groups(axes):
                    full = torch.cat([bufs[i] for i in g], dim=dim)
                    for i in g:
                        new[i] = full
                bufs = new
        return [bufs]

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (self._reshard_cot(cot, primals[0]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return gather_all_axes(tangents[0])


# ---------------------------------------------------------------- all_reduce
class AllReduceOp(_LayoutOp):
    @classmethod
    def estimate_cost(cls, size_bytes: int, mesh, axes, input_specs=None, output_specs=None) -> float:
        return CollectiveOperation._ring_cost(size_bytes, mesh, axes, factor=2.0)

    def _plan(self, x: Tensor, mesh, kwargs):
        sp = _spec_of(x, mesh)
        axes = set(kwargs["reduce_axes"])
        dims = []
        shape = list(x._impl._shape)
        for d, ds in enumerate(sp.dim_specs):
            keep = [a for a in ds.axes if a not in axes]
            gone = [a for a in ds.axes if a in axes]
            if gone:
                # psum over a dim-sharding axis: the shards are summed elementwise, the result
                # has the local extent along that dim
                div = math.prod(mesh.get_axis_size(a) for a in gone)
                shape[d] = math.ceil(shape[d] / div)
            dims.append(DimSpec(keep))
        out = ShardingSpec(mesh, dims, replicated_axes=set(sp.replicated_axes),
                           partial_sum_axes=set(sp.partial_sum_axes) - axes)
        return out, tuple(shape)

    def out_spec(self, x, mesh, kwargs):
        return self._plan(x, mesh, kwargs)[0]

    def __call__(self, x, **kwargs):
        mesh = kwargs.get("mesh") or x._impl.sharding.mesh
        self._shape = self._plan(x, mesh, kwargs)[1]
        return super().__call__(x, **kwargs)

    def kernel(self, x, **kwargs):
        shp = getattr(self, "_shape", None)
        if shp is not None and tuple(x.shape) != tuple(shp) and x.device.type == "meta":
            return torch.empty(shp, dtype=x.dtype, device="meta")
        return x

    def infer_outputs(self, tensors_meta, arg_leaves, treedef, kwargs):
        (shp, dt) = tensors_meta[0]
        return [(tuple(self._shape), dt)], pytree.tree_structure(0)

    def execute(self, node):
        mesh = self._mesh(node)
        x = node.input_impls()[0]
        axes = [a for a in mesh.axis_names if a in node.kwargs["reduce_axes"]] + \
               [a for a in node.kwargs["reduce_axes"] if a not in mesh.axis_names]
        op = node.kwargs.get("reduce_op", "sum")
        bufs = self._shards(x, mesh)
        if mesh.is_distributed:
            from ...parallel import backend

            return [[backend.all_reduce(bufs[0], mesh, axes, op)]]
        out: list[Any] = [None] * mesh.size
        for g in mesh.groups(axes):
            r = _reduce_bufs([bufs[i] for i in g], op)
            for i in g:
                out[i] = r
        return [out]

    def vjp_rule(self, primals, cot, outputs, kwargs):
        x = primals[0]
        sp = x._impl.sharding
        if sp is not None and any(set(d.axes) & set(kwargs["reduce_axes"]) for d in sp.dim_specs):
            # psum over dim-sharding axes: every device's addend receives the same cotangent
            return (_psum_transpose(cot, x, kwargs),)
        return (self._reshard_cot(cot, x),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        t = tangents[0]
        if t._impl.sharding is None:
            return t
        sp = t._impl.sharding
        ax = set(kwargs["reduce_axes"])
        if kwargs.get("reduce_op", "sum") != "sum":
            # the max / min combination that finishes a reduction over a sharded axis. The rule of
            # that reduction already masks with the extreme over ALL shards, so each device holds
            # its addend of the tangent: they are summed, whatever the primal's combination was
            # (the counterpart of the identity this op's VJP applies to the cotangent)
            if any(set(d.axes) & ax for d in sp.dim_specs):
                return _all_reduce_op(t, reduce_axes=kwargs["reduce_axes"], reduce_op="sum")
            spec = sp.clone()
            spec.partial_sum_axes = set(spec.partial_sum_axes) | ax
            return _all_reduce_op(relabel_spec(t, spec), reduce_axes=kwargs["reduce_axes"], reduce_op="sum")
        if not (sp.partial_sum_axes & ax) and not any(set(d.axes) & ax for d in sp.dim_specs):
            return t
        return _all_reduce_op(t, **kwargs)


def _psum_transpose(cot: Tensor, x: Tensor, kwargs) -> Tensor:
    # cotangent is replicated over the reduced axes with the local shape; tiling it along the
    # formerly sharded dims gives every addend its copy
    sp = x._impl.sharding
    ax = set(kwargs["reduce_axes"])
    out = cot
    from ..view import concatenate

    for d, ds in enumerate(sp.dim_specs):
        gone = [a for a in ds.axes if a in ax]
        if gone:
            k = math.prod(sp.mesh.get_axis_size(a) for a in gone)
            out = concatenate([out] * k, axis=d - x._impl.batch_dims)
    want = sp.clone()
    want.partial_sum_axes = set()
    return reshard_to_spec(out, want)


# ---------------------------------------------------------------- reduce_scatter
class ReduceScatterOp(_LayoutOp):
    @classmethod
    def estimate_cost(cls, size_bytes: int, mesh, axes, input_specs=None, output_specs=None) -> float:
        return CollectiveOperation._ring_cost(size_bytes, mesh, axes, factor=1.0)

    def out_spec(self, x, mesh, kwargs):
        sp = _spec_of(x, mesh).clone()
        dim = kwargs["dim"]
        sc = [a for a in kwargs["scatter_axes"]]
        sp.dim_specs[dim] = DimSpec(list(sp.dim_specs[dim].axes) + [a for a in sc if a not in sp.dim_specs[dim].axes])
        sp.partial_sum_axes = set(sp.partial_sum_axes) - set(sc)
        return sp

    def execute(self, node):
        mesh = self._mesh(node)
        x = node.input_impls()[0]
        out = node.outputs()[0]
        dim = node.kwargs["dim"]
        axes = list(node.kwargs["scatter_axes"])
        bufs = self._shards(x, mesh)
        if mesh.is_distributed:
            from ...parallel import backend

            r = backend.reduce_scatter(bufs[0], mesh, axes, dim) if not (x.sharding and x.sharding.dim_specs[dim].axes) else None
            if r is None:
                full = backend.all_reduce(bufs[0], mesh, axes, "sum")
                r = self._slice(full, mesh, axes, dim, mesh.rank)
            return [[r]]
        res: list[Any] = [None] * mesh.size
        for g in mesh.groups(axes):
            s = _reduce_bufs([bufs[i] for i in g], "sum")
            for i in g:
                res[i] = self._slice(s, mesh, axes, dim, i)
        return [res]

    @staticmethod
    def _slice(full, mesh, axes, dim, dev):
        from ...core.sharding.spec import local_slice

        idx, tot = 0, 1
        for a in axes:
            n = mesh.get_axis_size(a)
            idx = idx * n + mesh.get_coordinate(dev, a)
            tot *= n
        st, ln = local_slice(full.shape[dim], idx, tot)
        return full.narrow(dim, st, ln).contiguous()

    def vjp_rule(self, primals, cot, outputs, kwargs):
        # every addend of the scattered sum receives the cotangent of its slice: the cotangent laid
        # out like the operand, without the pending sum (a cotangent that is not on a mesh, e.g. a
        # basis vector of jacrev, is placed on the operand's)
        x = primals[0]
        mesh = (cot._impl.sharding or x._impl.sharding).mesh
        want = _spec_of(x, mesh).clone()
        want.partial_sum_axes = set()
        return (reshard_to_spec(cot, want),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _reduce_scatter_op(tangents[0], **kwargs)


# ---------------------------------------------------------------- ppermute
class PPermuteOp(_LayoutOp):
    """Move whole shards between devices: ``perm = [(src, dst), ...]``; devices nobody sends
    to receive zeros."""

    def out_spec(self, x, mesh, kwargs):
        return _spec_of(x, mesh).clone()

    def execute(self, node):
        mesh = self._mesh(node)
        x = node.input_impls()[0]
        perm = node.kwargs["permutation"]
        bufs = self._shards(x, mesh)
        if mesh.is_distributed:
            from ...parallel import backend

            return [[backend.permute(bufs[0], mesh, perm)]]
        out: list[Any] = [None] * mesh.size
        for s, d in perm:
            out[d] = bufs[s]
        for i in range(mesh.size):
            if out[i] is None:
                out[i] = torch.zeros_like(bufs[i])
        return [out]

    def vjp_rule(self, primals, cot, outputs, kwargs):
        inv = tuple((d, s) for s, d in kwargs["permutation"])
        return (ppermute(cot, inv),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return ppermute(tangents[0], kwargs["permutation"])


# ---------------------------------------------------------------- device transfer
class TransferOp(Operation):
    def kernel(self, x, *, device: Device):
        if x.device.type == "meta":
            return x
        return x.to(device.to_torch())

    def output_device(self, tensors, kwargs):
        return kwargs["device"]

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (_transfer_op(cot, device=primals[0].device),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _transfer_op(tangents[0], device=kwargs["device"])


class RelabelOp(_LayoutOp):
    """Reinterpret the per-device buffers under another spec of the same local shapes (no data
    movement). Used to turn "pending partial sum" labels into plain per-device values before a
    max/min combination, and back."""

    def out_spec(self, x, mesh, kwargs):
        return kwargs["spec"].clone()

    def execute(self, node):
        mesh = self._mesh(node)
        return [self._shards(node.input_impls()[0], mesh)]

    def vjp_rule(self, primals, cot, outputs, kwargs):
        x = primals[0]
        sp = x._impl.sharding.clone()
        sp.partial_sum_axes = set()
        return (reshard_to_spec(cot, sp) if needs_reshard(cot._impl.sharding, sp) else cot,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _relabel_op(tangents[0], **kwargs)


class FanOutOp(_LayoutOp):
    """Identity on the buffers whose cotangent is summed over the ``copies`` devices that received
    the value: the derivative of handing one rank's value to every device of a mesh, each copy
    counted separately (reference: nabla/ops/communication/broadcast.py:89-96, "AllReduce(sum) back
    to root")."""

    def out_spec(self, x, mesh, kwargs):
        return x._impl.sharding.clone()

    def execute(self, node):
        mesh = self._mesh(node)
        return [self._shards(node.input_impls()[0], mesh)]

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (cot * float(kwargs["copies"]),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _fan_out_op(tangents[0], **kwargs)


_relabel_op = RelabelOp()
_fan_out_op = FanOutOp()


def relabel_spec(x, spec: ShardingSpec):
    return _relabel_op(x, spec=spec)


_shard_op, _all_gather_op, _gather_all_op = ShardOp(), AllGatherOp(), GatherAllAxesOp()
_all_reduce_op, _reduce_scatter_op, _ppermute_op, _transfer_op = (AllReduceOp(), ReduceScatterOp(), PPermuteOp(),
                                                                  TransferOp())


# ================================================================ functional API
def _full_dim_specs(x: Tensor, dim_specs) -> list[DimSpec]:
    """Accept a logical-rank spec on a vmapped tensor: batch specs are prepended."""
    specs = [DimSpec.from_raw(d).clone() for d in dim_specs]
    bd = x._impl.batch_dims
    if bd > 0 and len(specs) == len(x._impl.global_shape):
        cur = x._impl.sharding
        pre = [cur.dim_specs[i].clone() if cur is not None and i < len(cur.dim_specs) else DimSpec([])
               for i in range(bd)]
        specs = pre + specs
    if len(specs) != len(x._impl._shape):
        raise ValueError(f"sharding spec of rank {len(specs)} for a tensor of rank {len(x._impl._shape)}")
    return specs


def reshard_to_spec(x: Tensor, target: ShardingSpec) -> Tensor:
    """Bring ``x`` to layout ``target``: gather dims that lose axes, resolve partial sums the
    target does not keep (only those), then slice dims that gain axes."""
    mesh = target.mesh
    cur = x._impl.sharding
    if cur is None:
        return _shard_op(x, mesh=mesh, dim_specs=tuple(target.dim_specs), replicated_axes=frozenset(target.replicated_axes),
                         partial_sum_axes=frozenset(target.partial_sum_axes))
    if not needs_reshard(cur, target):
        return x
    r = x
    for d in range(len(cur.dim_specs)):
        if cur.dim_specs[d].axes and cur.dim_specs[d].axes != target.dim_specs[d].axes:
            r = _all_gather_op(r, dim=d)
    drop = set(r._impl.sharding.partial_sum_axes) - set(target.partial_sum_axes)
    if drop:
        # a pending sum over axes that the target uses to split a dim: reduce-scatter (half the
        # traffic of all-reduce + slice); the scattered axes must extend the dim's axis list
        now = r._impl.sharding
        for d in range(len(now.dim_specs)):
            have, want = list(now.dim_specs[d].axes), list(target.dim_specs[d].axes)
            extra = want[len(have):]
            if extra and want[:len(have)] == have and set(extra) <= drop and \
                    r._impl._shape[d] % math.prod(mesh.get_axis_size(a) for a in want) == 0:
                r = _reduce_scatter_op(r, dim=d, scatter_axes=tuple(extra))
                drop -= set(extra)
                now = r._impl.sharding
    if drop:
        r = _all_reduce_op(r, reduce_axes=frozenset(drop), reduce_op="sum")
    now = r._impl.sharding
    if any(a.axes != b.axes for a, b in zip(now.dim_specs, target.dim_specs)):
        r = _shard_op(r, mesh=mesh, dim_specs=tuple(target.dim_specs),
                      replicated_axes=frozenset(target.replicated_axes),
                      partial_sum_axes=frozenset(r._impl.sharding.partial_sum_axes))
    return r


def shard(x, mesh: DeviceMesh, dim_specs, replicated_axes=None, partial_sum_axes=None, **kwargs):
    """Distribute ``x`` (a Tensor or a pytree of Tensors) over ``mesh``: one entry of
    ``dim_specs`` (``None`` | axis name | tuple of names | ``DimSpec``; a ``P(...)`` works)
    per dimension."""
    if not isinstance(x, Tensor):
        if isinstance(x, (list, tuple, dict)):
            return pytree.tree_map(lambda t: shard(t, mesh, dim_specs, replicated_axes, partial_sum_axes)
                                   if isinstance(t, Tensor) else t, x)
        x = ensure_tensor(x)
    specs = _full_dim_specs(x, dim_specs)
    target = ShardingSpec(mesh, specs, replicated_axes=set(replicated_axes or ()),
                          partial_sum_axes=set(partial_sum_axes or ()))
    if x._impl.sharding is not None and x._impl.sharding.mesh != mesh:
        x = x.gather()
        x = Tensor(buffers=[x.realize()._impl._buffers[0]]) if not mesh.is_distributed else x
    return reshard_to_spec(x, target)


def reshard(x, mesh: DeviceMesh, dim_specs, replicated_axes=None, **kwargs):
    return shard(x, mesh, dim_specs, replicated_axes=replicated_axes, **kwargs)


def reshard_tensor(tensor, from_spec, to_spec, mesh=None):
    return reshard_to_spec(tensor, to_spec)


def broadcast(x, mesh: DeviceMesh | None = None, root: int = 0):
    x = ensure_tensor(x)
    if mesh is None:
        if x._impl.sharding is None:
            return x                       # one device, no mesh: nothing to replicate onto
        mesh = x._impl.sharding.mesh
    return reshard_to_spec(x, replicated_spec(mesh, len(x._impl._shape)))


def distributed_broadcast(x, mesh: DeviceMesh | None = None):
    """Hand the root's value to every device of the mesh. Unlike `broadcast` (a change of layout in
    the global view, gradient 1), every device's copy counts in the backward pass: the gradient is
    the sum over the ``len(mesh.devices)`` copies, as in the reference
    (nabla/ops/communication/broadcast.py:89-96; tests/unit/test_communication_rigorous.py:104-123)."""
    y = broadcast(x, mesh)
    return _fan_out_op(y, copies=len(y._impl.sharding.mesh.devices))


def all_gather(x, axis: int | None = None, **kwargs):
    """Gather logical ``axis`` (or every sharded dim when ``None``); ``physical_axis=`` indexes
    the physical shape instead."""
    x = ensure_tensor(x)
    if x._impl.sharding is None:
        return x
    if "physical_axis" in kwargs and kwargs["physical_axis"] is not None:
        dim = int(kwargs["physical_axis"])
    elif axis is None:
        return gather_all_axes(x)
    else:
        rank = len(x._impl.global_shape)
        dim = (axis + rank if axis < 0 else axis) + x._impl.batch_dims
    if not x._impl.sharding.dim_specs[dim].axes:
        return x
    return _all_gather_op(x, dim=dim)


def gather_all_axes(sharded_tensor):
    x = ensure_tensor(sharded_tensor)
    if x._impl.sharding is None:
        return x
    return _gather_all_op(x)


def all_reduce(x, mesh: DeviceMesh | None = None, reduce_axes=None, reduce_op: str = "sum", **kwargs):
    """Reduce across the sub-groups of the mesh spanned by ``reduce_axes`` (default: the
    tensor's pending partial axes, else every mesh axis)."""
    x = ensure_tensor(x)
    if x._impl.sharding is None:
        if mesh is None:
            return x
        x = reshard_to_spec(x, replicated_spec(mesh, len(x._impl._shape)))
    sp = x._impl.sharding
    if reduce_axes is None:
        reduce_axes = set(sp.partial_sum_axes) or set(sp.mesh.axis_names)
    elif isinstance(reduce_axes, str):
        reduce_axes = {reduce_axes}
    reduce_axes = frozenset(reduce_axes)
    if not reduce_axes:
        return x
    return _all_reduce_op(x, reduce_axes=reduce_axes, reduce_op=reduce_op)


def pmean(sharded_tensor, axis_name: str | None = None):
    x = ensure_tensor(sharded_tensor)
    sp = x._impl.sharding
    if sp is None:
        return x
    axes = {axis_name} if axis_name else set(sp.mesh.axis_names)
    n = math.prod(sp.mesh.get_axis_size(a) for a in axes)
    return all_reduce(x, reduce_axes=axes) * (1.0 / n)


def reduce_scatter(x, axis: int, scatter_axes=None, **kwargs):
    """Sum over ``scatter_axes`` and leave logical ``axis`` split over them."""
    x = ensure_tensor(x)
    sp = x._impl.sharding
    if sp is None:
        mesh = kwargs.get("mesh")
        if mesh is None:
            return x
        x = reshard_to_spec(x, replicated_spec(mesh, len(x._impl._shape)))
        sp = x._impl.sharding
    rank = len(x._impl.global_shape)
    dim = (axis + rank if axis < 0 else axis) + x._impl.batch_dims
    if scatter_axes is None:
        scatter_axes = set(sp.partial_sum_axes) or set(sp.dim_specs[dim].axes) or set(sp.mesh.axis_names)
    elif isinstance(scatter_axes, str):
        scatter_axes = {scatter_axes}
    ordered = tuple(sp.ordered_axes(set(scatter_axes)))
    if set(sp.dim_specs[dim].axes) & set(ordered):
        # the dim is already split over these axes: psum the shards, then split again
        r = all_reduce(x, reduce_axes=set(ordered))
        tgt = r._impl.sharding.clone()
        tgt.dim_specs[dim] = DimSpec(list(tgt.dim_specs[dim].axes) + list(ordered))
        return reshard_to_spec(r, tgt)
    return _reduce_scatter_op(x, dim=dim, scatter_axes=ordered)


def all_to_all(sharded_tensor, split_axis: int, concat_axis: int, tiled: bool = True):
    """Move the mesh axes that split ``concat_axis`` onto ``split_axis`` (Ulysses-style swap).
    Value-preserving in the global view; its VJP is the swap in the other direction."""
    x = ensure_tensor(sharded_tensor)
    sp = x._impl.sharding
    if sp is None:
        return x
    rank = len(x._impl.global_shape)
    bd = x._impl.batch_dims
    s = (split_axis + rank if split_axis < 0 else split_axis) + bd
    c = (concat_axis + rank if concat_axis < 0 else concat_axis) + bd
    tgt = sp.clone()
    moved = list(tgt.dim_specs[c].axes) or list(sp.mesh.axis_names[:1])
    n = 1
    for a in moved:
        n *= sp.mesh.get_axis_size(a)
    if int(x._impl._shape[s]) % n:
        raise ValueError(f"all_to_all: split axis {split_axis} of size {int(x._impl._shape[s])} is not divisible "
                         f"by the {n} devices it is split over")
    tgt.dim_specs[c] = DimSpec([])
    tgt.dim_specs[s] = DimSpec(list(tgt.dim_specs[s].axes) + [a for a in moved if a not in tgt.dim_specs[s].axes])
    return reshard_to_spec(x, tgt)


def ppermute(sharded_tensor, permutation=None, perm=None):
    x = ensure_tensor(sharded_tensor)
    p = permutation if permutation is not None else perm
    if p is None:
        raise TypeError("ppermute needs a permutation [(src, dst), ...]")
    if x._impl.sharding is None:
        raise ValueError("ppermute needs a tensor on a mesh")
    p = tuple((int(a), int(b)) for a, b in p)
    dsts = [b for _, b in p]
    if len(set(dsts)) != len(dsts):
        raise ValueError("ppermute: a destination appears twice")
    return _ppermute_op(x, permutation=p)


def axis_index(mesh: DeviceMesh, axis_name: str):
    """A length-``axis_size`` int32 vector split over ``axis_name``: each device holds its own
    coordinate along that axis."""
    from ..creation import arange
    from ...types import DType

    n = mesh.get_axis_size(axis_name)
    return shard(arange(0, n, 1, dtype=DType.int32, device=mesh.device_refs[0]), mesh, [axis_name])


def to_device(x, device=None, *, sharding: ShardingSpec | None = None):
    x = ensure_tensor(x)
    if sharding is not None:
        return reshard_to_spec(x, sharding)
    device = as_device(device)
    if x._impl.sharding is not None:
        x = x.gather()
        x.realize()
        x = Tensor(buffers=[x._impl._buffers[0]])
    if x.device == device:
        return x
    return _transfer_op(x, device=device)


transfer_to = to_device


def cpu(x):
    return to_device(x, CPU())


def gpu(x, device_id: int = 0):
    return to_device(x, Accelerator(device_id))


accelerator = gpu
