"""SPMD glue between ops and the sharding model (reference: nabla/core/sharding/spmd.py:18-370,
nabla/ops/utils.py:446-508).

``prepare`` is called by ``Operation.__call__`` when any operand lives on a mesh. It decides,
from shapes only, (a) which pending partial sums must be reduced *before* the op because the
op is not linear in that operand, (b) how operands must be laid out so that every shard can
run the kernel locally, (c) the output layout including new pending sums from sharded
contractions, and (d) reductions that must happen right after the op (max/min reductions).
"""
from __future__ import annotations

from typing import Any, Callable

from ..common import pytree
from .propagation import infer_from_rule, required_input_specs
from .spec import DeviceMesh, DimSpec, ShardingSpec


def get_mesh_from_args(args) -> DeviceMesh | None:
    for t in pytree.tensor_leaves(args):
        if t._impl.sharding is not None:
            return t._impl.sharding.mesh
    return None


def replicated_spec(mesh: DeviceMesh, rank: int) -> ShardingSpec:
    return ShardingSpec(mesh, [DimSpec([]) for _ in range(rank)])


create_replicated_spec = replicated_spec


def _fit_rank(spec: ShardingSpec, rank: int) -> ShardingSpec:
    dims = [d.clone() for d in spec.dim_specs[:rank]]
    while len(dims) < rank:
        dims.append(DimSpec([]))
    return ShardingSpec(spec.mesh, dims, set(spec.replicated_axes), set(spec.partial_sum_axes))


def prepare(op, args: tuple, kwargs: dict, mesh: DeviceMesh):
    """Returns ``(new_args, out_specs_fn, reduce_axes)``; ``out_specs_fn(out_shapes)`` gives one
    ``ShardingSpec`` per output."""
    from ..tensor.api import Tensor

    custom = getattr(op, "plan_layouts", None)       # ops that lay their output out themselves (collectives)
    if custom is not None:
        return custom(args, mesh, kwargs)

    leaves, treedef = pytree.tree_flatten(args)
    t_idx = [i for i, a in enumerate(leaves) if isinstance(a, Tensor)]
    tensors = [leaves[i] for i in t_idx]
    if not tensors:
        return args, (lambda shapes: [replicated_spec(mesh, len(s)) for s in shapes]), set()
    shapes = [t._impl._shape for t in tensors]
    specs = [t._impl.sharding.clone() if t._impl.sharding is not None else replicated_spec(mesh, len(s))
             for t, s in zip(tensors, shapes)]

    # (a) partial sums the op cannot carry are reduced on the inputs
    incoming: set[str] = set()
    for s in specs:
        incoming |= s.partial_sum_axes
    keep = op.partial_passthrough_axes(specs, kwargs) & incoming if incoming else set()
    # a mesh axis cannot both split a dim of this op and carry a pending sum through it: the sum over
    # that axis is taken first (otherwise `(x @ w) @ v`, with the first product pending over "b" and
    # `v` split over "b", would label the result as split over "b" and lose the sum)
    splitting = {a for sp in specs for d in sp.dim_specs for a in d.axes}
    keep -= splitting
    must_reduce = incoming - keep

    # (b) operand layouts that agree on every factor
    try:
        rule = op.sharding_rule(list(shapes), None, **kwargs)
    except NotImplementedError:
        rule = None
    if rule is None:
        want = [ShardingSpec(mesh, [DimSpec([]) for _ in s], partial_sum_axes=set(sp.partial_sum_axes))
                for s, sp in zip(shapes, specs)]
    else:
        want = required_input_specs(rule, specs, mesh, [len(s) for s in shapes])
    if must_reduce:
        from ...ops.communication import all_reduce

        for j, t in enumerate(tensors):
            # a pending axis that this operand's own required layout puts on a dim is left to the
            # re-layout below, which turns "sum, then split" into one reduce-scatter
            over = (specs[j].partial_sum_axes & must_reduce) - want[j].used_axes()
            if over:
                tensors[j] = all_reduce(t, reduce_axes=over)
                specs[j] = tensors[j]._impl.sharding.clone()
        for sp in want:
            sp.partial_sum_axes -= must_reduce
    # a dim of global extent 0 or 1 is never split (the output spec below drops such axes too): an
    # operand that arrives with one (a (1, n) bias split along its first dim: one device holds the
    # row, the others nothing) is gathered, so that operands and output label agree
    for sp, shp in zip(want, shapes):
        for d, ds in enumerate(sp.dim_specs):
            if ds.axes and d < len(shp) and int(shp[d]) <= 1:
                ds.axes = []
    from ...ops.communication import reshard_to_spec

    for j, t in enumerate(tensors):
        cur = specs[j]
        if any(a.axes != b.axes for a, b in zip(cur.dim_specs, want[j].dim_specs)) or t._impl.sharding is None \
                or (cur.partial_sum_axes - want[j].partial_sum_axes):
            tensors[j] = reshard_to_spec(t, want[j])
            specs[j] = tensors[j]._impl.sharding.clone()

    for i, t in zip(t_idx, tensors):
        leaves[i] = t
    new_args = pytree.tree_unflatten(treedef, leaves)

    # (c) + (d) output layouts
    non_sum = op.collective_reduce_type != "sum"
    reduce_axes: set[str] = set()
    contraction: set[str] = set()
    if rule is not None:
        _, contraction = infer_from_rule(rule, specs, mesh)
        if non_sum:
            reduce_axes = set(contraction)

    def out_specs_fn(out_shapes) -> list[ShardingSpec]:
        res = []
        for i, shp in enumerate(out_shapes):
            if rule is None or i >= max(1, len(rule.output_mappings)):
                spec = replicated_spec(mesh, len(shp))
                spec.partial_sum_axes = set(keep)
            else:
                spec, contr = infer_from_rule(rule, specs, mesh, output_index=i)
                spec = _fit_rank(spec, len(shp))
                # never shard a dim of extent 1 or one the axes do not cover sensibly
                for d, ds in enumerate(spec.dim_specs):
                    if ds.axes and shp[d] <= 1:
                        ds.axes = []
                used = spec.used_axes()
                spec.partial_sum_axes = {a for a in (set(contr) | set(keep)) if a not in used}
            res.append(spec)
        return res

    return new_args, out_specs_fn, reduce_axes


def ensure_specs(args, mesh: DeviceMesh):
    """Give every unsharded tensor argument a replicated spec on ``mesh`` (by resharding)."""
    from ...ops.communication import reshard_to_spec

    def f(x):
        if pytree.is_tensor(x) and x._impl.sharding is None:
            return reshard_to_spec(x, replicated_spec(mesh, len(x._impl._shape)))
        return x

    return pytree.tree_map(f, args)


def infer_output_sharding(op, args, mesh, kwargs=None):
    """Reference-shaped entry point: ``(output_spec, input_specs, reduce_axes)`` for the
    first output, without performing any data movement."""
    if mesh is None:
        return None, [], set()
    tensors = pytree.tensor_leaves(args)
    shapes = [t._impl._shape for t in tensors]
    specs = [t._impl.sharding.clone() if t._impl.sharding is not None else replicated_spec(mesh, len(s))
             for t, s in zip(tensors, shapes)]
    rule = op.sharding_rule(list(shapes), None, **(kwargs or {}))
    incoming: set[str] = set()
    for s in specs:
        incoming |= s.partial_sum_axes
    keep = op.partial_passthrough_axes(specs, kwargs) & incoming
    keep -= {a for sp in specs for d in sp.dim_specs for a in d.axes}      # as in `prepare`
    out, contr = infer_from_rule(rule, specs, mesh)
    used = out.used_axes()
    out.partial_sum_axes = {a for a in (contr | keep) if a not in used}
    return out, specs, incoming - keep


# ---- shard-level helpers (reference: nabla/core/sharding/spmd.py:44-370). The ops of this package go
# through `prepare` and their own `execute`; these are the same steps offered one by one, for code
# that wants to run something of its own once per shard.
def reshard_inputs(args, required_specs, mesh: DeviceMesh | None):
    """Lay the tensor leaves of ``args`` out as ``required_specs`` asks (one spec per tensor leaf,
    ``None`` = leave alone); everything else passes through."""
    if mesh is None or not required_specs:
        return args
    from ...ops.communication.collectives import needs_reshard, reshard_to_spec
    from ..tensor.api import Tensor

    leaves, td = pytree.tree_flatten(args)
    specs = iter(required_specs)
    out = []
    for leaf in leaves:
        if isinstance(leaf, Tensor):
            want = next(specs, None)
            if want is not None and needs_reshard(leaf._impl.sharding, want):
                leaf = reshard_to_spec(leaf, want)
        out.append(leaf)
    return pytree.tree_unflatten(td, out)


def get_shard_args(args, shard_idx: int, per_input_shardings=None, g=None, Tensor=None, pytree=None):
    """``args`` with every tensor replaced by its buffer on local shard ``shard_idx`` (a tensor
    that is not on a mesh gives its single buffer to every shard)."""
    from ..common import pytree as _pt          # (`g`, `Tensor`, `pytree` are the reference's extra parameters: unused)
    from ..tensor.api import Tensor as _T

    def pick(x):
        if not isinstance(x, _T):
            return x
        x.realize()
        bufs = x._impl._buffers
        return bufs[shard_idx] if len(bufs) > 1 else bufs[0]

    leaves, td = _pt.tree_flatten(args)
    return _pt.tree_unflatten(td, [pick(x) for x in leaves])


def execute_on_shards(op_fn: Callable, args, kwargs: dict, mesh: DeviceMesh | None, input_shardings=None, op=None) -> list:
    """Run ``op_fn(*shard buffers, **kwargs)`` once per local shard of ``mesh`` (once when there is
    no mesh) and return the per-shard results."""
    n = mesh.num_local if mesh is not None else 1
    out = []
    for i in range(n):
        a = get_shard_args(args, i, input_shardings)
        out.append(op_fn(*a, **kwargs) if isinstance(a, (tuple, list)) else op_fn(a, **kwargs))
    return out


def create_sharded_output(results: list, sharding: ShardingSpec | None, is_traced: bool = False, batch_dims: int = 0,
                          mesh: DeviceMesh | None = None, physical_shapes=None, shard_dtypes=None, shard_devices=None):
    """A tensor made of the per-shard buffers ``results``; with a mesh but no spec they are taken
    as replicas."""
    from ..tensor.api import Tensor
    from ..tensor.impl import TensorImpl

    if sharding is None and mesh is not None:
        sharding = replicated_spec(mesh, results[0].dim())
    impl = TensorImpl(list(results) if sharding is not None else [results[0]], sharding=sharding, batch_dims=batch_dims,
                      is_traced=is_traced)
    return Tensor(impl=impl)
