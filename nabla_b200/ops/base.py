"""Operation base classes and the op-call pipeline (reference: nabla/ops/base.py:91-1205,
nabla/ops/utils.py:410-762).

Calling an op never computes data. ``Operation.__call__`` :

1. flattens the arguments and collects metadata (vmap batch dims, tracing, mesh);
2. translates logical kwargs to physical ones (``adapt_kwargs``: axes shift past batch dims);
3. on a mesh: infers the output sharding from the op's factor rule, all-reduces partial
   inputs the op cannot carry, reshards operands that disagree;
4. infers output shapes/dtypes by running the op's torch kernel on ``meta`` tensors (cached);
5. creates promise tensors linked to a new ``OpNode``;
6. in eager mode evaluates immediately;
7. applies output-side reductions the sharding inference asked for.

Execution happens later in ``execute``: the kernel runs once per locally held shard.
"""
from __future__ import annotations

import weakref
from typing import Any, Sequence

import torch

from .. import config
from ..core.common import pytree
from ..core.graph.tracing import OpNode
from ..core.tensor.api import Tensor
from ..core.tensor.impl import TensorImpl
from ..types import Device, DType

_META_CACHE: dict[Any, Any] = {}


def _tracing_suppressed() -> bool:
    from ..core.autograd.backward import tracing_suppressed

    return tracing_suppressed()


def _freeze(v: Any) -> Any:
    from ..core.graph.engine import _freeze as f

    return f(v)


def ensure_tensor(x: Any, like: Tensor | None = None) -> Tensor:
    """Promote python scalars / numpy / torch values to a Tensor (dtype and device of ``like``)."""
    if isinstance(x, Tensor):
        return x
    from .creation import constant

    if like is not None:
        dtype = like.dtype
        if isinstance(x, float) and not dtype.is_float():
            dtype = DType.float32
        if isinstance(x, bool):
            dtype = DType.bool if like.dtype is DType.bool else like.dtype
        elif isinstance(x, int) and like.dtype is DType.bool:
            dtype = DType.int32            # True + 2 is 3, not True (numpy's promotion of bool with an integer)
        return constant(x, dtype=dtype, device=like.device)
    return constant(x)


class Operation:
    """Base class of all ops. Subclasses implement ``kernel`` plus optional rules."""

    #: which pending partial sums may flow through: 'none' (reduce first), 'all' (only if
    #: every tensor input carries the axis), 'one' (at most one input), 'first' (input 0 only)
    partial_policy = "none"
    collective_reduce_type = "sum"
    _name: str | None = None

    # ------------------------------------------------------------------ identity
    @property
    def name(self) -> str:
        if self._name is not None:
            return self._name
        n = type(self).__name__
        if n.endswith("Op"):
            n = n[:-2]
        out = []
        for i, ch in enumerate(n):
            if ch.isupper() and i and (not n[i - 1].isupper()):
                out.append("_")
            out.append(ch.lower())
        return "".join(out)

    def __repr__(self) -> str:
        return f"<op {self.name}>"

    # ------------------------------------------------------------------ to override
    def kernel(self, *args, **kwargs):
        raise NotImplementedError(f"{self.name}.kernel")

    def adapt_kwargs(self, args: tuple, kwargs: dict, batch_dims: int) -> dict:
        return kwargs

    def output_batch_dims(self, batch_dims: int, kwargs: dict) -> int:
        return batch_dims

    def sharding_rule(self, input_shapes, output_shapes, **kwargs):
        """Factor rule; default = right-aligned elementwise broadcasting."""
        from ..core.sharding.propagation import elementwise_rule

        rank = len(output_shapes[0]) if output_shapes else max((len(s) for s in input_shapes), default=0)
        return elementwise_rule(input_shapes, rank)

    def shard_kwargs(self, kwargs: dict, node: OpNode, shard_idx: int, device_id: int) -> dict:
        """kwargs for one shard (ops carrying global shapes/offsets localise them here)."""
        return kwargs

    def vjp_rule(self, primals, cotangents, outputs, kwargs):
        raise NotImplementedError(f"'{self.name}' has no vjp_rule")

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        raise NotImplementedError(f"'{self.name}' has no jvp_rule")

    def compute_cost(self, input_shapes, output_shapes) -> float:
        """FLOP estimate used by the auto-sharding cost model."""
        n = 1
        for s in output_shapes[:1]:
            for d in s:
                n *= int(d)
        return float(n)

    def memory_cost(self, input_shapes, output_shapes, dtype_bytes: int = 4) -> int:
        """Bytes of the op's outputs (reference: nabla/ops/base.py:226-239)."""
        tot = 0
        for s in output_shapes:
            n = 1
            for d in s:
                n *= int(d)
            tot += n * int(dtype_bytes)
        return tot

    def infer_output_rank(self, input_shapes, **kwargs) -> int:
        return len(input_shapes[0]) if input_shapes else 0

    # ------------------------------------------------------------------ partial-sum policy
    multiple_results: bool = False       # the reference's flag for ops with several outputs (ops/base.py:121)

    @property
    def allows_partial_passthrough(self) -> bool:
        """Whether this op may ever defer the all-reduce of a pending partial sum
        (reference: nabla/ops/base.py:140-146); `partial_passthrough_axes` decides per call."""
        return self.partial_policy != "none"

    def get_sharding_rule_template(self):
        """Ops here give their rule through `sharding_rule` (instantiated per call); there is no
        shape-independent template object (reference: nabla/ops/base.py:472-473 returns None too)."""
        return None

    def compute_physical_shape(self, args, kwargs, output_sharding=None):
        """Per-shard output shapes, dtypes and devices of a call, without running it
        (reference: nabla/ops/base.py:397-410). Shapes come from the op's own shape inference on
        meta tensors; with an output sharding every shard's extent follows the ceil-div rule."""
        from ..core.sharding.spec import compute_local_shape
        from ..core.tensor.api import Tensor

        probe = self(*args, **(kwargs or {}))
        outs = [t for t in pytree.tree_leaves(probe) if isinstance(t, Tensor)]
        shapes, dtypes, devices = [], [], []
        for t in outs:
            sp = output_sharding if output_sharding is not None else t.sharding
            g = tuple(int(d) for d in t._impl.physical_global_shape)
            if sp is None:
                shapes.append(g)
            else:
                shapes.append([compute_local_shape(g, sp, d) for d in range(len(sp.mesh.devices))])
            dtypes.append(t.dtype)
            devices.append(t.device)
        return shapes, dtypes, devices

    def partial_passthrough_axes(self, input_specs: Sequence, kwargs: dict | None = None) -> set[str]:
        specs = [s for s in input_specs if s is not None]
        if not specs or self.partial_policy == "none":
            return set()
        axes: set[str] = set()
        for s in specs:
            axes |= s.partial_sum_axes
        ok: set[str] = set()
        for a in axes:
            carriers = [i for i, s in enumerate(input_specs) if s is not None and a in s.partial_sum_axes]
            n_inputs = len(input_specs)
            if self.partial_policy == "all" and len(carriers) == n_inputs:
                ok.add(a)
            elif self.partial_policy == "one" and len(carriers) == 1:
                ok.add(a)
            elif self.partial_policy == "first" and carriers == [0]:
                ok.add(a)
            elif self.partial_policy == "any":
                ok.add(a)
        return ok

    # ------------------------------------------------------------------ shape inference
    def infer_outputs(self, tensors_meta: list[tuple[tuple[int, ...], torch.dtype]], arg_leaves: list, treedef,
                      kwargs: dict):
        """Run the kernel on meta tensors; returns (list of (shape, torch dtype), out treedef)."""
        key = (type(self), self.name, tuple(tensors_meta),
               tuple(_freeze(a) if not isinstance(a, Tensor) else "T" for a in arg_leaves), _freeze(kwargs))
        hit = _META_CACHE.get(key)
        if hit is not None:
            return hit
        it = iter(tensors_meta)
        leaves = []
        for a in arg_leaves:
            if isinstance(a, Tensor):
                shp, dt = next(it)
                leaves.append(torch.empty(shp, dtype=dt, device="meta"))
            else:
                leaves.append(a)
        args = pytree.tree_unflatten(treedef, leaves)
        out = self.kernel(*args, **self.meta_kwargs(kwargs))
        out_leaves, out_td = pytree.tree_flatten(out)
        res = ([(tuple(o.shape), o.dtype) for o in out_leaves], out_td)
        if len(_META_CACHE) > 20000:
            _META_CACHE.clear()
        _META_CACHE[key] = res
        return res

    def meta_kwargs(self, kwargs: dict) -> dict:
        return kwargs

    def infer_output_shape(self, input_shapes, **kwargs):
        """Output shape(s) for operands of the given PHYSICAL shapes, found by running the kernel
        on storage-less tensors: a tuple for one output, a list of tuples for several. ``dtype=``
        picks the operands' dtype (float32 by default)."""
        dt = kwargs.pop("dtype", torch.float32)
        metas = [torch.empty(tuple(int(d) for d in s), dtype=dt, device="meta") for s in input_shapes]
        out = self.kernel(*metas, **self.meta_kwargs(kwargs))
        leaves = [o for o in pytree.tree_leaves(out) if isinstance(o, torch.Tensor)]
        shapes = [tuple(int(d) for d in o.shape) for o in leaves]
        return shapes[0] if len(shapes) == 1 else shapes

    def infer_sharding_spec(self, args, mesh, kwargs=None):
        """``(output spec, input specs as the op wants them, mesh axes whose pending sums must be
        reduced first)`` from the operands' layouts alone; nothing is moved."""
        from ..core.sharding import spmd

        return spmd.infer_output_sharding(self, args, mesh, kwargs)

    def output_device(self, tensors: list[Tensor], kwargs: dict) -> Device:
        if tensors:
            return tensors[0]._impl.device
        from ..core.common.context import get_default_device

        return kwargs.get("device") or get_default_device()

    # ------------------------------------------------------------------ the call pipeline
    def __call__(self, *args, **kwargs):
        arg_leaves, treedef = pytree.tree_flatten(args)
        tensors = [a for a in arg_leaves if isinstance(a, Tensor)]
        batch_dims = 0
        traced = False
        mesh = None
        for t in tensors:
            im = t._impl
            if im.batch_dims > batch_dims:
                batch_dims = im.batch_dims
            traced = traced or im.is_traced
            if mesh is None and im.sharding is not None:
                mesh = im.sharding.mesh
        if mesh is None:
            mesh = kwargs.get("mesh")
        if traced and _tracing_suppressed():
            traced = False
        phys_kwargs = self.adapt_kwargs(args, kwargs, batch_dims)

        out_specs = None
        reduce_axes: set[str] = set()
        if mesh is not None:
            from ..core.sharding import spmd

            args, out_specs_fn, reduce_axes = spmd.prepare(self, args, phys_kwargs, mesh)
            arg_leaves, treedef = pytree.tree_flatten(args)
            tensors = [a for a in arg_leaves if isinstance(a, Tensor)]
        metas = [(t._impl._shape, t._impl.dtype.to_torch()) for t in tensors]
        if config.debug_stream("OP_CALL"):
            desc = "; ".join(f"arg{i}:shape={tuple(t._impl.global_shape)},batch_dims={t._impl.batch_dims},"
                             f"physical={tuple(t._impl._shape)}" for i, t in enumerate(tensors))
            print(f"[NABLA_DEBUG_OP_CALL] op={self.name} max_batch_dims={batch_dims} any_traced={traced} "
                  f"any_sharded={mesh is not None} kwargs={kwargs} adapted_kwargs={phys_kwargs} args=[{desc}]")
        out_meta, out_td = self.infer_outputs(metas, arg_leaves, treedef, phys_kwargs)
        if config.debug_stream("PHYS"):
            print(f"[NABLA_DEBUG_PHYS] {self.name}.infer_outputs: in={[m[0] for m in metas]} kwargs={phys_kwargs} "
                  f"out={[m[0] for m in out_meta]}")
        if mesh is not None:
            out_specs = out_specs_fn([m[0] for m in out_meta])

        node = OpNode(self, [a._impl if isinstance(a, Tensor) else a for a in arg_leaves], treedef, phys_kwargs,
                      kwargs)
        node.out_treedef = out_td
        device = self.output_device(tensors, phys_kwargs)
        out_bd = self.output_batch_dims(batch_dims, phys_kwargs)
        outs = []
        for i, (shp, dt) in enumerate(out_meta):
            impl = TensorImpl(None, shape=shp, dtype=DType.from_torch(dt), device=device,
                              sharding=out_specs[i] if out_specs is not None else None, batch_dims=out_bd,
                              is_traced=traced)
            impl.output_refs = node
            impl.output_index = i
            node.out_refs.append(weakref.ref(impl))
            outs.append(Tensor(impl=impl))
        if traced and len(outs) > 1:
            # auxiliary outputs saved for the backward (pre-activations, statistics) must live
            # as long as the primary output does, even if the caller drops their handles
            outs[0]._impl._keepalive = [o._impl for o in outs[1:]]
        if config.get_flag("EAGER_MAX_GRAPH") and not config.get_flag("TRACING"):
            from ..core.graph.engine import GRAPH

            GRAPH.evaluate(*outs)
        if reduce_axes:
            from .communication import all_reduce

            outs = [all_reduce(o, reduce_axes=reduce_axes, reduce_op=self.collective_reduce_type) for o in outs]
        return pytree.tree_unflatten(out_td, outs)

    # ------------------------------------------------------------------ execution
    def execute(self, node: OpNode) -> list[list[torch.Tensor]]:
        """Run the kernel once per local shard. Returns per-output lists of shard buffers."""
        leaves = node.arg_leaves
        impls = [a for a in leaves if isinstance(a, TensorImpl)]
        n_shards = 1
        mesh = None
        for im in impls:
            if im.sharding is not None:
                mesh = im.sharding.mesh
                n_shards = mesh.num_local
                break
        if mesh is None:
            for r in node.out_refs:
                o = r()
                if o is not None and o.sharding is not None:
                    mesh = o.sharding.mesh
                    n_shards = mesh.num_local
                    break
        per_output: list[list[torch.Tensor]] | None = None
        local_ids = mesh.local_ids if mesh is not None else [0]
        for s in range(n_shards):
            shard_leaves = []
            for a in leaves:
                if isinstance(a, TensorImpl):
                    bufs = a._buffers
                    if bufs is None:
                        raise RuntimeError(f"input of '{self.name}' is not realized (graph ordering bug)")
                    shard_leaves.append(bufs[s] if len(bufs) > 1 else bufs[0])
                else:
                    shard_leaves.append(a)
            args = pytree.tree_unflatten(node.arg_treedef, shard_leaves)
            kw = self.shard_kwargs(node.kwargs, node, s, local_ids[s]) if mesh is not None else node.kwargs
            out = self.kernel(*args, **kw)
            flat = pytree.tree_leaves(out)
            if per_output is None:
                per_output = [[] for _ in flat]
            for i, o in enumerate(flat):
                per_output[i].append(o)
        if config.get_flag("VERIFY_EAGER_SHAPES"):
            self._verify_shapes(node, per_output)
        return per_output

    def _verify_shapes(self, node: OpNode, per_output) -> None:
        for i, r in enumerate(node.out_refs):
            o = r()
            if o is None:
                continue
            for s, buf in enumerate(per_output[i]):
                want = o.physical_local_shape(s) if o._buffers is None else tuple(buf.shape)
                if tuple(buf.shape) != tuple(want):
                    raise RuntimeError(f"{self.name}: predicted shard shape {want} but kernel produced "
                                       f"{tuple(buf.shape)} (output {i}, shard {s})")


# ---------------------------------------------------------------------- families
def _align_batch_dims(tensors: list[Tensor]) -> list[Tensor]:
    """Bring operands to a common number of batch dims and logical rank (numpy broadcasting in
    the logical part, batch dims always leading)."""
    bd = max(t._impl.batch_dims for t in tensors)
    if bd == 0:
        return tensors
    from .view.batch import broadcast_batch_dims
    from .view.axes import unsqueeze_physical

    rank = max(len(t._impl.global_shape) for t in tensors)
    batch_shape = None
    for t in tensors:
        if t._impl.batch_dims == bd:
            batch_shape = t._impl.batch_shape
            break
    out = []
    for t in tensors:
        im = t._impl
        # pad logical rank with leading 1s (after the batch dims)
        while len(t._impl.global_shape) < rank:
            t = unsqueeze_physical(t, axis=t._impl.batch_dims)
        if t._impl.batch_dims < bd:
            t = broadcast_batch_dims(t, batch_shape)
        out.append(t)
    return out


class BinaryOperation(Operation):
    """Elementwise op of two operands with numpy broadcasting."""

    #: name of the op in ``native.kernels.BINARY_OPS`` when the pointwise kernel family covers it
    native_op: str | None = None

    def torch_fn(self, a, b):
        raise NotImplementedError

    def kernel(self, a, b):
        if self.native_op is not None and a.is_cuda:
            from ..native import kernels

            out = kernels.binary(a, b, self.native_op)
            if out is not None:
                return out
        return self.torch_fn(a, b)

    def __call__(self, a, b):
        if not isinstance(a, Tensor):
            a = ensure_tensor(a, b)
        if not isinstance(b, Tensor):
            b = ensure_tensor(b, a)
        if a._impl.batch_dims or b._impl.batch_dims:
            a, b = _align_batch_dims([a, b])
        return super().__call__(a, b)

    def compute_cost(self, input_shapes, output_shapes) -> float:
        return super().compute_cost(input_shapes, output_shapes)


class UnaryOperation(Operation):
    """Elementwise op of one operand. ``_derivative(x, y)`` gives dy/dx for VJP and JVP."""

    #: name of the op in ``native.kernels.UNARY_OPS`` when the pointwise kernel family covers it
    native_op: str | None = None

    def torch_fn(self, x):
        raise NotImplementedError

    def kernel(self, x, **kwargs):
        if self.native_op is not None and x.is_cuda:
            from ..native import kernels

            out = kernels.unary(x, self.native_op)
            if out is not None:
                return out
        return self.torch_fn(x)

    def _derivative(self, x: Tensor, y: Tensor, kwargs: dict) -> Tensor | None:
        return None

    def vjp_rule(self, primals, cotangents, outputs, kwargs):
        d = self._derivative(primals[0], outputs, kwargs)
        if d is None:
            raise NotImplementedError(f"'{self.name}' has no vjp_rule")
        return (cotangents * d,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        d = self._derivative(primals[0], outputs, kwargs)
        if d is None:
            raise NotImplementedError(f"'{self.name}' has no jvp_rule")
        return tangents[0] * d


def _norm_axis(axis: int, rank: int) -> int:
    if axis < 0:
        axis += rank
    if not 0 <= axis < max(rank, 1):
        raise ValueError(f"axis {axis} out of range for rank {rank}")
    return axis


class AxisOp(Operation):
    """Op with an ``axis`` kwarg given in logical coordinates; kernels see physical axes."""

    axis_keys: tuple[str, ...] = ("axis",)
    #: ops that INSERT a dim count the axis against the output rank (reference: ops/base.py:704)
    axis_offset_for_insert: bool = False

    @property
    def axis_arg_names(self) -> set[str]:
        """Names of the kwargs that hold axes (the reference's attribute, ops/base.py:706)."""
        return set(self.axis_keys)

    def adapt_kwargs(self, args, kwargs, batch_dims):
        t = None
        for a in pytree.tree_leaves(args):
            if isinstance(a, Tensor):
                t = a
                break
        rank = len(t._impl.global_shape) if t is not None else 0
        rank = self.logical_rank_for_axis(rank, kwargs)
        out = dict(kwargs)
        own_bd = t._impl.batch_dims if t is not None else 0
        for k in self.axis_keys:
            if k in out and out[k] is not None:
                v = out[k]
                if isinstance(v, (tuple, list)):
                    out[k] = tuple(_norm_axis(int(x), rank) + max(batch_dims, own_bd) for x in v)
                else:
                    out[k] = _norm_axis(int(v), rank) + max(batch_dims, own_bd)
        return out

    def logical_rank_for_axis(self, rank: int, kwargs: dict) -> int:
        return rank


class ReduceOperation(AxisOp):
    """Reduction over one axis with ``keepdims``; the reduced dim is a contracting factor."""

    partial_policy = "any"

    #: name of the reduction in ``native.kernels.REDUCE_OPS`` when the reduction kernels cover it
    native_op: str | None = None

    def torch_reduce(self, x, axis, keepdims):
        raise NotImplementedError

    def infer_output_shape(self, input_shapes, **kwargs) -> tuple[int, ...]:
        """Shape after reducing ``axis`` of ``input_shapes[0]`` (reference: ops/base.py:881-895)."""
        axis, keepdims = int(kwargs.get("axis", 0)), bool(kwargs.get("keepdims", False))
        shape = tuple(int(d) for d in input_shapes[0])
        axis = axis + len(shape) if axis < 0 else axis
        if keepdims:
            return tuple(1 if i == axis else d for i, d in enumerate(shape))
        return tuple(d for i, d in enumerate(shape) if i != axis)

    def kernel(self, x, *, axis: int, keepdims: bool = False):
        if self.native_op is not None and x.is_cuda and x.dim() and x.shape[axis] > 0:
            from ..native import kernels

            out = kernels.reduce(x, axis, self.native_op, keepdims)
            if out is not None:
                return out
        return self.torch_reduce(x, axis, keepdims)

    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, keepdims: bool = False, **kw):
        from ..core.sharding.propagation import OpShardingRule

        rank = len(input_shapes[0])
        ins = {i: [f"d{i}"] for i in range(rank)}
        outs = {}
        j = 0
        for i in range(rank):
            if i == axis:
                if keepdims:
                    outs[j] = [f"r{i}"]
                    j += 1
            else:
                outs[j] = [f"d{i}"]
                j += 1
        return OpShardingRule([ins], [outs])

    def partial_passthrough_axes(self, input_specs, kwargs=None):
        if self.collective_reduce_type != "sum":
            return set()
        return super().partial_passthrough_axes(input_specs, kwargs)


class ShapeOp(Operation):
    """View-like op with shape-valued kwargs."""

    partial_policy = "any"


class CreationOperation(Operation):
    """Op without tensor inputs: ``shape``, ``dtype``, ``device`` come from kwargs.
    Random creation ops draw an independent stream per shard."""

    def output_device(self, tensors, kwargs):
        from ..types import as_device

        return as_device(kwargs.get("device"))


class CollectiveOperation(Operation):
    """Base of the communication ops (see ``nabla_b200.ops.communication``)."""

    partial_policy = "any"

    # ---- cost model used by the auto-sharding solver (reference: nabla/ops/communication/base.py:51-66,
    # 245-279): time of a ring over the devices of ``axes``, in bytes / ``mesh.bandwidth`` units
    @staticmethod
    def _ring_cost(size_bytes: int, mesh, axes, factor: float = 1.0) -> float:
        if not axes:
            return 0.0
        n = 1
        for a in axes:
            n *= mesh.get_axis_size(a)
        if n <= 1:
            return 0.0
        return factor * (n - 1) / n * size_bytes / float(getattr(mesh, "bandwidth", 1.0) or 1.0)

    @classmethod
    def estimate_cost(cls, size_bytes: int, mesh, axes, input_specs=None, output_specs=None) -> float:
        """Cost of moving ``size_bytes`` over the mesh axes ``axes``; 0 for ops that move nothing."""
        return 0.0

    def communication_cost(self, input_specs, output_specs, input_shapes, output_shapes, mesh) -> float:
        if not input_shapes:
            return 0.0
        n = 1
        for d in input_shapes[0]:
            n *= int(d)
        axes: list[str] = []
        if input_specs and input_specs[0]:
            for ds in input_specs[0].dim_specs:
                axes.extend(ds.axes)
        return self.estimate_cost(n * 4, mesh, axes, input_specs, output_specs)
