"""Op helpers: un-broadcasting and the custom-kernel entry point
(reference: nabla/ops/utils.py:765-824, nabla/core/autograd/backward.py:31-54)."""
from __future__ import annotations

from typing import Any, Sequence

from ..core.tensor.api import Tensor


def reduce_to_shape(x: Tensor, shape: Sequence[int]) -> Tensor:
    """Sum ``x`` over the dimensions that numpy broadcasting added to reach ``x.shape`` from
    ``shape`` (used to map cotangents back onto broadcast operands)."""
    from .reduction import reduce_sum

    shape = tuple(int(s) for s in shape)
    cur = tuple(x._impl.global_shape)
    if cur == shape:
        return x
    extra = len(cur) - len(shape)
    if extra > 0:
        x = reduce_sum(x, axis=tuple(range(extra)), keepdims=False)
        cur = tuple(x._impl.global_shape)
    axes = tuple(i for i, (c, s) in enumerate(zip(cur, shape)) if s == 1 and c != 1)
    if axes:
        x = reduce_sum(x, axis=axes, keepdims=True)
    if tuple(x._impl.global_shape) != shape:
        from .view import reshape

        x = reshape(x, shape)
    return x


def call_custom_kernel(func_name: str, kernel_path: Any, values, out_types, device=None, **kwargs):
    """Run a registered custom CUDA (or host) kernel as one op.

    Signature kept from the reference (nabla/ops/utils.py:765-824), where ``kernel_path`` is a
    directory of Mojo kernels. Here ``kernel_path`` may be a ``.cu`` file (compiled with nvcc
    for sm_100a on first use), a built ``.so`` or ``None`` when ``func_name`` was registered
    with ``nabla_b200.ops.custom.register_kernel``. ``out_types`` describes the outputs:
    ``(shape, dtype)`` pairs or Tensors to imitate.
    """
    from .custom import call_custom_kernel as impl

    return impl(func_name, kernel_path, values, out_types, device=device, **kwargs)


# ---------------------------------------------------------------- hashable keys (reference: nabla/ops/utils.py:74-160)
_HASHABLE_CACHE: dict[int, Any] = {}


def _clear_hashable_cache() -> None:
    """Drop the per-object cache of ``_make_hashable``."""
    _HASHABLE_CACHE.clear()


def _get_tensor_hash(t) -> tuple:
    """Structural key of a tensor: shape, dtype, device and sharding signature (no values)."""
    impl = t._impl if hasattr(t, "_impl") else t
    sp = impl.sharding
    sharding_key = None
    if sp is not None:
        mesh = sp.mesh
        sharding_key = ((mesh.name, tuple(mesh.shape), tuple(mesh.axis_names)),
                        tuple((tuple(d.axes),) for d in sp.dim_specs), tuple(sorted(sp.replicated_axes)),
                        tuple(sorted(sp.partial_sum_axes)))
    return ("tensor", tuple(int(d) for d in impl._shape), str(impl.dtype), str(impl.device), int(impl.batch_dims),
            sharding_key)


def _make_hashable(obj: Any) -> Any:
    """Stable, hashable key of an op argument: tensors by structure, containers element-wise,
    everything else by value (or by ``repr`` when it is not hashable)."""
    from ..core.tensor.api import Tensor

    if isinstance(obj, Tensor):
        key = _HASHABLE_CACHE.get(id(obj))
        if key is None:
            key = _get_tensor_hash(obj)
            if len(_HASHABLE_CACHE) > 1024:
                _HASHABLE_CACHE.clear()
            _HASHABLE_CACHE[id(obj)] = key
        return key
    if isinstance(obj, (list, tuple)):
        return tuple(_make_hashable(o) for o in obj)
    if isinstance(obj, dict):
        return tuple(sorted(((k, _make_hashable(v)) for k, v in obj.items()), key=lambda kv: str(kv[0])))
    if isinstance(obj, (set, frozenset)):
        return tuple(sorted((_make_hashable(o) for o in obj), key=repr))
    try:
        hash(obj)
        return obj
    except TypeError:
        return repr(obj)


# ---------------------------------------------------------------- stages of an op call, one by one
# (reference: nabla/ops/utils.py:410-762, where `Operation.__call__` is assembled from these).
# `Operation.__call__` of this package does the same work inline; these give the same answers for
# code that inspects or drives the steps itself.
def ensure_tensor(x: Any, like: Any = None) -> Tensor:
    from .base import ensure_tensor as impl

    return impl(x, like)


def collect_metadata(args: Any) -> tuple[int, bool, bool, bool]:
    """``(max vmap depth, any traced, any sharded, any with a tangent attached)`` over the tensors in
    ``args``. Forward mode here replays a trace instead of attaching tangents to tensors, so the
    last entry is True only for tensors a caller gave a ``tangent`` by hand."""
    from ..core.common import pytree

    depth, traced, sharded, tangent = 0, False, False, False
    for t in pytree.tensor_leaves(args):
        im = t._impl
        depth = max(depth, int(im.batch_dims))
        traced = traced or bool(im.is_traced)
        sharded = sharded or im.sharding is not None
        tangent = tangent or im.tangent is not None
    return depth, traced, sharded, tangent


def compute_structural_hash(op_name: str, resharded_args: Any, adapted_kwargs: dict | None) -> tuple:
    """Key of an op call that ignores values: the op, the structure of every argument and kwarg."""
    return (op_name, tuple(_make_hashable(a) for a in resharded_args),
            tuple(sorted(((k, _make_hashable(v)) for k, v in (adapted_kwargs or {}).items()), key=lambda kv: str(kv[0]))))


def apply_auto_reduction(op: Any, output: Any, mesh: Any, reduce_axes: Any) -> Any:
    """All-reduce every tensor of ``output`` over ``reduce_axes`` (the op's own reduction kind: sum,
    or max / min for the extreme reductions); unchanged when there is nothing to reduce."""
    if not (reduce_axes and mesh):
        return output
    from ..core.common import pytree
    from .communication import all_reduce

    kind = getattr(op, "collective_reduce_type", "sum") or "sum"
    return pytree.tree_map(lambda t: all_reduce(t, reduce_axes=set(reduce_axes), reduce_op=kind) if isinstance(t, Tensor) else t,
                           output)


def verify_eager_shapes(op: Any, execution_results: Any, output_physical_shapes: Any) -> None:
    """With ``VERIFY_EAGER_SHAPES`` on: raise when a computed buffer's shape is not the inferred
    one. ``execution_results`` are per-output lists of per-shard buffers, ``output_physical_shapes``
    the matching shapes."""
    from .. import config

    if not config.get_flag("VERIFY_EAGER_SHAPES") or execution_results is None or output_physical_shapes is None:
        return
    for o, (bufs, shapes) in enumerate(zip(execution_results, output_physical_shapes)):
        for i, (b, want) in enumerate(zip(bufs, shapes)):
            if tuple(b.shape) != tuple(int(d) for d in want):
                raise RuntimeError(f"{getattr(op, 'name', op)}: output {o} shard {i} has shape {tuple(b.shape)}, "
                                   f"shape inference said {tuple(want)}")
