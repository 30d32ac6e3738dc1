"""``shard_map`` (reference: nabla/transforms/shard_map.py:21-417).

``shard_map(fn, mesh, in_specs, out_specs, auto_sharding=False)`` runs ``fn`` with its inputs
laid out as ``in_specs`` and constrains outputs to ``out_specs``. Because every op already
propagates shardings eagerly, the body is simply executed on the resharded inputs (the
reference records a logical trace and replays it on ``.dual`` tensors). With
``auto_sharding=True`` input specs marked ``None`` are chosen by the cost-based solver in
``nabla_b200.core.sharding.optimizer``.
"""
from __future__ import annotations

from typing import Any, Callable

from ..core.common import pytree
from ..core.sharding.spec import DeviceMesh, DimSpec, ShardingSpec
from ..core.tensor.api import Tensor


def _apply_spec(t: Tensor, mesh: DeviceMesh, spec) -> Tensor:
    from ..ops.communication import reshard_to_spec, shard

    if spec is None:
        return t
    if isinstance(spec, ShardingSpec):
        return reshard_to_spec(t, spec)
    return shard(t, mesh, list(spec))


def _map_specs(tree: Any, specs: Any, mesh: DeviceMesh) -> Any:
    if isinstance(tree, Tensor):
        return _apply_spec(tree, mesh, specs)
    if isinstance(specs, dict) and isinstance(tree, dict):
        return {k: _map_specs(v, specs.get(k), mesh) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)) and isinstance(specs, (list, tuple)) and len(tree) == len(specs) \
            and not all(isinstance(s, (str, type(None))) for s in specs):
        return type(tree)(_map_specs(t, s, mesh) for t, s in zip(tree, specs))
    return pytree.tree_map(lambda t: _apply_spec(t, mesh, specs) if isinstance(t, Tensor) else t, tree)


def shard_map(func: Callable, mesh: DeviceMesh, in_specs: Any, out_specs: Any = None, auto_sharding: bool = False,
              debug: bool = False) -> Callable:
    def wrapped(*args: Any) -> Any:
        specs = in_specs
        if isinstance(specs, dict) and all(isinstance(k, int) for k in specs):
            specs = tuple(specs.get(i) for i in range(len(args)))
        if not isinstance(specs, (list, tuple)) or (len(args) == 1 and len(specs) != 1):
            specs = (specs,) * len(args) if not isinstance(specs, (list, tuple)) else (specs,)
        if auto_sharding:
            from ..core.sharding.optimizer.auto_sharding import solve_for_function

            specs = solve_for_function(func, args, mesh, list(specs), debug=debug)
        placed = tuple(_map_specs(a, s, mesh) for a, s in zip(args, specs))
        out = func(*placed)
        if out_specs is None:
            return out
        ospecs = out_specs
        if isinstance(ospecs, dict) and all(isinstance(k, int) for k in ospecs):
            outs = list(out) if isinstance(out, (list, tuple)) else [out]
            res = [_map_specs(o, ospecs.get(i), mesh) for i, o in enumerate(outs)]
            return type(out)(res) if isinstance(out, (list, tuple)) else res[0]
        return _map_specs(out, ospecs, mesh)

    wrapped.__name__ = f"shard_map({getattr(func, '__name__', 'fn')})"
    return wrapped
