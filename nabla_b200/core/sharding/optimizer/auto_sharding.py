"""Cost-based auto-sharding (the reference's solver, nabla/core/sharding/optimizer/
auto_sharding.py:19-256, cannot be imported; this is a working seed-and-propagate solver with
the same idea).

For each un-annotated input of a traced function the solver enumerates candidate layouts
(replicated, or one dimension split over one mesh axis), runs the factor propagation through
the recorded ops *on shapes only*, and scores every candidate by

    sum over ops of  compute_cost / (shards that divide the op's work)
    + bytes moved by the collectives the propagation had to insert / mesh.bandwidth

keeping the cheapest. Matmuls dominate, so the decision is in effect "data parallel vs model
parallel per matmul", as in the reference's description.
"""
from __future__ import annotations

import itertools
import math
from typing import Any, Callable

from ...common import pytree
from ..spec import DeviceMesh, DimSpec, ShardingSpec

_COMM = {"all_reduce", "all_gather", "gather_all_axes", "reduce_scatter", "shard", "ppermute"}


def candidate_specs(shape: tuple[int, ...], mesh: DeviceMesh) -> list[list[Any]]:
    cands: list[list[Any]] = [[None] * len(shape)]
    for d, n in enumerate(shape):
        for ax in mesh.axis_names:
            k = mesh.get_axis_size(ax)
            if k > 1 and n % k == 0:
                spec: list[Any] = [None] * len(shape)
                spec[d] = ax
                cands.append(spec)
    return cands


def estimate_cost(func: Callable, args: tuple, mesh: DeviceMesh, specs: list) -> float:
    """Trace ``func`` on inputs laid out as ``specs`` (lazily: nothing executes) and sum op and
    communication costs of the recorded graph."""
    from ...graph.tracing import topo_nodes
    from ...tensor.api import Tensor
    from ....ops.communication import shard

    placed = []
    for a, s in zip(args, specs):
        if isinstance(a, Tensor) and s is not None:
            placed.append(shard(a, mesh, list(s)))
        else:
            placed.append(a)
    out = func(*placed)
    impls = [t._impl for t in pytree.tensor_leaves(out)]
    nodes = topo_nodes(impls, lambda i: i.is_realized)
    total = 0.0
    for n in nodes:
        ins = [tuple(i._shape) for i in n.input_impls()]
        outs = [tuple(o._shape) for o in n.outputs() if o is not None]
        if n.op.name in _COMM:
            nbytes = sum(math.prod(s) for s in outs) * 2.0
            if n.op.name == "shard":
                continue
            total += nbytes / max(mesh.bandwidth, 1e-9) * 1e-3
            continue
        shards = 1
        for o in n.outputs():
            if o is not None and o.sharding is not None:
                shards = max(shards, o.sharding.total_shards * max(1, math.prod(
                    mesh.get_axis_size(a) for a in o.sharding.partial_sum_axes)))
        try:
            total += n.op.compute_cost(ins, outs) / shards
        except Exception:
            pass
    return total


def solve_for_function(func: Callable, args: tuple, mesh: DeviceMesh, specs: list, debug: bool = False) -> list:
    """Fill the ``None`` entries of ``specs`` (one per positional arg) with the cheapest layout."""
    from ...tensor.api import Tensor

    specs = list(specs) + [None] * (len(args) - len(specs))
    free = [i for i, (a, s) in enumerate(zip(args, specs)) if s is None and isinstance(a, Tensor)]
    if not free:
        return specs
    options = [candidate_specs(tuple(args[i]._impl.global_shape), mesh) for i in free]
    best, best_cost = None, float("inf")
    combos = itertools.product(*options)
    for k, combo in enumerate(combos):
        if k >= 256:
            break
        trial = list(specs)
        for i, c in zip(free, combo):
            trial[i] = c
        try:
            cost = estimate_cost(func, args, mesh, trial)
        except Exception:
            continue
        if debug:
            print(f"[auto_sharding] {[trial[i] for i in free]} -> {cost:.4g}")
        if cost < best_cost:
            best, best_cost = trial, cost
    return best if best is not None else specs


class AutoShardingSolver:
    """Object form kept for API parity with the reference's solver entry point."""

    def __init__(self, mesh: DeviceMesh, debug: bool = False):
        self.mesh = mesh
        self.debug = debug

    def solve(self, func: Callable, args: tuple, specs: list | None = None) -> list:
        return solve_for_function(func, args, self.mesh, specs or [None] * len(args), debug=self.debug)


# ---------------------------------------------------------------------------------------------
# Graph-as-JSON interface (reference: nabla/core/sharding/optimizer/auto_sharding.py:19-330 and the
# extractor in nabla/transforms/shard_map.py:260-417). The reference's module imports a
# `PropagationStrategy` its propagation module no longer has, so it cannot be loaded; this one works.
#
#   graph    = {"tensors": [{"id", "shape", "fixed_sharding": {"dims": [...], "replicated": [...]} | None}],
#               "nodes":   [{"id", "op_name", "inputs": [tensor ids], "outputs": [tensor ids],
#                            "sharding_rule": {"equation", "factor_sizes"}, "compute_stats": {"flops"}}]}
#   solution = {"nodes": {node id: {"inputs": {i: {"dims", "replicated"}}, "outputs": {...}}}}
def graph_to_json(func: Callable, args: tuple, indent: int | None = None) -> str:
    """Trace ``func(*args)`` and describe the recorded ops in the JSON form above. Layouts that the
    arguments already have become ``fixed_sharding`` entries."""
    import json

    from ...graph.tracing import trace

    tr = trace(func, *args)
    ids: dict[int, int] = {}
    tensors: list[dict] = []

    def tid(impl) -> int:
        k = id(impl)
        if k not in ids:
            ids[k] = len(tensors)
            fixed = None
            if impl.sharding is not None:
                fixed = {"dims": [list(d.axes) if d.axes else None for d in impl.sharding.dim_specs],
                         "replicated": sorted(impl.sharding.replicated_axes)}
            tensors.append({"id": ids[k], "shape": [int(d) for d in impl._shape], "fixed_sharding": fixed})
        return ids[k]

    nodes = []
    for i, n in enumerate(tr.nodes):
        ins = n.input_impls()
        outs = [o for o in n.outputs() if o is not None]
        in_shapes = [tuple(int(d) for d in x._shape) for x in ins]
        out_shapes = [tuple(int(d) for d in x._shape) for x in outs]
        rule_info = None
        try:
            rule = n.op.sharding_rule(in_shapes, out_shapes, **(n.op_kwargs or {}))
            if rule is not None:
                rule_info = {"equation": rule.to_einsum_notation(), "factor_sizes": dict(rule.factor_sizes)}
        except Exception:
            pass
        try:
            flops = float(n.op.compute_cost(in_shapes, out_shapes))
        except Exception:
            flops = 0.0
        nodes.append({"id": i, "op_name": n.op.name, "inputs": [tid(x) for x in ins], "outputs": [tid(x) for x in outs],
                      "sharding_rule": rule_info, "compute_stats": {"flops": flops}})
    return json.dumps({"tensors": tensors, "nodes": nodes}, indent=indent)


class AutoSharding:
    """Seed-and-propagate solver over a JSON graph. Every matmul is seeded with the cheaper of
    "split the rows" (data parallel, no communication) and "split the contraction" (model parallel,
    one all-reduce of the output) on the first mesh axis; the seeds then flow through every op's
    factor rule in both directions until nothing changes. Fixed layouts are never overwritten."""

    SEED_PRIORITY = 5
    MAX_SWEEPS = 100

    def __init__(self, mesh_shape: tuple[int, ...], axis_names: tuple[str, ...]):
        self.mesh_shape = tuple(int(d) for d in mesh_shape)
        self.axis_names = tuple(axis_names)
        self.total_devices = math.prod(self.mesh_shape) if self.mesh_shape else 1
        self.mesh = DeviceMesh("solver_mesh", self.mesh_shape, self.axis_names, devices=list(range(self.total_devices)))

    # ---- pieces
    def _initial_spec(self, shape, fixed) -> ShardingSpec:
        if fixed:
            dims = [DimSpec([], is_open=True) if ax is None else DimSpec([ax] if isinstance(ax, str) else list(ax), is_open=False)
                    for ax in fixed.get("dims", [])]
            dims += [DimSpec([], is_open=True) for _ in range(len(shape) - len(dims))]
            return ShardingSpec(self.mesh, dims, replicated_axes=set(fixed.get("replicated", [])))
        return ShardingSpec(self.mesh, [DimSpec([], is_open=True) for _ in shape])

    @staticmethod
    def _free_for(spec: ShardingSpec, dim: int, axis: str) -> bool:
        """Can ``axis`` go on ``dim``: it is there already, or the dim is open and empty and no other
        dim of the tensor uses the axis."""
        dim = dim + len(spec.dim_specs) if dim < 0 else dim
        if not 0 <= dim < len(spec.dim_specs):
            return False
        if spec.dim_specs[dim].axes == [axis]:
            return True
        elsewhere = any(axis in d.axes for i, d in enumerate(spec.dim_specs) if i != dim)
        return not elsewhere and spec.dim_specs[dim].is_open and not spec.dim_specs[dim].axes \
            and axis not in spec.replicated_axes

    def _seed(self, spec: ShardingSpec, dim: int, axis: str) -> None:
        dim = dim + len(spec.dim_specs) if dim < 0 else dim
        if self._free_for(spec, dim, axis) and not spec.dim_specs[dim].axes:
            spec.dim_specs[dim] = DimSpec([axis], is_open=True, priority=self.SEED_PRIORITY)

    def _seed_matmul(self, node: dict, tensors: dict, specs: dict, debug: bool) -> dict | None:
        from ....ops.communication import AllReduceOp

        rule = node.get("sharding_rule")
        if not rule or not self.axis_names:
            return None
        sizes = rule.get("factor_sizes", {})
        axis, width = self.axis_names[0], self.mesh_shape[0]
        work = float(node.get("compute_stats", {}).get("flops", 0.0)) / max(width, 1)
        a, b = node["inputs"][:2]
        out = node["outputs"][0]
        rows = tensors[a]["shape"][-2] if len(tensors[a]["shape"]) >= 2 else sizes.get("m", 1)
        inner = tensors[a]["shape"][-1]
        dp_ok = rows % width == 0 and self._free_for(specs[a], -2, axis) and self._free_for(specs[out], -2, axis)
        mp_ok = inner % width == 0 and self._free_for(specs[a], -1, axis) and self._free_for(specs[b], -2, axis)
        dp = work if dp_ok else float("inf")
        mp = float("inf")
        if mp_ok:
            mp = work + AllReduceOp.estimate_cost(4 * math.prod(tensors[out]["shape"]), self.mesh, [axis])
        if debug:
            print(f"[AutoSharding] node {node['id']} matmul: data-parallel {dp:.3g}, model-parallel {mp:.3g}")
        if dp == mp == float("inf"):
            return {"strategy": "none", "axis": axis}
        if dp <= mp:
            self._seed(specs[a], -2, axis)
            self._seed(specs[out], -2, axis)
            return {"strategy": "dp", "axis": axis}
        self._seed(specs[a], -1, axis)
        self._seed(specs[b], -2, axis)
        return {"strategy": "mp", "axis": axis}

    def _propagate(self, node: dict, tensors: dict, specs: dict) -> bool:
        from ..propagation import OpShardingRuleTemplate, PropagationStrategy, propagate_sharding

        info = node.get("sharding_rule")
        if not info or "equation" not in info:
            return False
        in_shapes = [tuple(tensors[t]["shape"]) for t in node["inputs"]]
        out_shapes = [tuple(tensors[t]["shape"]) for t in node["outputs"]]
        try:
            rule = OpShardingRuleTemplate.parse(info["equation"], in_shapes).instantiate(in_shapes, out_shapes)
        except Exception:
            return False
        return propagate_sharding(rule, [specs[t] for t in node["inputs"]], [specs[t] for t in node["outputs"]],
                                  strategy=PropagationStrategy.BASIC)

    @staticmethod
    def _as_dict(spec: ShardingSpec) -> dict:
        return {"dims": [list(d.axes) if d.axes else None for d in spec.dim_specs],
                "replicated": sorted(spec.replicated_axes)}

    # ---- entry point
    def solve(self, json_graph: str, debug: bool = False) -> dict:
        import json

        graph = json.loads(json_graph) if isinstance(json_graph, str) else json_graph
        tensors = {t["id"]: t for t in graph["tensors"]}
        specs = {i: self._initial_spec(tuple(t["shape"]), t.get("fixed_sharding")) for i, t in tensors.items()}
        self.seeds: dict[str, dict] = {}
        for node in graph["nodes"]:
            if node["op_name"] == "matmul":
                s = self._seed_matmul(node, tensors, specs, debug)
                if s:
                    self.seeds[str(node["id"])] = s
        for sweep in range(self.MAX_SWEEPS):
            if not any([self._propagate(n, tensors, specs) for n in graph["nodes"]]):
                break
        if debug:
            print(f"[AutoSharding] settled after {sweep + 1} sweeps")
        return {"nodes": {str(n["id"]): {"inputs": {str(i): self._as_dict(specs[t]) for i, t in enumerate(n["inputs"])},
                                         "outputs": {str(i): self._as_dict(specs[t]) for i, t in enumerate(n["outputs"])}}
                          for n in graph["nodes"]}}
