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
