"""Graph walks over recorded op nodes (reference: nabla/core/graph/utils.py:17-106).

All four helpers take tensors or ``TensorImpl`` objects (a single one or any pytree of them) and
are built on the iterative ``tracing.topo_nodes`` walk, so deep graphs (thousands of chained ops)
do not hit the interpreter's recursion limit.
"""
from __future__ import annotations

from typing import Any, Callable

from ..tensor.impl import TensorImpl
from .tracing import OpNode, Trace, topo_nodes


def _impls(outputs: Any) -> list[TensorImpl]:
    from ..common import pytree

    if isinstance(outputs, Trace):
        return [t._impl for t in pytree.tensor_leaves(outputs.outputs)]
    leaves = pytree.tree_leaves(outputs, is_leaf=lambda x: isinstance(x, TensorImpl) or hasattr(x, "_impl"))
    return [l if isinstance(l, TensorImpl) else l._impl for l in leaves if isinstance(l, TensorImpl) or hasattr(l, "_impl")]


def _nodes(outputs: Any) -> list[OpNode]:
    return topo_nodes(_impls(outputs), lambda impl: False)


def get_operations_topological(outputs: Any) -> list[tuple[int, list[TensorImpl]]]:
    """One ``(node id, outputs of that node that are still alive)`` entry per recorded op call that
    the given outputs depend on, producers before consumers."""
    return [(id(n), [o for o in n.outputs() if o is not None]) for n in _nodes(outputs)]


def get_all_impls_topological(outputs: Any) -> list[TensorImpl]:
    """Every tensor the given outputs depend on (leaves included), each once, a tensor always after
    the tensors it was computed from."""
    seen: set[int] = set()
    order: list[TensorImpl] = []

    def add(impl: TensorImpl) -> None:
        if id(impl) not in seen:
            seen.add(id(impl))
            order.append(impl)

    for n in _nodes(outputs):
        for a in n.input_impls():
            add(a)
        for o in n.outputs():
            if o is not None:
                add(o)
    for impl in _impls(outputs):      # outputs that are leaves themselves
        add(impl)
    return order


def apply_to_operations(outputs: Any, fn: Callable[[int, list[TensorImpl]], None]) -> None:
    """Call ``fn(node id, alive outputs)`` for every op call, consumers first (the order a backward
    sweep visits them)."""
    for op_id, outs in reversed(get_operations_topological(outputs)):
        fn(op_id, outs)


def print_trace_graph(outputs: Any, show_siblings: bool = True) -> None:
    """Print the recorded computation: a ``Trace`` prints as its jaxpr-like text, anything else as a
    numbered list of op calls with input / output counts (and sibling outputs of multi-output ops)."""
    if isinstance(outputs, Trace):
        print(str(outputs))
        return
    ops = get_operations_topological(outputs)
    print(f"Computation Graph ({len(ops)} operations):")
    print("-" * 60)
    for idx, (_, outs) in enumerate(ops):
        head = outs[0] if outs else None
        name = head.op_name if head is not None else "unknown"
        print(f"{idx:3d}. {name}")
        print(f"      Inputs: {len(head.parents) if head is not None else 0}")
        print(f"      Outputs: {len(outs)}")
        if show_siblings and len(outs) > 1:
            for i, o in enumerate(outs):
                print(f"        [{i}] shape={tuple(o.logical_shape)}, index={o.output_index}")
    print("-" * 60)
