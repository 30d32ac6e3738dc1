"""Trace helpers (reference: nabla/core/graph/utils.py:17-106)."""
from __future__ import annotations

from .tracing import Trace, topo_nodes


def get_operations_topological(outputs) -> list:
    from ..common import pytree

    return topo_nodes([t._impl for t in pytree.tensor_leaves(outputs)], lambda i: False)


def print_trace_graph(trace: Trace) -> None:
    print(str(trace))
