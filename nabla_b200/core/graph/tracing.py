"""Operation records and traces (reference: nabla/core/graph/tracing.py:25-414).

Every op call creates one ``OpNode`` holding the op, its (tensor and static) arguments and
weak references to its outputs. Nodes hold their inputs strongly, outputs hold their node
strongly, so a lazy tensor keeps exactly the subgraph that produces it alive.

A ``Trace`` is the topologically ordered list of nodes between given inputs and outputs; it
is what autodiff replays (backward for VJP, forward for JVP) and what ``print(trace)`` shows.
"""
from __future__ import annotations

import weakref
from typing import Any, Callable, Iterable

from ..common import pytree
from ..tensor.impl import TensorImpl


class OpNode:
    """One recorded operation call."""

    __slots__ = ("op", "arg_leaves", "arg_treedef", "kwargs", "op_kwargs", "out_refs", "out_treedef", "_hash",
                 "__weakref__")

    def __init__(self, op, arg_leaves: list, arg_treedef, kwargs: dict, op_kwargs: dict):
        self.op = op
        self.arg_leaves = arg_leaves          # TensorImpl for tensor arguments, raw value otherwise
        self.arg_treedef = arg_treedef
        self.kwargs = kwargs                  # physical kwargs (axes shifted past batch dims)
        self.op_kwargs = op_kwargs            # kwargs as the user passed them (for VJP/JVP rules)
        self.out_refs: list[weakref.ref] = []
        self.out_treedef = None
        self._hash = None

    # ---- arguments
    def input_impls(self) -> list[TensorImpl]:
        return [a for a in self.arg_leaves if isinstance(a, TensorImpl)]

    def args_as_tensors(self):
        """The original positional arguments with tensors re-wrapped."""
        from ..tensor.api import Tensor

        leaves = [Tensor(impl=a) if isinstance(a, TensorImpl) else a for a in self.arg_leaves]
        return pytree.tree_unflatten(self.arg_treedef, leaves)

    def outputs(self) -> list[TensorImpl | None]:
        return [r() for r in self.out_refs]

    def outputs_as_tensors(self):
        from ..tensor.api import Tensor

        outs = [Tensor(impl=o) if o is not None else None for o in self.outputs()]
        return pytree.tree_unflatten(self.out_treedef, outs) if self.out_treedef is not None else outs

    @property
    def op_name(self) -> str:
        return self.op.name

    # ---- the reference's names for the same things (nabla/core/graph/tracing.py:28-60)
    @property
    def num_outputs(self) -> int:
        return len(self.out_refs)

    @property
    def op_args(self):
        return self.args_as_tensors()

    @property
    def tree_def(self):
        return self.out_treedef

    def get_alive_outputs(self) -> list[TensorImpl | None]:
        """Outputs that are still referenced (``None`` for those already collected)."""
        return self.outputs()

    def __repr__(self) -> str:
        return f"OpNode({self.op.name}, inputs={len(self.input_impls())}, outputs={len(self.out_refs)})"


def topo_nodes(output_impls: Iterable[TensorImpl], stop: Callable[[TensorImpl], bool]) -> list[OpNode]:
    """Nodes needed to produce ``output_impls`` in execution order (iterative DFS).
    ``stop(impl)`` marks boundaries whose producers are not followed."""
    order: list[OpNode] = []
    seen: set[int] = set()
    stack: list[tuple[OpNode, int]] = []
    for impl in output_impls:
        if impl is None or stop(impl):
            continue
        n = impl.output_refs
        if n is None or id(n) in seen:
            continue
        seen.add(id(n))
        stack.append((n, 0))
        while stack:
            node, i = stack.pop()
            inputs = node.arg_leaves
            advanced = False
            while i < len(inputs):
                a = inputs[i]
                i += 1
                if isinstance(a, TensorImpl) and not stop(a):
                    p = a.output_refs
                    if p is not None and id(p) not in seen:
                        seen.add(id(p))
                        stack.append((node, i))
                        stack.append((p, 0))
                        advanced = True
                        break
            if not advanced:
                order.append(node)
    return order


class Trace:
    """Ordered op list between ``inputs`` and ``outputs`` (both pytrees of Tensors)."""

    def __init__(self, inputs: Any, outputs: Any):
        self.inputs = inputs
        self.outputs = outputs
        self.input_impls = [t._impl for t in pytree.tensor_leaves(inputs)]
        self.output_impls = [t._impl for t in pytree.tensor_leaves(outputs)]
        self.nodes: list[OpNode] = []
        self._computed = False

    @staticmethod
    def from_outputs(outputs) -> "Trace":
        tr = Trace((), outputs)
        tr.compute_for_backward()
        return tr

    def compute(self) -> "Trace":
        ids = {id(i) for i in self.input_impls}
        self.nodes = topo_nodes(self.output_impls, lambda impl: id(impl) in ids)
        self._computed = True
        return self

    def compute_for_backward(self) -> "Trace":
        """Walk to true leaves; leaves with ``requires_grad`` become the trace inputs."""
        self.nodes = topo_nodes(self.output_impls, lambda impl: False)
        leaves: dict[int, TensorImpl] = {}
        for n in self.nodes:
            for a in n.input_impls():
                if a.output_refs is None and a.requires_grad:
                    leaves[id(a)] = a
        for o in self.output_impls:
            if o.output_refs is None and o.requires_grad:
                leaves[id(o)] = o
        self.input_impls = list(leaves.values())
        self._computed = True
        return self

    def __len__(self) -> int:
        return len(self.nodes)

    def refresh_graph_values(self) -> None:
        """Make the trace ready for a backward pass. The reference replays the ops here to rebuild
        their values in the graph under construction (nabla/core/graph/tracing.py:189); evaluation
        in this engine walks the recorded nodes on demand, so only the topology has to be known."""
        if not self._computed:
            self.compute()

    def __str__(self) -> str:
        if not self._computed:
            self.compute()
        from .printer import GraphPrinter

        return GraphPrinter(self).to_string()

    __repr__ = __str__


def trace(fn: Callable, *args, **kwargs) -> Trace:
    """Run ``fn`` on traced inputs and return the recorded ``Trace``."""
    from ..tensor.api import Tensor

    tensors = pytree.tensor_leaves((args, kwargs))
    prev = [t._impl.is_traced for t in tensors]
    for t in tensors:
        t._impl.is_traced = True
    try:
        out = fn(*args, **kwargs)
    finally:
        for t, p in zip(tensors, prev):
            t._impl.is_traced = p
    tr = Trace(args if not kwargs else (args, kwargs), out)
    tr.compute()
    return tr


def __getattr__(name: str):
    # `GraphPrinter` lives in `printer.py` (which imports this module); the reference keeps it here
    if name == "GraphPrinter":
        from .printer import GraphPrinter

        return GraphPrinter
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
