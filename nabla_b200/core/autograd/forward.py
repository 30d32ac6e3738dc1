"""Forward-mode engine: JVP by replaying a trace forwards
(reference: nabla/core/autograd/forward.py:34-218).

Walks the nodes in execution order, looks up the tangents of each node's tensor inputs
(zeros where none flows), and calls ``op.jvp_rule(primals, tangents, outputs, kwargs)``.
An op that returns ``None`` from its rule contributes a zero tangent; one without a rule raises.
"""
from __future__ import annotations

from ... import config as _config

from typing import Any

from ..common import pytree
from ..graph.tracing import Trace
from ..tensor.api import Tensor
from ..tensor.impl import TensorImpl
from .backward import suppress_tracing


def _lay_out_like(t: Tensor, primal: TensorImpl) -> Tensor:
    """An input tangent laid out like its primal (same mesh axes on the same dims, no pending sums;
    gathered when the primal is not on a mesh). The JVP rules combine tangents with values derived
    from the primal dim by dim, so the two must be split the same way."""
    ts, ps = t._impl.sharding, primal.sharding
    if ts is None and ps is None:
        return t
    if ps is None:
        return t.gather()
    if t._impl.batch_dims != primal.batch_dims or len(t._impl._shape) != len(primal._shape):
        return t                      # a basis mapped over extra dims (jacfwd): the rules align those themselves
    from ...ops.communication import reshard_to_spec
    from ..sharding.spec import needs_reshard

    want = ps.clone()
    want.partial_sum_axes = set()
    return reshard_to_spec(t, want) if ts is None or needs_reshard(ts, want) else t


class ForwardEngine:
    def __init__(self, trace: Trace, tangents: Any, *, create_graph: bool = True):
        self.trace = trace
        self.create_graph = create_graph
        self.tan: dict[int, Tensor] = {}
        tans = pytree.tree_leaves(tangents)
        ins = trace.input_impls
        if len(tans) != len(ins):
            raise ValueError(f"expected {len(ins)} tangents, got {len(tans)}")
        for i, t in zip(ins, tans):
            if t is not None:
                self.tan[id(i)] = _lay_out_like(t, i) if isinstance(t, Tensor) else t

    def run(self) -> None:
        if self.create_graph:
            self._run()
        else:
            with suppress_tracing():
                self._run()

    def _run(self) -> None:
        from ...ops.creation import zeros_like

        for node in self.trace.nodes:
            ins = node.input_impls()
            if not any(id(i) in self.tan for i in ins):
                continue
            primals = node.args_as_tensors()

            def tan_of(p):
                if isinstance(p, Tensor):
                    t = self.tan.get(id(p._impl))
                    if t is None:
                        return zeros_like(p) if p.dtype.is_float() else None
                    return t
                if isinstance(p, (list, tuple)):
                    return type(p)(tan_of(x) for x in p)
                return None

            tangents = tuple(tan_of(p) for p in primals)
            outputs = node.outputs_as_tensors()
            # an op that is not differentiable returns None from its rule; one WITHOUT a rule raises,
            # and that is passed on: a zero tangent here would be a silently wrong derivative
            try:
                out_t = node.op.jvp_rule(primals, tangents, outputs, node.op_kwargs)
            except NotImplementedError as e:
                if not any(o is not None and o.dtype.is_float() for o in node.outputs()):
                    out_t = None          # integer / bool outputs carry no tangent whatever the op
                else:
                    raise NotImplementedError(f"forward mode through '{node.op.name}': {e}") from e
            if out_t is None:
                continue
            outs = node.outputs()
            flat = pytree.tree_leaves(out_t, is_leaf=lambda x: x is None or isinstance(x, Tensor))
            for o, t in zip(outs, flat):
                if o is not None and isinstance(t, Tensor):
                    if t.dtype is not o.dtype and o.dtype.is_float():
                        from ...ops.unary import cast

                        t = cast(t, o.dtype)
                    if tuple(t._impl.global_shape) != tuple(o.global_shape):
                        from ...ops.view import broadcast_to

                        t = broadcast_to(t, tuple(o.global_shape))
                    if _config.debug_stream("NESTED_JVP"):
                        print("[NABLA_DEBUG_NESTED_JVP]", node.op.name, "tangent_has_parent=", t._impl.output_refs is not None)
                    self.tan[id(o)] = t

    def output_tangents(self) -> list[Tensor | None]:
        return [self.tan.get(id(o)) for o in self.trace.output_impls]


def forward_on_trace(trace: Trace, tangents: Any, *, create_graph: bool = True) -> list[Tensor | None]:
    eng = ForwardEngine(trace, tangents, create_graph=create_graph)
    eng.run()
    return eng.output_tangents()
