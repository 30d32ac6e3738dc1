"""Reverse-mode engine: VJP by replaying a trace backwards
(reference: nabla/core/autograd/backward.py:31-460).

``BackwardEngine`` walks ``reversed(trace.nodes)``, asks each op for input cotangents via
``op.vjp_rule(primals, cotangents, outputs, kwargs)``, un-broadcasts them to the operand's
shape and accumulates. On a mesh, cotangents may carry pending partial sums; contributions
are added while still partial where the add is legal and the cross-device reduction happens
once, at finalisation, when the gradient is laid out like its primal.
"""
from __future__ import annotations

from contextvars import ContextVar
from typing import Any

from ..common import pytree
from ..graph.tracing import Trace
from ..tensor.api import Tensor
from ..tensor.impl import TensorImpl

_NO_TRACE: ContextVar[bool] = ContextVar("nabla_no_trace", default=False)


def tracing_suppressed() -> bool:
    return _NO_TRACE.get()


class suppress_tracing:
    """Ops called inside produce untraced outputs (their graph is dropped once realized)."""

    def __enter__(self):
        self._tok = _NO_TRACE.set(True)

    def __exit__(self, *exc):
        _NO_TRACE.reset(self._tok)


def _reduce_to_shape(g: Tensor, target: Tensor) -> Tensor:
    from ...ops.utils import reduce_to_shape

    if g._impl.batch_dims > target._impl.batch_dims:
        # a cotangent with more vmap dims than its primal: the primal was broadcast over them
        from ...ops.reduction import reduce_sum_physical

        while g._impl.batch_dims > target._impl.batch_dims:
            g = reduce_sum_physical(g, axis=0, keepdims=False)
    if tuple(g._impl.global_shape) != tuple(target._impl.global_shape):
        g = reduce_to_shape(g, tuple(target._impl.global_shape))
    if g.dtype is not target.dtype and target.dtype.is_float():
        from ...ops.unary import cast

        g = cast(g, target.dtype)
    return g


def _match_layout(g: Tensor, target: Tensor) -> Tensor:
    """Resolve pending sums of ``g`` that the primal does not carry and lay it out like it."""
    gs, ts = g._impl.sharding, target._impl.sharding
    if gs is None:
        return g
    from ...ops.communication import all_reduce, reshard_to_spec
    from ..sharding.spmd import replicated_spec

    t_partial = ts.partial_sum_axes if ts is not None else set()
    extra = gs.partial_sum_axes - t_partial
    if extra:
        g = all_reduce(g, reduce_axes=extra)
        gs = g._impl.sharding
    want = ts.clone() if ts is not None else replicated_spec(gs.mesh, len(g._impl._shape))
    want.partial_sum_axes = set(gs.partial_sum_axes)
    if any(a.axes != b.axes for a, b in zip(gs.dim_specs, want.dim_specs)):
        g = reshard_to_spec(g, want)
    return g


class BackwardEngine:
    def __init__(self, trace: Trace, cotangents: Any, *, create_graph: bool = False):
        self.trace = trace
        self.create_graph = create_graph
        self.cot: dict[int, Tensor] = {}
        self.keep: dict[int, TensorImpl] = {}
        # the inputs of the trace always receive a gradient, whatever their flags say now: `trace()`
        # restores `is_traced` on return, and the caller asks for them by naming them as inputs
        self.wanted: set[int] = {id(i) for i in trace.input_impls}
        cots = [c for c in pytree.tree_leaves(cotangents)]
        outs = trace.output_impls
        if len(cots) != len(outs):
            raise ValueError(f"expected {len(outs)} cotangents, got {len(cots)}")
        for o, c in zip(outs, cots):
            if c is not None:
                self._accumulate(o, c if isinstance(c, Tensor) else Tensor.constant(c))

    def _accumulate(self, impl: TensorImpl, g: Tensor, op_name: str = "seed") -> None:
        from ... import config

        k = id(impl)
        self.keep[k] = impl
        cur = self.cot.get(k)
        if config.debug_stream("COT_FLOW"):
            what = "init" if cur is None else "add"
            extra = "" if cur is None else (f"existing_shape={tuple(cur._impl.global_shape)} "
                                            f"existing_batch_dims={cur._impl.batch_dims} existing_phys={tuple(cur._impl._shape)} ")
            print(f"[NABLA_DEBUG_COT_FLOW] {what} op={op_name} target_shape={tuple(impl.global_shape)} "
                  f"target_batch_dims={impl.batch_dims} target_phys={tuple(impl._shape)} {extra}"
                  f"cot_shape={tuple(g._impl.global_shape)} cot_batch_dims={g._impl.batch_dims} cot_phys={tuple(g._impl._shape)}")
        if cur is None:
            self.cot[k] = g
            return
        try:
            self.cot[k] = cur + g
        except Exception:
            if config.debug_stream("COT_ACCUM"):
                print(f"[NABLA_DEBUG_COT_ACCUM] add failed: target shape={tuple(impl.global_shape)} "
                      f"batch_dims={impl.batch_dims} phys={tuple(impl._shape)} | existing shape={tuple(cur._impl.global_shape)} "
                      f"batch_dims={cur._impl.batch_dims} phys={tuple(cur._impl._shape)} | incoming "
                      f"shape={tuple(g._impl.global_shape)} batch_dims={g._impl.batch_dims} phys={tuple(g._impl._shape)}")
            raise

    def run(self) -> dict[int, Tensor]:
        if self.create_graph:
            self._run()
        else:
            with suppress_tracing():
                self._run()
        return self.cot

    def _run(self) -> None:
        for node in reversed(self.trace.nodes):
            outs = node.outputs()
            cots = [self.cot.pop(id(o), None) if o is not None else None for o in outs]
            if all(c is None for c in cots):
                continue
            if node.out_treedef is None or node.out_treedef.kind == "leaf":
                cot_tree = cots[0]
            else:
                cot_tree = _unflatten_with_none(node.out_treedef, cots)
            primals = node.args_as_tensors()
            outputs = node.outputs_as_tensors()
            try:
                in_cots = node.op.vjp_rule(primals, cot_tree, outputs, node.op_kwargs)
            except NotImplementedError as e:
                raise NotImplementedError(f"backward through '{node.op.name}': {e}") from e
            if not isinstance(in_cots, (tuple, list)):
                in_cots = (in_cots,)
            self._scatter(primals, tuple(in_cots), node.op.name)

    def _scatter(self, primals: tuple, in_cots: tuple, op_name: str = "?") -> None:
        for p, g in zip(primals, in_cots):
            if g is None:
                continue
            if isinstance(p, Tensor):
                if not isinstance(g, Tensor):
                    continue
                if not (p._impl.is_traced or p._impl.requires_grad or id(p._impl) in self.wanted):
                    continue
                if not p.dtype.is_float():
                    continue
                self._accumulate(p._impl, _reduce_to_shape(g, p), op_name)
            elif isinstance(p, (list, tuple)) and isinstance(g, (list, tuple)):
                self._scatter(tuple(p), tuple(g), op_name)
            elif isinstance(p, dict) and isinstance(g, dict):
                self._scatter(tuple(p[k] for k in sorted(p)), tuple(g.get(k) for k in sorted(p)), op_name)

    def finalize(self, wrt: list[TensorImpl]) -> dict[int, Tensor]:
        """Gradients for the requested inputs, laid out like the inputs."""
        out: dict[int, Tensor] = {}
        ctx = suppress_tracing() if not self.create_graph else None
        if ctx:
            ctx.__enter__()
        try:
            for impl in wrt:
                g = self.cot.get(id(impl))
                if g is None:
                    continue
                out[id(impl)] = _match_layout(g, Tensor(impl=impl))
        finally:
            if ctx:
                ctx.__exit__(None, None, None)
        return out


def _unflatten_with_none(td, cots):
    """Like tree_unflatten but keeps ``None`` placeholders for outputs without a cotangent."""
    it = iter(cots)

    def rec(d):
        k = d.kind
        if k == "leaf":
            return next(it)
        if k == "none":
            return None
        if k == "list":
            return [rec(c) for c in d.children]
        if k == "tuple":
            return tuple(rec(c) for c in d.children)
        if k == "dict":
            return {key: rec(c) for key, c in zip(d.meta, d.children)}
        return [rec(c) for c in d.children]

    return rec(td)


def backward_on_trace(trace: Trace, cotangents: Any, *, create_graph: bool = False, checkpoint_policy: str = "none"
                      ) -> dict[Tensor, Tensor]:
    """Run the VJP of ``trace``. Returns ``{input Tensor: gradient}`` for the trace inputs.
    ``checkpoint_policy`` is accepted for signature compatibility (no rematerialisation)."""
    eng = BackwardEngine(trace, cotangents, create_graph=create_graph)
    eng.run()
    grads = eng.finalize(trace.input_impls)
    res: dict[Tensor, Tensor] = {}
    for t in pytree.tensor_leaves(trace.inputs):
        g = grads.get(id(t._impl))
        if g is not None:
            res[t] = g
    return res


def backward(outputs: Any, cotangents: Any = None, *, retain_graph: bool = False, create_graph: bool = False) -> None:
    """PyTorch-style: fill ``.grad`` of every ``requires_grad`` leaf reachable from ``outputs``
    (accumulating into an existing ``.grad``) and realize the gradients in one batch."""
    from ...ops.creation import ones_like

    outs = pytree.tensor_leaves(outputs)
    if cotangents is None:
        if len(outs) != 1:
            raise ValueError("backward() requires explicit cotangents for multiple outputs.")
        o = outs[0]
        n = 1
        for d in o._impl.global_shape:
            n *= d
        if n != 1:
            raise ValueError(f"backward() requires cotangents for non-scalar outputs. Output has shape {o.shape}.")
        cotangents = ones_like(o)
    tr = Trace((), outputs)
    tr.compute_for_backward()
    eng = BackwardEngine(tr, cotangents, create_graph=create_graph)
    eng.run()
    grads = eng.finalize(tr.input_impls)
    todo = []
    for impl in tr.input_impls:
        g = grads.get(id(impl))
        if g is None:
            continue
        if impl.grad is not None:
            with suppress_tracing():
                g = impl.grad + g
        impl.grad = g
        impl.cotangent = g
        todo.append(g)
    if todo:
        from ..tensor.api import realize_all

        realize_all(*todo)
    if not retain_graph and not create_graph:
        # drop the recorded graph of intermediates so their buffers can be freed
        for node in tr.nodes:
            for o in node.outputs():
                if o is not None and o.is_realized and not o.requires_grad:
                    o.output_refs = None
