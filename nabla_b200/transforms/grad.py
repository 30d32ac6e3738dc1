"""``grad`` and ``value_and_grad`` (reference: nabla/transforms/grad.py:21-172).

Trace the function, seed a ones cotangent on its scalar output, replay the trace backwards.
With the default ``create_graph=True`` everything stays lazy and differentiable, so forward,
backward and a following optimizer update evaluate as ONE plan at the next ``realize``.
"""
from __future__ import annotations

from typing import Any, Callable

from ..core.autograd.backward import backward_on_trace
from ..core.common import pytree
from ..core.graph.tracing import Trace, trace
from ..core.tensor.api import Tensor
from .utils import select_argnums


def _run(fun, args, kwargs, argnums, has_aux, create_graph, realize, want_value):
    from ..ops.creation import ones_like

    argn = (argnums,) if isinstance(argnums, int) else tuple(argnums)
    diff_args = tuple(args[i] for i in argn)
    tensors = pytree.tensor_leaves(diff_args)
    prev = [t._impl.is_traced for t in tensors]
    for t in tensors:
        t._impl.is_traced = True
    try:
        out = fun(*args, **kwargs)
    finally:
        pass
    aux = None
    if has_aux:
        out, aux = out
    if not isinstance(out, Tensor):
        raise TypeError(f"grad: output must be a Tensor, got {type(out)}")
    # a non-scalar output is pulled back with a cotangent of ones (the gradient of its sum), exactly as
    # the reference does (nabla/transforms/grad.py:60-62); its graph-tracing tutorial relies on it
    tr = Trace(diff_args, out)
    tr.compute()
    try:
        gmap = backward_on_trace(tr, ones_like(out), create_graph=create_graph)
    finally:
        for t, p in zip(tensors, prev):
            t._impl.is_traced = p
    leaves, td = pytree.tree_flatten(diff_args)
    gleaves = [gmap.get(l) if isinstance(l, Tensor) else None for l in leaves]
    if not create_graph:
        _release_trace(tr, keep=[out] + pytree.tensor_leaves(aux))
        if realize:
            from ..core.tensor.api import realize_all

            todo = [g for g in gleaves if isinstance(g, Tensor)] + ([out] if want_value else [])
            realize_all(*todo)
    grads_struct = pytree.tree_unflatten(td, gleaves)
    grads = grads_struct[0] if isinstance(argnums, int) else grads_struct
    return out, grads, aux


def _release_trace(tr: Trace, keep) -> None:
    """After a first-order gradient nobody will differentiate again: un-trace intermediates so
    that executed nodes drop their inputs (activations are freed as soon as they are dead)."""
    keep_ids = {id(t._impl) for t in keep}
    in_ids = {id(i) for i in tr.input_impls}
    for node in tr.nodes:
        for o in node.outputs():
            if o is not None and id(o) not in in_ids and not o.requires_grad:
                o.is_traced = False
                if o.is_realized:
                    o.output_refs = None


def grad(fun: Callable, argnums: int | tuple[int, ...] = 0, create_graph: bool = True, realize: bool = True,
         has_aux: bool = False) -> Callable:
    """Gradient of a scalar-valued function with respect to ``argnums``."""

    def wrapper(*args: Any, **kwargs: Any):
        _, g, aux = _run(fun, args, kwargs, argnums, has_aux, create_graph, realize, False)
        return (g, aux) if has_aux else g

    wrapper.__name__ = f"grad({getattr(fun, '__name__', 'fn')})"
    return wrapper


def value_and_grad(fun: Callable, argnums: int | tuple[int, ...] = 0, create_graph: bool = True, realize: bool = True,
                   has_aux: bool = False) -> Callable:
    """Like ``grad`` but also returns the function value: ``(value, grads)``."""

    def wrapper(*args: Any, **kwargs: Any):
        v, g, aux = _run(fun, args, kwargs, argnums, has_aux, create_graph, realize, True)
        return ((v, aux), g) if has_aux else (v, g)

    wrapper.__name__ = f"value_and_grad({getattr(fun, '__name__', 'fn')})"
    return wrapper
