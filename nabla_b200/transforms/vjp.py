"""``vjp`` (reference: nabla/transforms/vjp.py:28-94): ``out, pullback = vjp(fn, *primals)``;
``pullback(cotangent)`` returns one gradient per primal (a tuple)."""
from __future__ import annotations

from typing import Any, Callable

from ..core.autograd.backward import backward_on_trace
from ..core.common import pytree
from ..core.graph.tracing import Trace
from ..core.tensor.api import Tensor


def vjp(fn: Callable, *primals: Any, has_aux: bool = False, create_graph: bool = True):
    tensors = pytree.tensor_leaves(primals)
    prev = [t._impl.is_traced for t in tensors]
    for t in tensors:
        t._impl.is_traced = True
    out = fn(*primals)
    aux = None
    if has_aux:
        out, aux = out
    tr = Trace(primals, out)
    tr.compute()
    for t, p in zip(tensors, prev):
        t._impl.is_traced = p

    def pullback(cotangent):
        for t in tensors:
            t._impl.is_traced = True
        try:
            gmap = backward_on_trace(tr, cotangent, create_graph=create_graph)
        finally:
            for t, p in zip(tensors, prev):
                t._impl.is_traced = p
        from ..ops.creation import zeros_like

        leaves, td = pytree.tree_flatten(primals)
        gl = []
        for l in leaves:
            if isinstance(l, Tensor):
                g = gmap.get(l)
                gl.append(g if g is not None else zeros_like(l))
            else:
                gl.append(None)
        return pytree.tree_unflatten(td, gl)

    return (out, pullback, aux) if has_aux else (out, pullback)
