"""``jvp`` (reference: nabla/transforms/jvp.py:46-121): forward-mode by replaying the trace
in order with ``op.jvp_rule``. Returns ``(out, tangent_out[, aux])``."""
from __future__ import annotations

from typing import Any, Callable

from ..core.autograd.forward import forward_on_trace
from ..core.common import pytree
from ..core.graph.tracing import Trace
from ..core.tensor.api import Tensor


def jvp(fn: Callable, primals, tangents, has_aux: bool = False, create_graph: bool = True):
    if not isinstance(primals, (tuple, list)):
        primals, tangents = (primals,), (tangents,)
    primals, tangents = tuple(primals), tuple(tangents)
    if len(primals) != len(tangents):
        raise ValueError("primals and tangents must have the same length")
    tensors = pytree.tensor_leaves(primals)
    prev = [t._impl.is_traced for t in tensors]
    for t in tensors:
        t._impl.is_traced = True
    try:
        out = fn(*primals)
        aux = None
        if has_aux:
            out, aux = out
        tr = Trace(primals, out)
        tr.compute()
        tan_leaves = pytree.tree_leaves(tangents, is_leaf=lambda x: x is None or isinstance(x, Tensor))
        tan_leaves = [t for t, p in zip(tan_leaves, pytree.tree_leaves(
            primals, is_leaf=lambda x: x is None or isinstance(x, Tensor))) if isinstance(p, Tensor)]
        outs_t = forward_on_trace(tr, tan_leaves, create_graph=create_graph)
    finally:
        for t, p in zip(tensors, prev):
            t._impl.is_traced = p
    from ..ops.creation import zeros_like

    out_leaves, td = pytree.tree_flatten(out)
    it = iter(outs_t)
    res = []
    for o in out_leaves:
        if isinstance(o, Tensor):
            t = next(it)
            res.append(t if t is not None else zeros_like(o))
        else:
            res.append(None)
    tan_out = pytree.tree_unflatten(td, res)
    return (out, tan_out, aux) if has_aux else (out, tan_out)


def _clear_jvp_cache() -> None:
    """Kept for API compatibility; this implementation holds no JVP cache."""
