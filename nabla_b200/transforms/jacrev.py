"""``jacrev``: Jacobian by reverse mode (reference: nabla/transforms/jacrev.py:78-196).
One pullback per output element (a loop over the one-hot basis of the output), rows stacked
and reshaped to ``(*out_shape, *in_shape)``. Single-output functions only, as in the
reference. Nesting (``jacrev(jacrev(f))``, ``jacfwd(grad(f))``) gives Hessians."""
from __future__ import annotations

from typing import Any, Callable

from ..core.common import pytree
from ..core.tensor.api import Tensor
from .utils import std_basis
from .vjp import vjp


def jacrev(fn: Callable, argnums: int | tuple[int, ...] | list[int] | None = None, has_aux: bool = False) -> Callable:
    def wrapper(*args: Any):
        from ..ops.view import reshape, stack

        # argnums=None (the default) differentiates with respect to every argument; the result is a
        # single Jacobian for one differentiated argument given as None / int, a tuple otherwise
        # (reference: nabla/transforms/utils.py:52-67, jacrev.py:118-160)
        if argnums is None:
            argn = tuple(range(len(args)))
        elif isinstance(argnums, int):
            argn = (argnums,)
        else:
            argn = tuple(argnums)
        argn = tuple(a if a >= 0 else len(args) + a for a in argn)
        for a in argn:
            if not 0 <= a < len(args):
                raise ValueError(f"argnum {a} out of bounds for {len(args)} arguments")
        single = isinstance(argnums, int) or (argnums is None and len(argn) == 1)

        def partial(*diff):
            full = list(args)
            for i, d in zip(argn, diff):
                full[i] = d
            return fn(*full)

        diff_args = tuple(args[i] for i in argn)
        res = vjp(partial, *diff_args, has_aux=has_aux)
        out, pullback = res[0], res[1]
        if not isinstance(out, Tensor):
            raise TypeError("jacrev supports functions with a single Tensor output")
        out_shape = tuple(out._impl.global_shape)
        basis = std_basis(out)
        n = int(basis.shape[0])
        rows = [pullback(basis[i]) for i in range(n)]
        jacs = []
        for k, a in enumerate(diff_args):
            leaves_a, td = pytree.tree_flatten(a)
            per_leaf = []
            for li, leaf in enumerate(leaves_a):
                if not isinstance(leaf, Tensor):
                    per_leaf.append(None)
                    continue
                col = [pytree.tree_leaves(r[k], is_leaf=lambda x: x is None or isinstance(x, Tensor))[li] for r in rows]
                j = stack(col, axis=0)
                per_leaf.append(reshape(j, out_shape + tuple(leaf._impl.global_shape)))
            jacs.append(pytree.tree_unflatten(td, per_leaf))
        jac = jacs[0] if single else tuple(jacs)
        return (jac, res[2]) if has_aux else jac

    wrapper.__name__ = f"jacrev({getattr(fn, '__name__', 'fn')})"
    return wrapper
