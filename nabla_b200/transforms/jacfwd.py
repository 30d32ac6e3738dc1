"""``jacfwd``: Jacobian by forward mode (reference: nabla/transforms/jacfwd.py:79-216).
One JVP per input element (loop over the one-hot basis of the input), columns stacked on the
last axes: result shape ``(*out_shape, *in_shape)``."""
from __future__ import annotations

from typing import Any, Callable

from ..core.tensor.api import Tensor
from .jvp import jvp
from .utils import std_basis


def jacfwd(fn: Callable, argnums: int | tuple[int, ...] | list[int] | None = None, has_aux: bool = False) -> Callable:
    def wrapper(*args: Any):
        from ..ops.creation import zeros_like
        from ..ops.view import moveaxis, reshape, stack

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
        jacs = []
        aux = None
        for which in argn:
            x = args[which]
            if not isinstance(x, Tensor):
                raise TypeError("jacfwd differentiates with respect to Tensor arguments")

            def partial(xx, _w=which):
                full = list(args)
                full[_w] = xx
                return fn(*full)

            basis = std_basis(x)
            n = int(basis.shape[0])
            cols = []
            out_shape = None
            for i in range(n):
                r = jvp(partial, (x,), (basis[i],), has_aux=has_aux)
                out, t = r[0], r[1]
                if has_aux:
                    aux = r[2]
                if not isinstance(out, Tensor):
                    raise TypeError("jacfwd supports functions with a single Tensor output")
                out_shape = tuple(out._impl.global_shape)
                cols.append(t)
            j = stack(cols, axis=0)                     # (n, *out)
            j = moveaxis(j, 0, -1) if len(out_shape) else j   # (*out, n)
            jacs.append(reshape(j, out_shape + tuple(x._impl.global_shape)))
        jac = jacs[0] if single else tuple(jacs)
        return (jac, aux) if has_aux else jac

    wrapper.__name__ = f"jacfwd({getattr(fn, '__name__', 'fn')})"
    return wrapper
