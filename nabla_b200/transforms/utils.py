"""Helpers shared by the transforms (reference: nabla/transforms/utils.py:70-192)."""
from __future__ import annotations

from typing import Any

from ..core.common import pytree


def select_argnums(grads_struct: tuple, argnums):
    """A single entry for an int ``argnums``, a tuple for a tuple."""
    if isinstance(argnums, int):
        return grads_struct[argnums]
    return tuple(grads_struct[i] for i in argnums)


def zeros_for_missing(arg, grad):
    """Replace ``None`` gradients by zeros shaped like the corresponding inputs."""
    from ..ops.creation import zeros_like

    def f(a, g):
        if g is None and pytree.is_tensor(a):
            return zeros_like(a)
        return g

    leaves_a, td = pytree.tree_flatten(arg)
    leaves_g = pytree.tree_leaves(grad, is_leaf=lambda x: x is None or pytree.is_tensor(x))
    if len(leaves_a) != len(leaves_g):
        return grad
    return pytree.tree_unflatten(td, [f(a, g) for a, g in zip(leaves_a, leaves_g)])


def std_basis(x):
    """One-hot basis of a tensor: shape ``(numel, *x.shape)``."""
    import numpy as np

    from ..ops.creation import constant

    shape = tuple(x._impl.global_shape)
    n = 1
    for d in shape:
        n *= d
    eye = np.eye(n, dtype=np.float32).reshape((n,) + shape)
    return constant(eye, dtype=x.dtype, device=x.device)
