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
    """One-hot basis of a tensor: shape ``(numel, *x.shape)``. Given a LIST of tensors it follows the
    reference's convention (nabla/transforms/utils.py:130-156): ``(sizes, basis)`` where the basis of
    every tensor spans the joint index space of all of them, shape ``(total, *t.shape)``."""
    import numpy as np

    from ..ops.creation import constant

    if isinstance(x, (list, tuple)):
        sizes = []
        for t in x:
            n = 1
            for d in t.shape:
                n *= int(d)
            sizes.append(max(n, 1))
        total, offset, basis = sum(sizes), 0, []
        for t, n in zip(x, sizes):
            sh = tuple(int(d) for d in t.shape)
            bp = np.zeros((total, n), dtype=np.float32)
            bp[np.arange(offset, offset + n), np.arange(n)] = 1.0
            basis.append(constant(bp.reshape((total,) + sh), dtype=t.dtype, device=t.device))
            offset += n
        return sizes, basis

    shape = tuple(x._impl.global_shape)
    n = 1
    for d in shape:
        n *= d
    eye = np.eye(n, dtype=np.float32).reshape((n,) + shape)
    return constant(eye, dtype=x.dtype, device=x.device)


def lift_basis_to_batch_prefix(basis: list, references: list) -> list:
    """Give Jacobian basis tensors the batch prefix of their reference tensors, which is what
    ``vmap(jacrev(f))`` / ``vmap(jacfwd(f))`` need when an outer ``vmap`` is already active
    (reference: nabla/transforms/utils.py:159-192). A basis that already carries the prefix is left alone."""
    from ..ops.view.batch import broadcast_batch_dims

    if len(basis) != len(references):
        raise ValueError(f"basis/reference length mismatch: {len(basis)} != {len(references)}")
    lifted = []
    for b, ref in zip(basis, references):
        if ref.batch_dims <= 0 or b.batch_dims >= ref.batch_dims:
            lifted.append(b)
            continue
        prefix = tuple(int(d) for d in ref._impl.physical_global_shape[: ref.batch_dims])
        lifted.append(broadcast_batch_dims(b, prefix))
    return lifted
