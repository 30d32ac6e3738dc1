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


def std_basis(flat_tensors):
    """One-hot basis of a tensor: shape ``(numel, *x.shape)``. Given a LIST of tensors it follows the
    reference's convention (nabla/transforms/utils.py:130-156): ``(sizes, basis)`` where the basis of
    every tensor spans the joint index space of all of them, shape ``(total, *t.shape)``."""
    import numpy as np

    from ..ops.creation import constant

    x = flat_tensors
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


# ---- small helpers shared by the transforms (reference: nabla/transforms/utils.py:40-127)
def split_aux(raw: Any, has_aux: bool, name: str) -> tuple[Any, Any]:
    """``(output, aux)`` of a function called with ``has_aux``; ``(raw, None)`` without it."""
    if not has_aux:
        return raw, None
    if not isinstance(raw, tuple) or len(raw) != 2:
        raise ValueError(f"{name} with has_aux=True expects fn to return (output, aux), got {type(raw)}")
    return raw[0], raw[1]


def resolve_argnums(argnums, n_args: int) -> tuple[int, ...]:
    """``argnums`` (None = all, int, or sequence; negatives count from the end) as a tuple of valid
    positions."""
    sel = tuple(range(n_args)) if argnums is None else ((argnums,) if isinstance(argnums, int) else tuple(argnums))
    out = tuple(a + n_args if a < 0 else a for a in sel)
    for a in out:
        if not 0 <= a < n_args:
            raise ValueError(f"argnum {a} out of bounds for {n_args} arguments")
    return out


def collect_grads(grads_map: dict, input_leaves: list, *, skip_non_diff: bool = True) -> list:
    """Per-leaf gradients out of a ``{input tensor: gradient}`` map: ``None`` for leaves that are
    not tensors (or not floating point, with ``skip_non_diff``), zeros for tensors the output does
    not depend on."""
    from ..core.tensor.api import Tensor
    from ..ops.creation import zeros_like

    out = []
    for leaf in input_leaves:
        if not isinstance(leaf, Tensor) or (skip_non_diff and not leaf.dtype.is_float()):
            out.append(None)
        elif leaf in grads_map:
            out.append(grads_map[leaf])
        else:
            out.append(zeros_like(leaf))
    return out


def realize_tensors(tensors: list) -> None:
    """Realize the lazy tensors of ``tensors`` in one evaluation."""
    from ..core.tensor.api import Tensor, realize_all

    lazy = [t for t in tensors if isinstance(t, Tensor) and not t.is_realized]
    if lazy:
        realize_all(*lazy)


def create_jacobian_helpers(fn, argnums, args: tuple):
    """``(differentiated args, fn with the other args fixed)`` for jacrev / jacfwd."""
    norm = resolve_argnums(argnums, len(args))

    def partial_fn(*diff):
        full = list(args)
        for i, a in zip(norm, diff):
            full[i] = a
        return fn(*full)

    return tuple(args[i] for i in norm), partial_fn
