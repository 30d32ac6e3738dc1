"""Control flow (reference: nabla/ops/control_flow.py:21-507): ``where`` (differentiable),
``cond`` and ``while_loop`` (data-dependent, host-evaluated predicate, not differentiable, as
in the reference), ``scan`` (Python-unrolled, differentiable through its body)."""
from __future__ import annotations

from typing import Any, Callable

import torch

from ..core.common import pytree
from ..core.tensor.api import Tensor, realize_all
from .base import Operation, _align_batch_dims, ensure_tensor


class WhereOp(Operation):
    def kernel(self, c, a, b):
        return torch.where(c.bool(), a, b)

    def partial_passthrough_axes(self, input_specs, kwargs=None):
        # linear in (a, b) jointly: carry an axis only if both branches carry it
        if len(input_specs) < 3:
            return set()
        return set(input_specs[1].partial_sum_axes) & set(input_specs[2].partial_sum_axes) - set(input_specs[0].partial_sum_axes)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .creation import zeros_like

        c, a, b = primals
        z = zeros_like(cot)
        return (None, where(c, cot, z), where(c, z, cot))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        from .creation import zeros_like

        c, a, b = primals
        ta = tangents[1] if tangents[1] is not None else zeros_like(a)
        tb = tangents[2] if tangents[2] is not None else zeros_like(b)
        return where(c, ta, tb)


_where = WhereOp()


def where(condition, x, y) -> Tensor:
    """Elementwise select with three-way numpy broadcasting."""
    if not isinstance(x, Tensor) and not isinstance(y, Tensor):
        x = ensure_tensor(x)
    x = ensure_tensor(x, y if isinstance(y, Tensor) else None)
    y = ensure_tensor(y, x)
    condition = ensure_tensor(condition, None)
    if x.dtype is not y.dtype:
        from .unary import cast

        if x.dtype.is_float() and not y.dtype.is_float():
            y = cast(y, x.dtype)
        elif y.dtype.is_float() and not x.dtype.is_float():
            x = cast(x, y.dtype)
    if condition._impl.batch_dims or x._impl.batch_dims or y._impl.batch_dims:
        condition, x, y = _align_batch_dims([condition, x, y])
    return _where(condition, x, y)


def cond(pred, true_fn: Callable, false_fn: Callable, *operands: Any):
    """Run ``true_fn(*operands)`` or ``false_fn(*operands)`` depending on the scalar ``pred``.

    The predicate is read on the host (one device->host sync), then only the taken branch is
    traced and executed; both branches must produce the same structure of shapes and dtypes.
    """
    if isinstance(pred, Tensor):
        p = bool(pred.item())
    else:
        p = bool(pred)
    return true_fn(*operands) if p else false_fn(*operands)


def while_loop(cond_fn: Callable, body_fn: Callable, init_val: Any):
    """``while cond_fn(*state): state = body_fn(*state)`` with a host-evaluated condition.
    ``init_val`` may be a single value or a tuple; the loop state is realized every iteration
    so the lazy graph does not grow with the trip count."""
    is_tuple = isinstance(init_val, (tuple, list))
    state = tuple(init_val) if is_tuple else (init_val,)
    while True:
        c = cond_fn(*state)
        c = bool(c.item()) if isinstance(c, Tensor) else bool(c)
        if not c:
            break
        new = body_fn(*state)
        state = tuple(new) if isinstance(new, (tuple, list)) else (new,)
        realize_all(*pytree.tensor_leaves(state))
    return (type(init_val)(state) if isinstance(init_val, list) else state) if is_tuple else state[0]


def scan(f: Callable, init: Any, xs: Any, length: int | None = None, reverse: bool = False):
    """``carry, y_t = f(carry, x_t)`` over the leading axis of ``xs`` (unrolled in Python, so it
    is differentiable). Returns ``(final_carry, stacked ys)``."""
    if reverse:
        raise NotImplementedError("scan(reverse=True) is not supported")
    from .view import stack

    leaves = pytree.tensor_leaves(xs)
    n = length if length is not None else (int(leaves[0].shape[0]) if leaves else 0)
    carry = init
    ys = []
    for t in range(n):
        x_t = pytree.tree_map(lambda a: a[t] if isinstance(a, Tensor) else a, xs)
        carry, y = f(carry, x_t)
        ys.append(y)
    if not ys or ys[0] is None:
        return carry, None
    flat0, td = pytree.tree_flatten(ys[0])
    cols = [[pytree.tree_leaves(y)[i] for y in ys] for i in range(len(flat0))]
    stacked = [stack(c, axis=0) for c in cols]
    return carry, pytree.tree_unflatten(td, stacked)
