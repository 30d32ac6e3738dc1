"""Pure optimizer steps (reference: nabla/nn/optim/functional.py:14-162).

``adamw_step`` / ``sgd_step`` work on single tensors. On GPU (or with ``NABLA_B200_FUSED=1``)
they are ONE fused kernel per tensor instead of ~15 primitive ops; the mixed-precision form
the benchmarks use (bf16 parameters, fp32 moments: ``state_dtype=float32`` in ``adamw_init``)
is handled by the same kernel. The primitive composition stays as the reference path.
"""
from __future__ import annotations

import math
from typing import Any

from ...core.common.pytree import is_tensor, tree_leaves, tree_map
from ...core.tensor.api import Tensor, realize_all
from ...ops import fused
from ...ops.unary import cast, exp, sqrt


def _fused_ok(p: Tensor, *others) -> bool:
    from ..functional.layers import use_fused

    return use_fused(p) and all(o is None or is_tensor(o) for o in others)


def sgd_step(param: Tensor, grad: Tensor, momentum_buffer: Tensor | None = None, *, lr: float,
             weight_decay: float = 0.0, momentum: float = 0.0) -> tuple[Tensor, Tensor | None]:
    if _fused_ok(param) and (momentum == 0.0 or momentum_buffer is not None):
        if momentum != 0.0:
            p, b = fused.sgd_step_fused(param, grad, momentum_buffer, lr=lr, momentum=momentum, weight_decay=weight_decay)
            return p, b
        return fused.sgd_step_fused(param, grad, None, lr=lr, weight_decay=weight_decay), momentum_buffer
    update = grad
    if weight_decay != 0.0:
        update = update + param * weight_decay
    if momentum != 0.0:
        momentum_buffer = update if momentum_buffer is None else momentum * momentum_buffer + update
        update = momentum_buffer
    return param - update * lr, momentum_buffer


def adamw_step(param: Tensor, grad: Tensor, m: Tensor, v: Tensor, step, *, lr: float, beta1: float = 0.9,
               beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0, bias_correction: bool = True
               ) -> tuple[Tensor, Tensor, Tensor]:
    """Single-tensor AdamW update; ``step`` is a python number or a 0-d tensor."""
    if _fused_ok(param):
        return tuple(fused.adamw_step_fused(param, grad, m, v, step, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                                            weight_decay=weight_decay, bias_correction=bias_correction))
    g = grad if grad.dtype is m.dtype else cast(grad, m.dtype)
    m_t = m * beta1 + g * (1.0 - beta1)
    v_t = v * beta2 + (g * g) * (1.0 - beta2)
    if bias_correction:
        if is_tensor(step):
            bc1 = 1.0 - exp(step * math.log(beta1))
            bc2 = 1.0 - exp(step * math.log(beta2))
        else:
            bc1 = 1.0 - beta1 ** step
            bc2 = 1.0 - beta2 ** step
    else:
        bc1 = bc2 = 1.0
    update = (m_t / bc1) / (sqrt(v_t / bc2) + eps)
    p32 = param if param.dtype is m.dtype else cast(param, m.dtype)
    if weight_decay != 0.0:
        update = update + p32 * weight_decay
    new_p = p32 - update * lr
    if new_p.dtype is not param.dtype:
        new_p = cast(new_p, param.dtype)
    return new_p, m_t, v_t


def sgd_update(params: Any, grads: Any, state: dict[str, Any] | None = None, *, lr: float, momentum: float = 0.0,
               weight_decay: float = 0.0) -> tuple[Any, dict[str, Any]]:
    from ...ops.creation import zeros_like

    if state is None:
        bufs = tree_map(lambda p: zeros_like(p) if (is_tensor(p) and momentum != 0.0) else None, params,
                        is_leaf=lambda x: x is None or is_tensor(x))
        state = {"momentum_buffers": bufs, "step": 0}
    step = int(state["step"]) + 1
    leaf = lambda x: x is None or is_tensor(x)  # noqa: E731
    from ...core.common.pytree import tree_flatten, tree_unflatten

    p_leaves, td = tree_flatten(params, is_leaf=leaf)
    g_leaves = tree_leaves(grads, is_leaf=leaf)
    b_leaves = tree_leaves(state["momentum_buffers"], is_leaf=leaf)
    if len(b_leaves) != len(p_leaves):
        b_leaves = [None] * len(p_leaves)
    new_p, new_b = [], []
    for p, g, b in zip(p_leaves, g_leaves, b_leaves):
        if is_tensor(p) and is_tensor(g):
            np_, nb_ = sgd_step(p, g, b, lr=lr, weight_decay=weight_decay, momentum=momentum)
        else:
            np_, nb_ = p, b
        new_p.append(np_)
        new_b.append(nb_)
    new_params = tree_unflatten(td, new_p)
    new_state = {"momentum_buffers": tree_unflatten(td, new_b), "step": step}
    from .optimizer import Optimizer

    if Optimizer._AUTO_REALIZE_UPDATED_PARAMS:
        realize_all(*[t for t in new_p if is_tensor(t)])
    return new_params, new_state
