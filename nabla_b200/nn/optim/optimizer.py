"""Stateful and functional optimizers (reference: nabla/nn/optim/optimizer.py:35-305).

``optimizer.step(grads=None)`` returns the NEW parameter pytree (for a Module: a new Module)
with detached leaves; the functional pair ``adamw_init`` / ``adamw_update`` carries the state
explicitly. ``adamw_init(params, state_dtype=DType.float32)`` keeps fp32 moments for bf16
parameters (the reference keeps them in the parameter dtype: nn/optim/optimizer.py:104-105).
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, ClassVar

from ...core.common.pytree import is_tensor, tree_flatten, tree_leaves, tree_map, tree_unflatten
from ...core.tensor.api import Tensor, realize_all
from ...types import as_dtype
from .functional import adamw_step, sgd_step

_LEAF = lambda x: x is None or is_tensor(x)  # noqa: E731


def _zeros_state(params: Any, state_dtype=None) -> Any:
    from ...ops.creation import zeros_like
    from ...ops.unary import cast

    def z(p):
        if not is_tensor(p):
            return None
        t = zeros_like(p)
        if state_dtype is not None and as_dtype(state_dtype) is not p.dtype:
            t = cast(t, as_dtype(state_dtype))
        return t

    return tree_map(z, params, is_leaf=_LEAF)


def _detach_like(new_tree: Any, old_tree: Any) -> Any:
    """New leaves become plain leaf tensors (no history) that keep ``requires_grad``."""
    new_l, td = tree_flatten(new_tree, is_leaf=_LEAF)
    old_l = tree_leaves(old_tree, is_leaf=_LEAF)
    out = []
    for n, o in zip(new_l, old_l):
        if is_tensor(n) and is_tensor(o) and n is not o:
            if n._impl.is_realized:
                n._impl.output_refs = None
                n._impl.is_traced = False
            n._impl.requires_grad = o._impl.requires_grad
            if o._impl.requires_grad:
                n._impl.is_traced = True
            n._impl.grad = None
        out.append(n)
    return tree_unflatten(td, out)


class Optimizer(ABC):
    _AUTO_REALIZE_UPDATED_PARAMS: ClassVar[bool] = True
    _AUTO_REALIZE_UPDATED_STATE: ClassVar[bool] = True

    def __init__(self, params: Any) -> None:
        self.params = params

    @classmethod
    def set_execution_policy(cls, *, auto_realize_updated_params: bool | None = None,
                             auto_realize_updated_state: bool | None = None) -> None:
        if auto_realize_updated_params is not None:
            Optimizer._AUTO_REALIZE_UPDATED_PARAMS = bool(auto_realize_updated_params)
        if auto_realize_updated_state is not None:
            Optimizer._AUTO_REALIZE_UPDATED_STATE = bool(auto_realize_updated_state)

    @classmethod
    def get_execution_policy(cls) -> dict[str, bool]:
        return {"auto_realize_updated_params": Optimizer._AUTO_REALIZE_UPDATED_PARAMS,
                "auto_realize_updated_state": Optimizer._AUTO_REALIZE_UPDATED_STATE}

    @abstractmethod
    def step(self, grads: Any = None) -> Any:
        ...

    def _grads_from_params(self) -> Any:
        return tree_map(lambda p: p.grad if is_tensor(p) else None, self.params, is_leaf=_LEAF)

    def zero_grad(self) -> None:
        for p in tree_leaves(self.params):
            if is_tensor(p):
                p.grad = None


class AdamW(Optimizer):
    def __init__(self, params: Any, *, lr: float, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, state_dtype=None) -> None:
        super().__init__(params)
        self.lr, self.beta1, self.beta2 = float(lr), float(betas[0]), float(betas[1])
        self.eps, self.weight_decay = float(eps), float(weight_decay)
        self.step_count = 0
        self.m = _zeros_state(params, state_dtype)
        self.v = _zeros_state(params, state_dtype)

    def step(self, grads: Any = None) -> Any:
        if grads is None:
            grads = self._grads_from_params()
        old = self.params
        self.step_count += 1
        p_l, td = tree_flatten(self.params, is_leaf=_LEAF)
        g_l = tree_leaves(grads, is_leaf=_LEAF)
        m_l = tree_leaves(self.m, is_leaf=_LEAF)
        v_l = tree_leaves(self.v, is_leaf=_LEAF)
        np_, nm, nv = [], [], []
        for p, g, m, v in zip(p_l, g_l, m_l, v_l):
            if is_tensor(p) and is_tensor(g) and is_tensor(m) and is_tensor(v):
                a, b, c = adamw_step(p, g, m, v, self.step_count, lr=self.lr, beta1=self.beta1, beta2=self.beta2,
                                     eps=self.eps, weight_decay=self.weight_decay)
            else:
                a, b, c = p, m, v
            np_.append(a); nm.append(b); nv.append(c)
        self.params, self.m, self.v = tree_unflatten(td, np_), tree_unflatten(td, nm), tree_unflatten(td, nv)
        todo = []
        if self._AUTO_REALIZE_UPDATED_PARAMS:
            todo += [t for t in np_ if is_tensor(t)]
        if self._AUTO_REALIZE_UPDATED_STATE:
            todo += [t for t in nm + nv if is_tensor(t)]
        if todo:
            realize_all(*todo)
        self.params = _detach_like(self.params, old)
        return self.params


class SGD(Optimizer):
    def __init__(self, params: Any, *, lr: float, momentum: float = 0.0, weight_decay: float = 0.0) -> None:
        super().__init__(params)
        self.lr, self.momentum, self.weight_decay = float(lr), float(momentum), float(weight_decay)
        self.step_count = 0
        self.momentum_buffers = _zeros_state(params) if momentum != 0.0 else tree_map(lambda p: None, params, is_leaf=_LEAF)

    def step(self, grads: Any = None) -> Any:
        if grads is None:
            grads = self._grads_from_params()
        old = self.params
        self.step_count += 1
        p_l, td = tree_flatten(self.params, is_leaf=_LEAF)
        g_l = tree_leaves(grads, is_leaf=_LEAF)
        b_l = tree_leaves(self.momentum_buffers, is_leaf=_LEAF)
        np_, nb = [], []
        for p, g, b in zip(p_l, g_l, b_l):
            if is_tensor(p) and is_tensor(g):
                a, c = sgd_step(p, g, b, lr=self.lr, weight_decay=self.weight_decay, momentum=self.momentum)
            else:
                a, c = p, b
            np_.append(a); nb.append(c)
        self.params, self.momentum_buffers = tree_unflatten(td, np_), tree_unflatten(td, nb)
        todo = []
        if self._AUTO_REALIZE_UPDATED_PARAMS:
            todo += [t for t in np_ if is_tensor(t)]
        if self._AUTO_REALIZE_UPDATED_STATE:
            todo += [t for t in nb if is_tensor(t)]
        if todo:
            realize_all(*todo)
        self.params = _detach_like(self.params, old)
        return self.params


def adamw_init(params: Any, state_dtype=None) -> dict[str, Any]:
    return {"m": _zeros_state(params, state_dtype), "v": _zeros_state(params, state_dtype), "step": 0}


def adamw_update(params: Any, grads: Any, state: dict[str, Any], *, lr: float, weight_decay: float = 0.0,
                 beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, bias_correction: bool = True,
                 realize: bool | None = None) -> tuple[Any, dict[str, Any]]:
    prev = state["step"]
    step = prev + 1.0 if is_tensor(prev) else int(prev) + 1
    p_l, td = tree_flatten(params, is_leaf=_LEAF)
    g_l = tree_leaves(grads, is_leaf=_LEAF)
    m_l = tree_leaves(state["m"], is_leaf=_LEAF)
    v_l = tree_leaves(state["v"], is_leaf=_LEAF)
    np_, nm, nv = [], [], []
    for p, g, m, v in zip(p_l, g_l, m_l, v_l):
        if is_tensor(p) and is_tensor(g) and is_tensor(m) and is_tensor(v):
            a, b, c = adamw_step(p, g, m, v, step, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                                 weight_decay=weight_decay, bias_correction=bias_correction)
        else:
            a, b, c = p, m, v
        np_.append(a); nm.append(b); nv.append(c)
    new_params = tree_unflatten(td, np_)
    new_state = {"m": tree_unflatten(td, nm), "v": tree_unflatten(td, nv), "step": step}
    do = Optimizer._AUTO_REALIZE_UPDATED_PARAMS if realize is None else bool(realize)
    if do:
        todo = [t for t in np_ if is_tensor(t)]
        if Optimizer._AUTO_REALIZE_UPDATED_STATE:
            todo += [t for t in nm + nv if is_tensor(t)]
        realize_all(*todo)
    return new_params, new_state
