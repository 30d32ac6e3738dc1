"""JAX-style pytrees (reference: nabla/core/common/pytree.py:35-413).

Containers: list, tuple, dict (keys flattened in **sorted** order), ``None`` (a structural
node with no leaves) and classes registered with ``register_pytree_node``. Everything else is
a leaf. ``PyTreeDef`` is immutable, hashable and comparable so it can key caches.
"""
from __future__ import annotations

from typing import Any, Callable

_registry: dict[type, tuple[Callable, Callable]] = {}


def register_pytree_node(cls: type, flatten_fn: Callable, unflatten_fn: Callable) -> None:
    """Register ``cls`` as a container: ``flatten_fn(obj) -> (children, aux)``,
    ``unflatten_fn(aux, children) -> obj``."""
    if not isinstance(cls, type):
        raise TypeError("cls must be a type")
    _registry[cls] = (flatten_fn, unflatten_fn)


def _freeze(v: Any) -> Any:
    if isinstance(v, (str, bytes, int, float, bool, type(None))):
        return v
    if isinstance(v, (tuple, list)):
        return tuple(_freeze(x) for x in v)
    if isinstance(v, dict):
        return tuple(sorted(((_freeze(k), _freeze(x)) for k, x in v.items()), key=repr))
    if isinstance(v, (set, frozenset)):
        return frozenset(_freeze(x) for x in v)
    try:
        hash(v)
        return v
    except TypeError:
        return (type(v).__qualname__, repr(v))


class PyTreeDef:
    """Structure of a pytree: node kind, node metadata and child structures."""

    __slots__ = ("kind", "meta", "children", "num_leaves", "_hash")

    def __init__(self, kind: str, meta: Any, children: tuple["PyTreeDef", ...], num_leaves: int):
        self.kind = kind
        self.meta = meta
        self.children = children
        self.num_leaves = num_leaves
        self._hash = None

    def __repr__(self) -> str:
        k = self.kind
        if k == "leaf":
            return "*"
        if k == "none":
            return "None"
        if k == "dict":
            return f"dict{list(self.meta)}"
        if k == "custom":
            return f"custom[{self.meta[0].__name__}]"
        return f"{k}[{len(self.children)}]"

    def __eq__(self, o: Any) -> bool:
        if self is o:
            return True
        if not (isinstance(o, PyTreeDef) and self.kind == o.kind and self.num_leaves == o.num_leaves):
            return False
        if self._hash is not None and o._hash is not None and self._hash != o._hash:
            return False
        try:
            same_meta = bool(self.meta == o.meta)        # plain comparison first (lists of keys, None, ints)
        except Exception:
            same_meta = False
        return (same_meta or _freeze(self.meta) == _freeze(o.meta)) and self.children == o.children

    def __hash__(self) -> int:
        if self._hash is None:
            self._hash = hash((self.kind, _freeze(self.meta), self.children))
        return self._hash

    def unflatten(self, leaves) -> Any:
        return tree_unflatten(self, leaves)


_LEAF = PyTreeDef("leaf", None, (), 1)
_NONE = PyTreeDef("none", None, (), 0)


def _flatten(tree: Any, leaves: list, is_leaf) -> PyTreeDef:
    if is_leaf is not None and is_leaf(tree):
        leaves.append(tree)
        return _LEAF
    if tree is None:
        return _NONE
    t = type(tree)
    if t is list or t is tuple:
        ch = tuple(_flatten(x, leaves, is_leaf) for x in tree)
        return PyTreeDef("list" if t is list else "tuple", None, ch, sum(c.num_leaves for c in ch))
    if t is dict:
        keys = sorted(tree.keys(), key=lambda k: (str(type(k)), k) if not isinstance(k, str) else ("", k))
        ch = tuple(_flatten(tree[k], leaves, is_leaf) for k in keys)
        return PyTreeDef("dict", tuple(keys), ch, sum(c.num_leaves for c in ch))
    reg = _registry.get(t)
    if reg is None:
        for cls, r in _registry.items():
            if isinstance(tree, cls):
                reg = r
                break
    if reg is not None:
        children, aux = reg[0](tree)
        ch = tuple(_flatten(x, leaves, is_leaf) for x in children)
        return PyTreeDef("custom", (t, aux), ch, sum(c.num_leaves for c in ch))
    if isinstance(tree, tuple) and hasattr(tree, "_fields"):  # namedtuple
        ch = tuple(_flatten(x, leaves, is_leaf) for x in tree)
        return PyTreeDef("custom", (t, "namedtuple"), ch, sum(c.num_leaves for c in ch))
    leaves.append(tree)
    return _LEAF


def tree_flatten(tree: Any, is_leaf: Callable[[Any], bool] | None = None) -> tuple[list, PyTreeDef]:
    leaves: list = []
    td = _flatten(tree, leaves, is_leaf)
    return leaves, td


def _unflatten(td: PyTreeDef, it) -> Any:
    k = td.kind
    if k == "leaf":
        return next(it)
    if k == "none":
        return None
    if k == "list":
        return [_unflatten(c, it) for c in td.children]
    if k == "tuple":
        return tuple(_unflatten(c, it) for c in td.children)
    if k == "dict":
        return {key: _unflatten(c, it) for key, c in zip(td.meta, td.children)}
    cls, aux = td.meta
    children = [_unflatten(c, it) for c in td.children]
    if aux == "namedtuple" and hasattr(cls, "_fields"):
        return cls(*children)
    reg = _registry.get(cls)
    if reg is None:
        for c2, r in _registry.items():
            if issubclass(cls, c2):
                reg = r
                break
    return reg[1](aux, children)


def tree_unflatten(treedef: PyTreeDef, leaves) -> Any:
    leaves = list(leaves)
    if len(leaves) != treedef.num_leaves:
        raise ValueError(f"expected {treedef.num_leaves} leaves, got {len(leaves)}")
    return _unflatten(treedef, iter(leaves))


def tree_leaves(tree: Any, is_leaf=None) -> list:
    return tree_flatten(tree, is_leaf)[0]


def leaf_names(treedef: PyTreeDef, prefix: str = "") -> list[str]:
    """One path string per leaf of ``treedef``, in flatten order: dict entries as ``.key``, items of
    lists / tuples / registered containers as ``[i]`` (e.g. ``layers[2].attn.q``). With a prefix the
    first dict key is joined with a dot (``lora.w``)."""
    out: list[str] = []

    def walk(td: PyTreeDef, path: str) -> None:
        if td.kind == "leaf":
            out.append(path)
        elif td.kind == "none":
            return
        elif td.kind == "dict":
            for k, c in zip(td.meta, td.children):
                walk(c, f"{path}.{k}" if path else str(k))
        else:
            for i, c in enumerate(td.children):
                walk(c, f"{path}[{i}]")

    walk(treedef, prefix)
    return out


def tree_flatten_with_names(tree: Any, is_leaf=None) -> tuple[list, list[str], PyTreeDef]:
    """``tree_flatten`` plus the path name of every leaf: ``(leaves, names, treedef)``."""
    leaves, td = tree_flatten(tree, is_leaf)
    return leaves, leaf_names(td), td


def tree_flatten_full(tree: Any, is_leaf=None) -> tuple[list, PyTreeDef]:
    """``tree_flatten`` that keeps ``None`` as a leaf instead of a structural node
    (reference: nabla/core/common/pytree.py:227-236)."""
    return tree_flatten(tree, is_leaf=lambda x: x is None or (is_leaf(x) if is_leaf else False))


def tree_structure(tree: Any, is_leaf=None) -> PyTreeDef:
    return tree_flatten(tree, is_leaf)[1]


def tree_map(fn: Callable, tree: Any, *rest: Any, is_leaf=None) -> Any:
    """Map ``fn`` over the leaves of ``tree`` (and matching leaves of ``rest``)."""
    leaves, td = tree_flatten(tree, is_leaf)
    if not rest:
        return tree_unflatten(td, [fn(x) for x in leaves])
    others = []
    for r in rest:
        # flatten `r` up to the structure of `tree`: its leaves may be subtrees of r
        others.append(_flatten_up_to(td, r))
    return tree_unflatten(td, [fn(x, *ys) for x, *ys in zip(leaves, *others)])


def _flatten_up_to(td: PyTreeDef, tree: Any) -> list:
    out: list = []

    def rec(d: PyTreeDef, t: Any):
        k = d.kind
        if k == "leaf":
            out.append(t)
        elif k == "none":
            if t is not None:
                raise ValueError("tree structure mismatch: expected None")
        elif k in ("list", "tuple"):
            if not isinstance(t, (list, tuple)) or len(t) != len(d.children):
                raise ValueError(f"tree structure mismatch at {d}: got {type(t).__name__}")
            for c, x in zip(d.children, t):
                rec(c, x)
        elif k == "dict":
            if not isinstance(t, dict) or set(t.keys()) != set(d.meta):
                raise ValueError("tree structure mismatch: dict keys differ")
            for key, c in zip(d.meta, d.children):
                rec(c, t[key])
        else:
            cls, aux = d.meta
            if aux == "namedtuple":
                children = list(t)
            else:
                reg = _registry.get(type(t)) or _registry.get(cls)
                children, _ = reg[0](t)
            if len(children) != len(d.children):
                raise ValueError("tree structure mismatch in custom node")
            for c, x in zip(d.children, children):
                rec(c, x)

    rec(td, tree)
    return out


# ---------------------------------------------------------------- tensor helpers
def is_tensor(obj: Any) -> bool:
    from ..tensor.api import Tensor

    return isinstance(obj, Tensor)


def tensor_leaves(tree: Any) -> list:
    return [x for x in tree_leaves(tree) if is_tensor(x)]


def _set_traced(tree: Any, flag: bool) -> Any:
    for t in tensor_leaves(tree):
        t._impl.is_traced = flag
    return tree


def traced(tree: Any) -> Any:
    """Mark every tensor leaf as traced (its producing ops are kept for autodiff)."""
    return _set_traced(tree, True)


def untraced(tree: Any) -> Any:
    return _set_traced(tree, False)


def with_batch_dims(tree: Any, delta: int) -> Any:
    """Return a tree whose tensor leaves have ``batch_dims`` shifted by ``delta``."""
    from ...ops.view.batch import decr_batch_dims, incr_batch_dims

    def f(x):
        if not is_tensor(x):
            return x
        for _ in range(abs(delta)):
            x = incr_batch_dims(x) if delta > 0 else decr_batch_dims(x)
        return x

    return tree_map(f, tree)


def tree_unflatten_full(treedef: PyTreeDef, leaves: list) -> Any:
    """Inverse of a flatten that kept ``None`` leaves (reference: nabla/core/common/pytree.py:239-241)."""
    return tree_unflatten(treedef, leaves)


def is_tensor_value(obj: Any) -> bool:
    """Is ``obj`` a value of the execution backend (reference: pytree.py:416, a MAX graph value)?
    Here that is a device buffer."""
    import torch

    return isinstance(obj, torch.Tensor)
