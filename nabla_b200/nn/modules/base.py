"""``Module`` base class (reference: nabla/nn/modules/base.py:18-337).

A Module is a registered pytree node: its children are parameters, buffers and submodules
(each group in sorted-key order); everything else, including the ``_training`` flag, is
static auxiliary data. So a model can be passed straight through ``grad`` / ``vmap`` /
``compile`` and comes out as a new Module with new leaves (``model = optimizer.step()``).
"""
from __future__ import annotations

from collections import OrderedDict
from contextvars import ContextVar
from typing import Any, ClassVar, Iterator

from ...core.common.pytree import is_tensor, register_pytree_node
from ...core.tensor.api import Tensor, realize_all

_CALL_DEPTH: ContextVar[int] = ContextVar("nabla_module_call_depth", default=0)
_MODULE_CALL_DEPTH = _CALL_DEPTH      # the reference's name (nabla/nn/modules/base.py:15)
_RESERVED = ("_parameters", "_buffers", "_modules", "_training")


def _flatten(m: "Module"):
    pk = tuple(sorted(m._parameters))
    bk = tuple(sorted(m._buffers))
    mk = tuple(sorted(m._modules))
    children = [m._parameters[k] for k in pk] + [m._buffers[k] for k in bk] + [m._modules[k] for k in mk]
    extras = tuple(sorted(((k, v) for k, v in m.__dict__.items()
                           if k not in _RESERVED and k not in m._parameters and k not in m._buffers
                           and k not in m._modules), key=lambda kv: kv[0]))
    return children, (type(m), pk, bk, mk, extras, bool(m._training))


def _unflatten(aux, children) -> "Module":
    cls, pk, bk, mk, extras, training = aux
    obj = object.__new__(cls)
    d = obj.__dict__
    d["_parameters"], d["_buffers"], d["_modules"], d["_training"] = OrderedDict(), OrderedDict(), OrderedDict(), training
    it = iter(children)
    for k in pk:
        v = next(it)
        obj._parameters[k] = v
        d[k] = v
    for k in bk:
        v = next(it)
        obj._buffers[k] = v
        d[k] = v
    for k in mk:
        v = next(it)
        obj._modules[k] = v
        d[k] = v
    for k, v in extras:
        d[k] = v
    return obj


class Module:
    """Base class of all layers. Subclasses implement ``forward``."""

    _AUTO_REALIZE_TOPLEVEL_FORWARD: ClassVar[bool] = False
    _AUTO_REALIZE_BACKWARD_GRADS: ClassVar[bool] = False

    def __init_subclass__(cls, **kwargs: Any) -> None:
        super().__init_subclass__(**kwargs)
        register_pytree_node(cls, _flatten, _unflatten)

    def __init__(self) -> None:
        d = self.__dict__
        d["_parameters"], d["_buffers"], d["_modules"], d["_training"] = OrderedDict(), OrderedDict(), OrderedDict(), True

    # ---- execution policy
    @classmethod
    def set_execution_policy(cls, *, auto_realize_toplevel_forward: bool | None = None,
                             auto_realize_backward_grads: bool | None = None) -> None:
        if auto_realize_toplevel_forward is not None:
            Module._AUTO_REALIZE_TOPLEVEL_FORWARD = bool(auto_realize_toplevel_forward)
        if auto_realize_backward_grads is not None:
            Module._AUTO_REALIZE_BACKWARD_GRADS = bool(auto_realize_backward_grads)

    @classmethod
    def get_execution_policy(cls) -> dict[str, bool]:
        return {"auto_realize_toplevel_forward": Module._AUTO_REALIZE_TOPLEVEL_FORWARD,
                "auto_realize_backward_grads": Module._AUTO_REALIZE_BACKWARD_GRADS}

    # ---- attribute routing
    def __setattr__(self, name: str, value: Any) -> None:
        if "_parameters" not in self.__dict__:
            raise AttributeError("call super().__init__() before assigning attributes to a Module")
        for group in (self._parameters, self._buffers, self._modules):
            group.pop(name, None)
        if isinstance(value, Module):
            self._modules[name] = value
        elif is_tensor(value):
            (self._parameters if value.requires_grad else self._buffers)[name] = value
        self.__dict__[name] = value

    def register_buffer(self, name: str, tensor: Tensor | None) -> None:
        self._parameters.pop(name, None)
        if tensor is not None:
            self._buffers[name] = tensor
        self.__dict__[name] = tensor

    def register_parameter(self, name: str, tensor: Tensor | None) -> None:
        self._buffers.pop(name, None)
        if tensor is not None:
            tensor.requires_grad = True
            self._parameters[name] = tensor
        self.__dict__[name] = tensor

    # ---- calling
    def forward(self, *args: Any, **kwargs: Any) -> Any:
        raise NotImplementedError(f"{type(self).__name__}.forward")

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        depth = _CALL_DEPTH.get()
        tok = _CALL_DEPTH.set(depth + 1)
        try:
            out = self.forward(*args, **kwargs)
        finally:
            _CALL_DEPTH.reset(tok)
        if depth == 0 and Module._AUTO_REALIZE_TOPLEVEL_FORWARD:
            from ...core.common.pytree import tensor_leaves

            realize_all(*tensor_leaves(out))
        return out

    def backward(self, loss: Tensor, gradient: Tensor | None = None, retain_graph: bool = False,
                 create_graph: bool = False, *, realize_grads: bool | None = None) -> None:
        loss.backward(gradient=gradient, retain_graph=retain_graph, create_graph=create_graph)
        do = Module._AUTO_REALIZE_BACKWARD_GRADS if realize_grads is None else bool(realize_grads)
        if do:
            realize_all(*[p.grad for p in self.parameters() if is_tensor(p.grad)])

    # ---- traversal
    def named_parameters(self, prefix: str = "") -> Iterator[tuple[str, Tensor]]:
        for k, v in self._parameters.items():
            yield (f"{prefix}{k}", v)
        for k, m in self._modules.items():
            yield from m.named_parameters(f"{prefix}{k}.")

    def parameters(self) -> Iterator[Tensor]:
        for _, p in self.named_parameters():
            yield p

    def named_buffers(self, prefix: str = "") -> Iterator[tuple[str, Tensor]]:
        for k, v in self._buffers.items():
            yield (f"{prefix}{k}", v)
        for k, m in self._modules.items():
            yield from m.named_buffers(f"{prefix}{k}.")

    def buffers(self) -> Iterator[Tensor]:
        for _, b in self.named_buffers():
            yield b

    def modules(self) -> Iterator["Module"]:
        yield self
        for m in self._modules.values():
            yield from m.modules()

    def children(self) -> Iterator["Module"]:
        yield from self._modules.values()

    def train(self, mode: bool = True) -> "Module":
        for m in self.modules():
            m.__dict__["_training"] = bool(mode)
        return self

    def eval(self) -> "Module":
        return self.train(False)

    @property
    def training(self) -> bool:
        return self._training

    def zero_grad(self) -> None:
        for p in self.parameters():
            p.grad = None

    def state_dict(self) -> "OrderedDict[str, Tensor]":
        out: OrderedDict[str, Tensor] = OrderedDict()
        for k, v in self.named_parameters():
            out[k] = v
        for k, v in self.named_buffers():
            out[k] = v
        return out

    def load_state_dict(self, state_dict, strict: bool = False) -> None:
        """Set the parameters and buffers named in ``state_dict``. As in the reference
        (nabla/nn/modules/base.py:305-311) a partial dict is fine: entries that are not given keep
        their value. ``strict=True`` also wants every own entry to be present and no unknown names."""
        own = self.state_dict()
        if strict:
            missing = [k for k in own if k not in state_dict]
            if missing:
                raise KeyError(f"missing keys in state_dict: {missing}")
        for name, value in state_dict.items():
            if strict and name not in own:
                raise KeyError(f"unexpected key in state_dict: {name}")
            mod: Module = self
            parts = name.split(".")
            for p in parts[:-1]:
                mod = mod._modules[p] if p in mod._modules else getattr(mod, p)
            was_param = parts[-1] in mod._parameters
            if was_param:
                value.requires_grad = True
            setattr(mod, parts[-1], value)

    def extra_repr(self) -> str:
        return ""

    def __repr__(self) -> str:
        lines = [f"{type(self).__name__}({self.extra_repr()}"]
        for k, m in self._modules.items():
            sub = repr(m).replace("\n", "\n  ")
            lines.append(f"  ({k}): {sub}")
        if len(lines) == 1:
            return lines[0] + ")"
        return "\n".join(lines) + "\n)"


register_pytree_node(Module, _flatten, _unflatten)
