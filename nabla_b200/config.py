"""Runtime flags (reference: nabla/config.py:26-109).

Three ContextVar-backed flags with environment defaults, module-level read access
(``config.TRACING``), setters and scoped context managers:

* ``EAGER_MAX_GRAPH``  - execute every op immediately instead of deferring to ``realize()``
  (name kept from the reference; here it means "eager dispatch").
* ``VERIFY_EAGER_SHAPES`` - cross-check predicted per-shard shapes against produced buffers.
* ``TRACING`` - set while a function is traced for ``compile``; ``realize_all`` is a no-op.
"""
from __future__ import annotations

import contextlib
import os
from contextvars import ContextVar


def _env(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default).strip().lower() in ("1", "true", "yes", "on")


_EAGER = ContextVar("nabla_eager_max_graph", default=_env("EAGER_MAX_GRAPH") or _env("NABLA_EAGER_MAX_GRAPH"))
_VERIFY = ContextVar("nabla_verify_eager_shapes",
                     default=_env("VERIFY_EAGER_SHAPES") or _env("NABLA_VERIFY_EAGER_SHAPES"))
_TRACING = ContextVar("nabla_tracing", default=False)
# set by compile(cuda_graph=True) while it traces: ops that would need a host decision at replay
# (cond) pick a lowering that stays on the device
_CAPTURABLE = ContextVar("nabla_capturable_trace", default=False)

_FLAGS = {"EAGER_MAX_GRAPH": _EAGER, "VERIFY_EAGER_SHAPES": _VERIFY, "TRACING": _TRACING}


def __getattr__(name: str):
    var = _FLAGS.get(name)
    if var is None:
        raise AttributeError(name)
    return var.get()


def get_flag(name: str) -> bool:
    return _FLAGS[name].get()


def set_eager_max_graph(v: bool) -> None:
    _EAGER.set(bool(v))


def set_verify_eager_shapes(v: bool) -> None:
    _VERIFY.set(bool(v))


def set_tracing(v: bool) -> None:
    _TRACING.set(bool(v))


@contextlib.contextmanager
def _scoped(var: ContextVar, v: bool):
    tok = var.set(bool(v))
    try:
        yield
    finally:
        var.reset(tok)


def eager_max_graph(v: bool = True):
    return _scoped(_EAGER, v)


def verify_eager_shapes(v: bool = True):
    return _scoped(_VERIFY, v)


def tracing(v: bool = True):
    return _scoped(_TRACING, v)


def capturable_trace(v: bool = True):
    return _scoped(_CAPTURABLE, v)


def is_capturable_trace() -> bool:
    return _CAPTURABLE.get()


_DEBUG_ON = ("1", "true", "TRUE", "True")


def debug_stream(name: str) -> bool:
    """True when the environment switches the debug print stream ``NABLA_DEBUG_<name>`` on. Read at
    call time, so a test (or a debugging session) can flip it without re-importing anything.
    Streams (names shared with the reference): OP_CALL (every op call with its operands'
    shapes), PHYS (physical-shape decisions of reductions and shape inference), PHYS_VJP
    (operands of reduction VJPs), COT_FLOW / COT_ACCUM (cotangents as the backward sweep creates,
    adds, or fails to add them), NESTED_JVP (tangent attachment in forward mode)."""
    return os.environ.get("NABLA_DEBUG_" + name, "0") in _DEBUG_ON
