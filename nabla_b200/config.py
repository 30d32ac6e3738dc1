"""Runtime flags (reference: nabla/config.py:26-109).

ContextVar-backed flags with environment defaults, module-level read access
(``config.TRACING``), setters and scoped context managers:

* ``EAGER_MAX_GRAPH``  - execute every op immediately instead of deferring to ``realize()``
  (name kept from the reference; here it means "eager dispatch").
* ``VERIFY_EAGER_SHAPES`` - cross-check predicted per-shard shapes against produced buffers.
* ``TRACING`` - set while a function is traced for ``compile``; ``realize_all`` is a no-op.
* ``DETERMINISTIC`` - deterministic replay (not in the reference, whose backend has no timing-dependent
  kernels of its own): see ``deterministic``.
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

# deterministic replay: every kernel path whose result or work order depends on timing is swapped
# for one that does not (see `deterministic`)
_DETERMINISTIC = ContextVar("nabla_deterministic", default=_env("NABLA_B200_DETERMINISTIC"))

_FLAGS = {"EAGER_MAX_GRAPH": _EAGER, "VERIFY_EAGER_SHAPES": _VERIFY, "TRACING": _TRACING,
          "DETERMINISTIC": _DETERMINISTIC}


def __getattr__(name: str):
    var = _FLAGS.get(name)
    if var is None:
        raise AttributeError(name)
    return var.get()


def get_flag(name: str) -> bool:
    return _FLAGS[name].get()


def set_eager_max_graph(value: bool) -> None:
    _EAGER.set(bool(value))


def set_verify_eager_shapes(value: bool) -> None:
    _VERIFY.set(bool(value))


def set_tracing(value: bool) -> None:
    _TRACING.set(bool(value))


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


def tracing(value: bool = True):
    return _scoped(_TRACING, value)


def capturable_trace(v: bool = True):
    return _scoped(_CAPTURABLE, v)


def is_capturable_trace() -> bool:
    return _CAPTURABLE.get()


def deterministic(v: bool = True):
    """Scope in which two runs of the same program from the same state give the same bits and walk
    their work in the same order (also switched on for a whole process by ``NABLA_B200_DETERMINISTIC=1``):

    * sums that use atomics (embedding scatter-add) take a sorted, serial-per-row path;
    * the fused GEMM + all-reduce hands its reduce jobs to CTAs in a fixed order instead of
      first-come-first-served, and adds the ranks' partial tiles with peer loads in rank order
      instead of in the switch; the all-reduce / all-gather kernels likewise leave ``multimem`` off;
    * copies and optimizer updates that normally run on side streams stay on the launching stream.

    Timing-dependent bugs (a missing flag wait, a buffer reused too early) then either reproduce on
    every run or never, and `nabla_b200.utils.replay.replay_check` can tell which."""
    return _scoped(_DETERMINISTIC, v)


def set_deterministic(v: bool) -> None:
    _DETERMINISTIC.set(bool(v))


def is_deterministic() -> bool:
    return _DETERMINISTIC.get()


# names the reference uses for the same things (nabla/config.py:26-39, 103-109)
_EAGER_MAX_GRAPH = _EAGER
_VERIFY_EAGER_SHAPES = _VERIFY
tracing_context = tracing


@contextlib.contextmanager
def eager_max_graph_context(value: bool):
    """Set EAGER_MAX_GRAPH inside a ``with`` block (reference: nabla/config.py:83-89)."""
    tok = _EAGER.set(bool(value))
    try:
        yield
    finally:
        _EAGER.reset(tok)


@contextlib.contextmanager
def verify_eager_shapes_context(value: bool):
    """Set VERIFY_EAGER_SHAPES inside a ``with`` block (reference: nabla/config.py:93-99)."""
    tok = _VERIFY.set(bool(value))
    try:
        yield
    finally:
        _VERIFY.reset(tok)

_DEBUG_ON = ("1", "true", "TRUE", "True")


def debug_stream(name: str) -> bool:
    """True when the environment switches the debug print stream ``NABLA_DEBUG_<name>`` on. Read at
    call time, so a test (or a debugging session) can flip it without re-importing anything.
    Streams (names shared with the reference): OP_CALL (every op call with its operands'
    shapes), PHYS (physical-shape decisions of reductions and shape inference), PHYS_VJP
    (operands of reduction VJPs), COT_FLOW / COT_ACCUM (cotangents as the backward sweep creates,
    adds, or fails to add them), NESTED_JVP (tangent attachment in forward mode)."""
    return os.environ.get("NABLA_DEBUG_" + name, "0") in _DEBUG_ON
