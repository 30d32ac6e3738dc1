"""Default device / dtype context (reference: nabla/core/common/context.py:29-139).

The default dtype is float32. The default device is the CPU unless the environment variable
``NABLA_DEFAULT_DEVICE`` is ``gpu`` (or ``cuda``) and a CUDA device is present. The reference's
global MAX ``InferenceSession`` has no counterpart: execution goes through
``nabla_b200.core.graph.engine``.
"""
from __future__ import annotations

import contextlib
import os
from contextvars import ContextVar

import torch

from ...types import CPU, Accelerator, Device, DType, as_device, as_dtype

_DEVICE: ContextVar[Device | None] = ContextVar("nabla_default_device", default=None)
_DTYPE: ContextVar[DType | None] = ContextVar("nabla_default_dtype", default=None)


def _initial_device() -> Device:
    want = os.environ.get("NABLA_DEFAULT_DEVICE", "cpu").strip().lower()
    if want in ("gpu", "cuda", "accelerator") and torch.cuda.is_available():
        return Accelerator(int(os.environ.get("LOCAL_RANK", torch.cuda.current_device())))
    return CPU()


def get_default_device() -> Device:
    d = _DEVICE.get()
    if d is None:
        d = _initial_device()
        _DEVICE.set(d)
    return d


def get_default_dtype() -> DType:
    return _DTYPE.get() or DType.float32


def defaults(dtype=None, device=None) -> tuple[DType, Device]:
    """Resolve ``(dtype, device)`` filling unspecified entries with the current defaults."""
    return (as_dtype(dtype) if dtype is not None else get_default_dtype(),
            as_device(device) if device is not None else get_default_device())


@contextlib.contextmanager
def default_device(device):
    tok = _DEVICE.set(as_device(device))
    try:
        yield
    finally:
        _DEVICE.reset(tok)


@contextlib.contextmanager
def default_dtype(dtype):
    tok = _DTYPE.set(as_dtype(dtype))
    try:
        yield
    finally:
        _DTYPE.reset(tok)


@contextlib.contextmanager
def defaults_like(like):
    """Use the dtype and device of ``like`` (a Tensor) as defaults inside the block."""
    with default_dtype(like.dtype), default_device(like.device):
        yield


def set_default_device(device) -> None:
    _DEVICE.set(as_device(device))


def _in_running_loop() -> bool:
    """True inside a running asyncio event loop (reference: nabla/core/common/context.py:142-148)."""
    import asyncio

    try:
        asyncio.get_running_loop()
    except RuntimeError:
        return False
    return True


@contextlib.contextmanager
def contextvar_context(var: ContextVar, value):
    """Set any ContextVar inside a ``with`` block (reference: nabla/core/common/context.py:37-42)."""
    tok = var.set(value)
    try:
        yield
    finally:
        var.reset(tok)
