"""Initializers (reference: nabla/nn/functional/init.py:14-40)."""
from __future__ import annotations

from ...ops.creation import gaussian
from ...types import DType


def xavier_normal(shape, *, dtype=DType.float32, device=None):
    if len(shape) < 2:
        raise ValueError("xavier_normal expects shape with at least 2 dims")
    std = (2.0 / float(int(shape[0]) + int(shape[1]))) ** 0.5
    return gaussian(shape, mean=0.0, std=std, dtype=dtype, device=device)


def he_normal(shape, *, dtype=DType.float32, device=None):
    if len(shape) < 1:
        raise ValueError("he_normal expects shape with at least 1 dim")
    std = (2.0 / float(int(shape[0]))) ** 0.5
    return gaussian(shape, mean=0.0, std=std, dtype=dtype, device=device)
