"""Comparison and logical ops; results are bool (reference: nabla/ops/comparison.py:27-192).
None of them is differentiable: VJP/JVP give zeros."""
from __future__ import annotations

import torch

from ..core.tensor.api import Tensor
from .base import BinaryOperation, UnaryOperation


class ComparisonOp(BinaryOperation):
    """Elementwise binary predicate with a bool result (reference: nabla/ops/comparison.py:27)."""

    fn = None

    def torch_fn(self, a, b):
        return type(self).fn(a, b)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (None, None)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return None


_Cmp = ComparisonOp


class _Logical(_Cmp):
    def torch_fn(self, a, b):
        return type(self).fn(a.bool(), b.bool())


def _mk(name, fn, base=_Cmp):
    cls = type(name, (base,), {"fn": staticmethod(fn)})
    return cls()


_equal = _mk("EqualOp", torch.eq)
_not_equal = _mk("NotEqualOp", torch.ne)
_greater = _mk("GreaterOp", torch.gt)
_greater_equal = _mk("GreaterEqualOp", torch.ge)
_less = _mk("LessOp", torch.lt)
_less_equal = _mk("LessEqualOp", torch.le)
_logical_and = _mk("LogicalAndOp", torch.logical_and, _Logical)
_logical_or = _mk("LogicalOrOp", torch.logical_or, _Logical)
_logical_xor = _mk("LogicalXorOp", torch.logical_xor, _Logical)


for _op in (_equal, _not_equal, _greater, _greater_equal, _less, _less_equal, _logical_and, _logical_or, _logical_xor):
    globals()[type(_op).__name__] = type(_op)
del _op


class ComparisonUnaryOp(UnaryOperation):
    """Elementwise unary predicate with a bool result (reference: nabla/ops/comparison.py:43)."""

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (None,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return None


class LogicalNotOp(ComparisonUnaryOp):
    def torch_fn(self, x):
        return torch.logical_not(x)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (None,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return None


_logical_not = LogicalNotOp()


def equal(x, y) -> Tensor: return _equal(x, y)
def not_equal(x, y) -> Tensor: return _not_equal(x, y)
def greater(x, y) -> Tensor: return _greater(x, y)
def greater_equal(x, y) -> Tensor: return _greater_equal(x, y)
def less(x, y) -> Tensor: return _less(x, y)
def less_equal(x, y) -> Tensor: return _less_equal(x, y)
def logical_and(x, y) -> Tensor: return _logical_and(x, y)
def logical_or(x, y) -> Tensor: return _logical_or(x, y)
def logical_xor(x, y) -> Tensor: return _logical_xor(x, y)
def logical_not(x) -> Tensor: return _logical_not(x)
