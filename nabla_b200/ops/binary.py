"""Binary ops and matmul (reference: nabla/ops/binary.py:18-602).

Partial-sum passthrough: add/sub carry a pending sum only when *both* operands carry it;
mul/matmul/outer when at most one does (they are linear in each operand); div only in the
numerator; mod/pow never.
"""
from __future__ import annotations

import torch

from ..core.tensor.api import Tensor
from ..types import DType
from .base import BinaryOperation, Operation, ensure_tensor


def _result_float(a: Tensor) -> bool:
    return a.dtype.is_float()


class AddOp(BinaryOperation):
    native_op = "add"
    partial_policy = "all"

    def torch_fn(self, a, b):
        return torch.add(a, b)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (cot, cot)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return tangents[0] + tangents[1]


class SubOp(BinaryOperation):
    native_op = "sub"
    partial_policy = "all"

    def torch_fn(self, a, b):
        return torch.sub(a, b)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (cot, -cot)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return tangents[0] - tangents[1]


class MulOp(BinaryOperation):
    native_op = "mul"
    partial_policy = "one"

    def torch_fn(self, a, b):
        return torch.mul(a, b)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        a, b = primals
        return (cot * b, cot * a)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        a, b = primals
        return tangents[0] * b + a * tangents[1]


class DivOp(BinaryOperation):
    native_op = "div"
    partial_policy = "first"

    def torch_fn(self, a, b):
        if not a.dtype.is_floating_point and not b.dtype.is_floating_point:
            return torch.div(a, b, rounding_mode="trunc") if False else torch.true_divide(a, b)
        return torch.div(a, b)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        a, b = primals
        return (cot / b, -(cot * outputs) / b)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        a, b = primals
        return (tangents[0] - outputs * tangents[1]) / b


class ModOp(BinaryOperation):
    def torch_fn(self, a, b):
        return torch.remainder(a, b)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .unary import floor

        a, b = primals
        return (cot, -(cot * floor(a / b)))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        from .unary import floor

        a, b = primals
        return tangents[0] - floor(a / b) * tangents[1]


class PowOp(BinaryOperation):
    def torch_fn(self, a, b):
        return torch.pow(a, b)

    @staticmethod
    def _safe_log(a):
        # d/db a^b = a^b log a is only defined for a > 0; elsewhere contribute 0 instead of NaN
        from .comparison import greater
        from .control_flow import where
        from .creation import ones_like, zeros_like
        from .unary import log

        pos = greater(a, 0.0)
        return where(pos, log(where(pos, a, ones_like(a))), zeros_like(a))

    def vjp_rule(self, primals, cot, outputs, kwargs):
        a, b = primals
        da = cot * b * pow(a, b - 1.0)
        db = cot * outputs * self._safe_log(a)
        return (da, db)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        a, b = primals
        return tangents[0] * b * pow(a, b - 1.0) + tangents[1] * outputs * self._safe_log(a)


class OuterOp(Operation):
    partial_policy = "one"

    def kernel(self, a, b):
        return a.unsqueeze(-1) * b.unsqueeze(-2)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        from ..core.sharding.propagation import OpShardingRuleTemplate

        return OpShardingRuleTemplate.parse("... i, ... j -> ... i j").instantiate(input_shapes)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .reduction import reduce_sum
        from .view import unsqueeze

        a, b = primals
        return (reduce_sum(cot * unsqueeze(b, axis=-2), axis=-1), reduce_sum(cot * unsqueeze(a, axis=-1), axis=-2))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        a, b = primals
        return outer(tangents[0], b) + outer(a, tangents[1])


class MatmulOp(Operation):
    """``(..., m, k) @ (..., k, n)``. On CUDA bf16 operands this is the tcgen05 GEMM."""

    partial_policy = "one"

    def kernel(self, a, b):
        from .. import native

        if native.use_native(a) and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.numel() and b.numel():
            return native.gemm_bf16(a, b) if (a.dim() <= 3 and b.dim() <= 3) else _bmm_nd(a, b)
        return torch.matmul(a, b)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        from ..core.sharding.propagation import OpShardingRuleTemplate

        return OpShardingRuleTemplate.parse("... m k, ... k n -> ... m n").instantiate(input_shapes)

    def infer_output_rank(self, input_shapes, **kw):
        return max(len(s) for s in input_shapes)

    def compute_cost(self, input_shapes, output_shapes) -> float:
        a, b = input_shapes[0], input_shapes[1]
        batch = 1
        for d in output_shapes[0][:-2]:
            batch *= int(d)
        return 2.0 * batch * int(a[-2]) * int(a[-1]) * int(b[-1])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .view import swap_axes

        a, b = primals
        return (matmul(cot, swap_axes(b, -2, -1)), matmul(swap_axes(a, -2, -1), cot))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        a, b = primals
        return matmul(tangents[0], b) + matmul(a, tangents[1])


def _bmm_nd(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    from .. import native

    bshape = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    a3 = a.expand(*bshape, *a.shape[-2:]).reshape(-1, *a.shape[-2:])
    b3 = b.expand(*bshape, *b.shape[-2:]).reshape(-1, *b.shape[-2:])
    return native.gemm_bf16(a3, b3).reshape(*bshape, a.shape[-2], b.shape[-1])


_add, _sub, _mul, _div, _mod, _pow, _outer, _matmul = (AddOp(), SubOp(), MulOp(), DivOp(), ModOp(), PowOp(),
                                                       OuterOp(), MatmulOp())


def add(x, y) -> Tensor:
    return _add(x, y)


def sub(x, y) -> Tensor:
    return _sub(x, y)


def mul(x, y) -> Tensor:
    return _mul(x, y)


def div(x, y) -> Tensor:
    return _div(x, y)


def mod(x, y) -> Tensor:
    return _mod(x, y)


def pow(x, y) -> Tensor:
    return _pow(x, y)


def outer(x, y) -> Tensor:
    a = ensure_tensor(x)
    b = ensure_tensor(y, a)
    return _outer(a, b)


def matmul(x, y) -> Tensor:
    """Matrix product with numpy semantics (1-D operands are promoted and squeezed back)."""
    from .view import squeeze, unsqueeze

    a = ensure_tensor(x, y if isinstance(y, Tensor) else None)
    b = ensure_tensor(y, a)
    a1 = a.rank == 1
    b1 = b.rank == 1
    if a1:
        a = unsqueeze(a, axis=0)
    if b1:
        b = unsqueeze(b, axis=-1)
    bd = max(a._impl.batch_dims, b._impl.batch_dims)
    if bd:
        # under vmap the physical arrays carry the mapped dims in front, so numpy's right-aligned
        # broadcasting of the LOGICAL batch dims has to be made explicit: first give both operands the
        # same mapped dims, then pad the shorter logical shape with size-1 dims just behind them
        from .view.axes import unsqueeze_physical
        from .view.batch import broadcast_batch_dims

        ref = a if a._impl.batch_dims == bd else b
        if a._impl.batch_dims < bd:
            a = broadcast_batch_dims(a, ref._impl.batch_shape)
        if b._impl.batch_dims < bd:
            b = broadcast_batch_dims(b, ref._impl.batch_shape)
        ra, rb = len(a._impl.global_shape), len(b._impl.global_shape)
        while ra < rb:
            a = unsqueeze_physical(a, axis=bd)
            ra += 1
        while rb < ra:
            b = unsqueeze_physical(b, axis=bd)
            rb += 1
    out = _matmul(a, b)
    if a1 and b1:
        out = squeeze(out, axis=(-2, -1))
    elif a1:
        out = squeeze(out, axis=-2)
    elif b1:
        out = squeeze(out, axis=-1)
    return out
