"""Unary elementwise ops, cast, softmax/logsoftmax (reference: nabla/ops/unary.py:20-871)."""
from __future__ import annotations

import math

import torch

from ..core.tensor.api import Tensor
from ..types import DType, as_dtype
from .base import AxisOp, Operation, UnaryOperation, ensure_tensor


def _u(name: str, fn, deriv=None, policy: str = "none", native: str | None = None):
    """Build a UnaryOperation subclass instance from a torch function and a derivative; ``native``
    names the entry of the pointwise kernel family that runs it on a GPU."""
    ns = {"torch_fn": lambda self, x: fn(x), "partial_policy": policy, "native_op": native}
    if deriv is not None:
        ns["_derivative"] = lambda self, x, y, kwargs: deriv(x, y)
    return type(name, (UnaryOperation,), ns)()


def _zeros_like(x):
    from .creation import zeros_like

    return zeros_like(x)


def _nondiff(name: str, fn, native: str | None = None):
    def vjp(self, primals, cot, outputs, kwargs):
        return (None,)

    def jvp(self, primals, tangents, outputs, kwargs):
        return None

    return type(name, (UnaryOperation,), {"torch_fn": lambda self, x: fn(x), "vjp_rule": vjp, "jvp_rule": jvp,
                                          "native_op": native})()


def _step(x):
    from .comparison import greater

    return cast(greater(x, 0.0), x.dtype)


def _sign(x):
    from .comparison import greater, less

    return cast(greater(x, 0.0), x.dtype) - cast(less(x, 0.0), x.dtype)


_relu = _u("ReluOp", torch.relu, lambda x, y: _step(x))


def _relu_vjp(self, primals, cotangents, outputs, kwargs):
    # one kernel (cot * [x > 0]) instead of greater -> cast -> mul
    from .fused import dact_mul

    return (dact_mul(cotangents, primals[0], "relu"),)


def _relu_jvp(self, primals, tangents, outputs, kwargs):
    from .fused import dact_mul

    return dact_mul(tangents[0], primals[0], "relu")


type(_relu).vjp_rule = _relu_vjp
type(_relu).jvp_rule = _relu_jvp
_sigmoid = _u("SigmoidOp", torch.sigmoid, lambda x, y: y * (1.0 - y), native="sigmoid")
_tanh = _u("TanhOp", torch.tanh, lambda x, y: 1.0 - y * y, native="tanh")
_exp = _u("ExpOp", torch.exp, lambda x, y: y, native="exp")
_abs = _u("AbsOp", torch.abs, lambda x, y: _sign(x), native="abs")
_log = _u("LogOp", torch.log, lambda x, y: 1.0 / x, native="log")
_sqrt = _u("SqrtOp", torch.sqrt, lambda x, y: 0.5 / y, native="sqrt")
_acos = _u("AcosOp", torch.acos, lambda x, y: -rsqrt(1.0 - x * x))
_atanh = _u("AtanhOp", torch.atanh, lambda x, y: 1.0 / (1.0 - x * x))
_cos = _u("CosOp", torch.cos, lambda x, y: -sin(x), native="cos")
_sin = _u("SinOp", torch.sin, lambda x, y: cos(x), native="sin")
_erf = _u("ErfOp", torch.erf, lambda x, y: (2.0 / math.sqrt(math.pi)) * exp(-(x * x)), native="erf")
_log1p = _u("Log1pOp", torch.log1p, lambda x, y: 1.0 / (1.0 + x), native="log1p")
_rsqrt = _u("RsqrtOp", torch.rsqrt, lambda x, y: -0.5 * y / x, native="rsqrt")
_silu = _u("SiluOp", torch.nn.functional.silu, lambda x, y: sigmoid(x) * (1.0 + x * (1.0 - sigmoid(x))))
_floor = _nondiff("FloorOp", torch.floor, native="floor")
_trunc = _nondiff("TruncOp", torch.trunc, native="trunc")
_round = _nondiff("RoundOp", torch.round, native="round")
_is_inf = _nondiff("IsInfOp", torch.isinf)
_is_nan = _nondiff("IsNanOp", torch.isnan)


# the generated op classes under their own names (`ExpOp`, `ReluOp`, ...; reference: nabla/ops/unary.py)
for _op in (_relu, _sigmoid, _tanh, _exp, _abs, _log, _sqrt, _acos, _atanh, _cos, _sin, _erf, _log1p, _rsqrt, _silu,
            _floor, _trunc, _round, _is_inf, _is_nan):
    globals()[type(_op).__name__] = type(_op)
del _op


class NegOp(UnaryOperation):
    partial_policy = "any"
    native_op = "neg"

    def torch_fn(self, x):
        return torch.neg(x)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (-cot,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return -tangents[0]


_neg = NegOp()


class GeluOp(UnaryOperation):
    def kernel(self, x, *, approximate: str = "none"):
        return torch.nn.functional.gelu(x, approximate="tanh" if approximate == "tanh" else "none")

    def _derivative(self, x, y, kwargs):
        if kwargs.get("approximate", "none") == "tanh":
            c = math.sqrt(2.0 / math.pi)
            u = c * (x + 0.044715 * x * x * x)
            t = tanh(u)
            return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * c * (1.0 + 3 * 0.044715 * x * x)
        cdf = 0.5 * (1.0 + erf(x * (1.0 / math.sqrt(2.0))))
        pdf = exp(-0.5 * (x * x)) * (1.0 / math.sqrt(2.0 * math.pi))
        return cdf + x * pdf


_gelu = GeluOp()


class StopGradientOp(UnaryOperation):
    """Identity whose derivative is zero (``jax.lax.stop_gradient``)."""

    partial_policy = "any"

    def torch_fn(self, x):
        return x

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (None,)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return None


_stop_gradient = StopGradientOp()


def stop_gradient(x) -> Tensor:
    return _stop_gradient(ensure_tensor(x))


class CastOp(Operation):
    """dtype conversion. Deliberately not partial-passthrough: rounding a partial sum and then
    summing differs from summing and then rounding."""

    def kernel(self, x, *, dtype: DType):
        return x.to(dtype.to_torch())

    def vjp_rule(self, primals, cot, outputs, kwargs):
        x = primals[0]
        if not x.dtype.is_float():
            return (None,)
        return (cast(cot, x.dtype),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        if not kwargs["dtype"].is_float():
            return None
        return cast(tangents[0], kwargs["dtype"])


_cast = CastOp()


class _SoftmaxBase(AxisOp):
    def sharding_rule(self, input_shapes, output_shapes, *, axis: int, **kw):
        from ..core.sharding.propagation import OpShardingRule

        rank = len(input_shapes[0])
        m = {i: [f"d{i}"] for i in range(rank)}
        return OpShardingRule([dict(m)], [dict(m)])


class SoftmaxOp(_SoftmaxBase):
    def kernel(self, x, *, axis: int = -1):
        from .. import native

        if native.use_native(x) and axis in (-1, x.dim() - 1) and x.dtype in (torch.bfloat16, torch.float32):
            from ..native import kernels

            if kernels.has("softmax"):
                return kernels.softmax(x, log=False)
        return torch.softmax(x, dim=axis)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .reduction import reduce_sum

        ax = kwargs.get("axis", -1)
        y = outputs
        return (y * (cot - reduce_sum(cot * y, axis=ax, keepdims=True)),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        from .reduction import reduce_sum

        ax = kwargs.get("axis", -1)
        y = outputs
        t = tangents[0]
        return y * (t - reduce_sum(t * y, axis=ax, keepdims=True))


class LogSoftmaxOp(_SoftmaxBase):
    def kernel(self, x, *, axis: int = -1):
        from .. import native

        if native.use_native(x) and axis in (-1, x.dim() - 1) and x.dtype in (torch.bfloat16, torch.float32):
            from ..native import kernels

            if kernels.has("softmax"):
                return kernels.softmax(x, log=True)
        return torch.log_softmax(x, dim=axis)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .reduction import reduce_sum

        ax = kwargs.get("axis", -1)
        return (cot - exp(outputs) * reduce_sum(cot, axis=ax, keepdims=True),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        from .reduction import reduce_sum

        ax = kwargs.get("axis", -1)
        t = tangents[0]
        return t - reduce_sum(exp(outputs) * t, axis=ax, keepdims=True)


_softmax, _logsoftmax = SoftmaxOp(), LogSoftmaxOp()


def _axis_is_sharded(x: Tensor, axis: int) -> bool:
    sp = x._impl.sharding
    if sp is None:
        return False
    rank = len(x._impl.global_shape)
    ax = axis + rank if axis < 0 else axis
    return bool(sp.dim_specs[ax + x._impl.batch_dims].axes)


def softmax(x: Tensor, axis: int = -1) -> Tensor:
    """Softmax along ``axis``. When that axis is split across devices it is decomposed into
    max / exp / sum so that the cross-shard max and sum run as collectives."""
    x = ensure_tensor(x)
    if _axis_is_sharded(x, axis):
        from .reduction import reduce_max, reduce_sum

        m = stop_gradient(reduce_max(x, axis=axis, keepdims=True))   # shift only: derivative is exactly 0
        e = exp(x - m)
        return e / reduce_sum(e, axis=axis, keepdims=True)
    return _softmax(x, axis=axis)


def logsoftmax(x: Tensor, axis: int = -1) -> Tensor:
    x = ensure_tensor(x)
    if _axis_is_sharded(x, axis):
        from .reduction import reduce_max, reduce_sum

        m = stop_gradient(reduce_max(x, axis=axis, keepdims=True))
        s = x - m
        return s - log(reduce_sum(exp(s), axis=axis, keepdims=True))
    return _logsoftmax(x, axis=axis)


def _wrap(op):
    def f(x) -> Tensor:
        return op(ensure_tensor(x))

    f.__name__ = op.name
    return f


relu, sigmoid, tanh, exp, abs, log, sqrt = map(_wrap, (_relu, _sigmoid, _tanh, _exp, _abs, _log, _sqrt))
acos, atanh, cos, sin, erf, log1p, rsqrt, silu = map(_wrap, (_acos, _atanh, _cos, _sin, _erf, _log1p, _rsqrt, _silu))
floor, trunc, round, is_inf, is_nan, neg = map(_wrap, (_floor, _trunc, _round, _is_inf, _is_nan, _neg))


def gelu(x, approximate: str = "none") -> Tensor:
    if approximate is True:
        approximate = "tanh"
    elif approximate in (False, None):
        approximate = "none"
    return _gelu(ensure_tensor(x), approximate=approximate)


def cast(x, dtype=None) -> Tensor:
    x = ensure_tensor(x)
    if dtype is None:          # the reference returns the tensor unchanged (nabla/ops/unary.py:792-798)
        return x
    dtype = as_dtype(dtype)
    if x.dtype is dtype:
        return x
    return _cast(x, dtype=dtype)
