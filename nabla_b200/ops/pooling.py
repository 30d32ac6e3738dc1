"""2-D pooling on NHWC tensors (reference: nabla/ops/pooling.py:24-214, where pooling is a
Python double loop of slice + reduce + stack per output pixel). Here each of avg/max pooling
is one op with a single forward and a single backward kernel. Average pooling counts padded
zeros in the divisor (kernel area), max pooling ignores padding."""
from __future__ import annotations

import torch
import torch.nn.functional as TF

from ..core.sharding.propagation import OpShardingRule
from ..core.tensor.api import Tensor
from .base import Operation, ensure_tensor
from .convolution import _fold, _pad4, _require_nonnegative, _require_positive, _two


def _native_ok(x):
    from .. import native

    return native.use_native(x) and x.dtype in (torch.bfloat16, torch.float32) and x.numel() > 0


def _rule(input_shapes):
    r = len(input_shapes[0])
    m = {i: [f"b{i}"] for i in range(r - 3)}
    m.update({r - 3: ["bcast_h"], r - 2: ["bcast_w"], r - 1: ["c"]})
    out = {i: [f"b{i}"] for i in range(r - 3)}
    out.update({r - 3: ["oh"], r - 2: ["ow"], r - 1: ["c"]})
    return m, out


class Pool2dOp(Operation):
    def kernel(self, x, *, kernel_size, stride, padding, mode: str):
        x4, lead = _fold(x)
        kh, kw = kernel_size
        pt, pb, pl, pr = padding
        if _native_ok(x4) and pt == pb and pl == pr:
            from ..native import kernels

            y = kernels.pool2d_fwd(x4, kh, kw, stride[0], stride[1], pt, pl, mode)
            return y.reshape(*lead, *y.shape[1:])
        xc = x4.permute(0, 3, 1, 2)
        if mode == "avg":
            xc = TF.pad(xc, (pl, pr, pt, pb))
            y = TF.avg_pool2d(xc, (kh, kw), stride)
        else:
            xc = TF.pad(xc, (pl, pr, pt, pb), value=float("-inf"))
            y = TF.max_pool2d(xc, (kh, kw), stride)
        y = y.permute(0, 2, 3, 1).contiguous()
        return y.reshape(*lead, *y.shape[1:])

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        m, out = _rule(input_shapes)
        return OpShardingRule([m], [out])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (_pool_bwd(primals[0], cot, **kwargs),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        if kwargs["mode"] == "avg":
            return _pool(tangents[0], **kwargs)
        # max: every window's tangent is the tangent at its arg-max (the transpose of the VJP routing)
        kw = {k: v for k, v in kwargs.items() if k != "mode"}
        return _pool_select(primals[0], tangents[0], **kw)


class Pool2dBwdOp(Operation):
    def kernel(self, x, dy, *, kernel_size, stride, padding, mode: str):
        x4, lead = _fold(x)
        dy4, _ = _fold(dy)
        kh, kw = kernel_size
        pt, pb, pl, pr = padding
        if _native_ok(x4) and pt == pb and pl == pr and dy4.dtype == x4.dtype:
            from ..native import kernels

            return kernels.pool2d_bwd(x4, dy4, kh, kw, stride[0], stride[1], pt, pl, mode).reshape(x.shape)
        xr = x4.detach().float().permute(0, 3, 1, 2).requires_grad_(True)
        with torch.enable_grad():
            if mode == "avg":
                y = TF.avg_pool2d(TF.pad(xr, (pl, pr, pt, pb)), (kh, kw), stride)
            else:
                y = TF.max_pool2d(TF.pad(xr, (pl, pr, pt, pb), value=float("-inf")), (kh, kw), stride)
            (g,) = torch.autograd.grad(y, xr, dy4.float().permute(0, 3, 1, 2))
        return g.permute(0, 2, 3, 1).contiguous().to(x.dtype).reshape(x.shape)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        m, out = _rule(input_shapes)
        return OpShardingRule([m, out], [dict(m)])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        if kwargs["mode"] == "avg":
            return (None, _pool(cot, **kwargs))
        # the routing is linear in dy (and piecewise constant in x): its transpose picks, for every
        # window, the cotangent at the window's arg-max
        kw = {k: v for k, v in kwargs.items() if k != "mode"}
        return (None, _pool_select(primals[0], cot, **kw))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _pool_bwd(primals[0], tangents[1], **kwargs) if tangents[1] is not None else None


class Pool2dSelectOp(Operation):
    """``out[window] = t[arg-max of x over the window]`` for max pooling's windows: the forward-mode
    derivative of ``max_pool2d`` at ``x`` applied to ``t``."""

    def kernel(self, x, t, *, kernel_size, stride, padding):
        x4, lead = _fold(x)
        t4, _ = _fold(t)
        kh, kw = kernel_size
        pt, pb, pl, pr = padding
        if _native_ok(x4) and pt == pb and pl == pr and t4.dtype == x4.dtype:
            from ..native import kernels

            y = kernels.pool2d_select(x4, t4, kh, kw, stride[0], stride[1], pt, pl)
            return y.reshape(*lead, *y.shape[1:])
        xc = TF.pad(x4.float().permute(0, 3, 1, 2), (pl, pr, pt, pb), value=float("-inf"))
        tc = TF.pad(t4.float().permute(0, 3, 1, 2), (pl, pr, pt, pb))
        y, idx = TF.max_pool2d(xc, (kh, kw), stride, return_indices=True)
        out = tc.flatten(2).gather(2, idx.flatten(2)).view_as(y)
        out = out.permute(0, 2, 3, 1).contiguous().to(t.dtype)
        return out.reshape(*lead, *out.shape[1:])

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        m, out = _rule(input_shapes)
        return OpShardingRule([m, dict(m)], [out])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (None, _pool_bwd(primals[0], cot, mode="max", **kwargs))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return _pool_select(primals[0], tangents[1], **kwargs) if tangents[1] is not None else None


_pool, _pool_bwd, _pool_select = Pool2dOp(), Pool2dBwdOp(), Pool2dSelectOp()


def _call(x, kernel_size, stride, padding, dilation, mode):
    x = ensure_tensor(x)
    if len(x.shape) < 4:
        raise ValueError(f"pool2d expects an NHWC tensor, got shape {tuple(x.shape)}")
    k = _two(kernel_size, "kernel_size")
    s = _two(stride if stride is not None else k, "stride")
    p = _pad4(padding)
    _require_positive(k, "kernel_size")
    _require_positive(s, "stride")
    _require_nonnegative(p, "padding")
    if _two(dilation, "dilation") != (1, 1):
        raise ValueError("pool2d currently supports only dilation=(1, 1)")
    H, W = int(x.shape[-3]), int(x.shape[-2])
    oh = (H + p[0] + p[1] - k[0]) // s[0] + 1
    ow = (W + p[2] + p[3] - k[1]) // s[1] + 1
    if oh <= 0 or ow <= 0:
        raise ValueError(f"Non-positive pool2d output size H={oh}, W={ow}.")
    return _pool(x, kernel_size=k, stride=s, padding=p, mode=mode)


def avg_pool2d(x, kernel_size, stride=None, padding=0, dilation=(1, 1)) -> Tensor:
    return _call(x, kernel_size, stride, padding, dilation, "avg")


def max_pool2d(x, kernel_size, stride=None, padding=0, dilation=(1, 1)) -> Tensor:
    return _call(x, kernel_size, stride, padding, dilation, "max")
