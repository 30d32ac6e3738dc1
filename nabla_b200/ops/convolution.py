"""2-D convolution (reference: nabla/ops/convolution.py:220-790).

``conv2d``: NHWC input, HWIO (R,S,C,F) filter, stride, 4-way padding (top, bottom, left,
right); dilation 1 and groups 1 only (as in the reference). ``conv2d_transpose``: filter
(K_h, K_w, C_out, C_in), no output padding. Leading vmap batch dims are folded into N.

On GPU every piece runs on this package's kernels (no cuDNN call):
  * forward: im2col + the tcgen05 GEMM for wide bf16 channels (C*R*S >= 64), a direct kernel
    for narrow ones or fp32;
  * input gradient: a convolution again - the cotangent, zero-dilated by the stride and padded to
    "full", correlated with the spatially flipped, channel-transposed filter - so it goes through
    the same forward paths (reference: nabla/ops/convolution.py:309-353);
  * filter gradient: im2col(x)^T @ dy on the tcgen05 GEMM (fp32 output) for wide bf16 channels,
    otherwise the direct reduction kernel ``conv2d_wgrad_direct`` (reference: :354-392);
  * ``conv2d_transpose``: the input-gradient computation with the roles of data and cotangent
    swapped (reference: :429-466).
On CPU the same ops use torch's convolution functions.
"""
from __future__ import annotations

import torch
import torch.nn.functional as TF

from ..core.sharding.propagation import OpShardingRule
from ..core.tensor.api import Tensor
from .base import Operation, ensure_tensor


def _two(v, name):
    if isinstance(v, int):
        return (v, v)
    v = tuple(int(a) for a in v)
    if len(v) != 2:
        raise ValueError(f"{name} must be an int or a pair, got {v}")
    return v


def _pad4(p):
    if isinstance(p, int):
        return (p, p, p, p)
    p = tuple(int(a) for a in p)
    if len(p) == 2:
        return (p[0], p[0], p[1], p[1])
    if len(p) == 4:
        return p
    raise ValueError(f"padding must be an int, (h, w) or (top, bottom, left, right), got {p}")


def _fold(x: torch.Tensor):
    """(B..., N, H, W, C) -> (B*N, H, W, C) and the leading shape to restore."""
    lead = x.shape[:-3]
    return x.reshape(-1, *x.shape[-3:]), lead


def _conv_fwd(x, w, bias, stride, padding):
    from .. import native

    x4, lead = _fold(x)
    pt, pb, pl, pr = padding
    R, S, C, F = w.shape
    if native.use_native(x4) and x4.dtype in (torch.bfloat16, torch.float32) and x4.numel():
        from ..native import kernels

        if x4.dtype == torch.bfloat16 and (C * R * S) % 8 == 0 and C * R * S >= 64 and F % 8 == 0:
            # im2col + tensor-core GEMM
            xp = TF.pad(x4, (0, 0, pl, pr, pt, pb))
            N, H, W, _ = xp.shape
            OH, OW = (H - R) // stride[0] + 1, (W - S) // stride[1] + 1
            cols = xp.unfold(1, R, stride[0]).unfold(2, S, stride[1])          # N,OH,OW,C,R,S
            cols = cols.permute(0, 1, 2, 4, 5, 3).reshape(N * OH * OW, R * S * C)
            y = native.gemm_bf16(cols, w.reshape(R * S * C, F), bias=bias)
            return y.reshape(*lead, OH, OW, F)
        y = kernels.conv2d_direct(x4, w, bias, stride, padding)
        return y.reshape(*lead, *y.shape[1:])
    xp = TF.pad(x4.permute(0, 3, 1, 2), (pl, pr, pt, pb))
    y = TF.conv2d(xp, w.permute(3, 2, 0, 1).to(xp.dtype), bias=None if bias is None else bias.to(xp.dtype), stride=stride)
    y = y.permute(0, 2, 3, 1)
    return y.reshape(*lead, *y.shape[1:])


def _own_kernels(t: torch.Tensor) -> bool:
    from .. import native

    return t.numel() > 0 and native.use_native(t) and t.dtype in (torch.bfloat16, torch.float32)


def _dgrad_as_conv(dy4: torch.Tensor, w: torch.Tensor, out_hw, stride, padding) -> torch.Tensor:
    """Input gradient of ``conv2d(x, w)`` for cotangent ``dy4`` (N, OH, OW, F), filter (R, S, C, F),
    as a stride-1 convolution over the zero-dilated cotangent; result (N, H, W, C)."""
    pt, pb, pl, pr = padding
    H, W = out_hw
    R, S, C, F = w.shape
    N, OH, OW, _ = dy4.shape
    sh, sw = stride
    hz, wz = (OH - 1) * sh + 1, (OW - 1) * sw + 1
    if sh > 1 or sw > 1:
        z = torch.zeros((N, hz, wz, F), dtype=dy4.dtype, device=dy4.device)
        z[:, ::sh, ::sw] = dy4
    else:
        z = dy4
    # out[o] = sum_r' zpad[o + r'] wf[r'] with wf the flipped filter; o = 0 must be input row 0
    top, left = R - 1 - pt, S - 1 - pl
    bottom, right = H + R - 1 - top - hz, W + S - 1 - left - wz
    if min(top, left, bottom, right) < 0:          # padding larger than the filter reach: crop instead
        z = z[:, max(0, -top): hz - max(0, -bottom), max(0, -left): wz - max(0, -right)]
        top, left, bottom, right = max(0, top), max(0, left), max(0, bottom), max(0, right)
    wf = w.flip(0, 1).permute(0, 1, 3, 2).contiguous()      # (R, S, F, C): in-channels F, out-channels C
    return _conv_fwd(z, wf, None, (1, 1), (top, bottom, left, right))


def _wgrad_own(x4: torch.Tensor, dy4: torch.Tensor, w_shape, stride, padding) -> torch.Tensor:
    from .. import native
    from ..native import kernels

    pt, pb, pl, pr = padding
    R, S, C, F = w_shape
    if x4.dtype == torch.bfloat16 and (C * R * S) % 8 == 0 and C * R * S >= 64 and F % 8 == 0:
        xp = TF.pad(x4, (0, 0, pl, pr, pt, pb))
        N = xp.shape[0]
        OH, OW = dy4.shape[1], dy4.shape[2]
        cols = xp.unfold(1, R, stride[0]).unfold(2, S, stride[1])[:, :OH, :OW]       # N,OH,OW,C,R,S
        cols = cols.permute(0, 1, 2, 4, 5, 3).reshape(N * OH * OW, R * S * C)
        dw = native.gemm_bf16(cols.t(), dy4.reshape(N * OH * OW, F).contiguous(), out_dtype=torch.float32)
        return dw.reshape(R, S, C, F).to(x4.dtype)
    return kernels.conv2d_wgrad_direct(x4, dy4, w_shape, stride, padding)


def _conv_transpose_fwd(x, w, bias, stride, padding):
    """x (N,H,W,Cin), w (R,S,Cout,Cin) -> (N, (H-1)*s+R - pt - pb, ..., Cout)."""
    x4, lead = _fold(x)
    pt, pb, pl, pr = padding
    if _own_kernels(x4):
        R, S = w.shape[0], w.shape[1]
        oh = (x4.shape[1] - 1) * stride[0] + R - pt - pb
        ow = (x4.shape[2] - 1) * stride[1] + S - pl - pr
        y = _dgrad_as_conv(x4, w.to(x4.dtype), (oh, ow), stride, padding)
        if bias is not None:
            y = y + bias.to(y.dtype)
        return y.reshape(*lead, *y.shape[1:])
    y = TF.conv_transpose2d(x4.permute(0, 3, 1, 2), w.permute(3, 2, 0, 1).to(x4.dtype), stride=stride)
    y = y.permute(0, 2, 3, 1)
    H, W = y.shape[1], y.shape[2]
    y = y[:, pt:H - pb, pl:W - pr, :]
    if bias is not None:
        y = y + bias.to(y.dtype)
    y = y.contiguous()
    return y.reshape(*lead, *y.shape[1:])


def _conv_rule(input_shapes, n_out=1):
    xs = input_shapes[0]
    r = len(xs)
    mx = {i: [f"b{i}"] for i in range(r - 3)}
    mx.update({r - 3: ["bcast_h"], r - 2: ["bcast_w"], r - 1: ["bcast_c"]})
    ins = [mx] + [{i: [f"bcast_w{j}_{i}"] for i in range(len(s))} for j, s in enumerate(input_shapes[1:])]
    out = {i: [f"b{i}"] for i in range(r - 3)}
    out.update({r - 3: ["oh"], r - 2: ["ow"], r - 1: ["of"]})
    return OpShardingRule(ins, [out])


class Conv2dOp(Operation):
    def kernel(self, x, w, bias=None, *, stride, padding, **kw):
        return _conv_fwd(x, w, bias, stride, padding)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        return _conv_rule(input_shapes)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        x, w = primals[0], primals[1]
        dx = _conv_dgrad(cot, w, x_shape=tuple(x._impl.global_shape[-3:]), stride=kwargs["stride"],
                         padding=kwargs["padding"])
        dw = _conv_wgrad(x, cot, w_shape=tuple(w._impl.global_shape), stride=kwargs["stride"], padding=kwargs["padding"])
        res = [dx, dw]
        if len(primals) > 2:
            from .reduction import reduce_sum

            res.append(reduce_sum(cot, axis=tuple(range(cot.rank - 1))))
        return tuple(res)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        x, w = primals[0], primals[1]
        t = _conv2d(tangents[0], w, **kwargs) + _conv2d(x, tangents[1], **kwargs)
        if len(primals) > 2 and tangents[2] is not None:
            t = t + tangents[2]
        return t


class ConvDgradOp(Operation):
    """Gradient of conv2d wrt its input."""

    def kernel(self, dy, w, *, x_shape, stride, padding):
        dy4, lead = _fold(dy)
        pt, pb, pl, pr = padding
        H, W, C = x_shape
        if _own_kernels(dy4):
            return _dgrad_as_conv(dy4, w.to(dy4.dtype), (H, W), stride, padding).reshape(*lead, H, W, C)
        g = torch.nn.grad.conv2d_input((dy4.shape[0], C, H + pt + pb, W + pl + pr), w.permute(3, 2, 0, 1).to(dy4.dtype),
                                       dy4.permute(0, 3, 1, 2), stride=stride)
        g = g[:, :, pt:pt + H, pl:pl + W].permute(0, 2, 3, 1).contiguous()
        return g.reshape(*lead, H, W, C)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        return _conv_rule(input_shapes)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        dy, w = primals
        ddy = _conv2d(cot, w, stride=kwargs["stride"], padding=kwargs["padding"])
        dw = _conv_wgrad(cot, dy, w_shape=tuple(w._impl.global_shape), stride=kwargs["stride"], padding=kwargs["padding"])
        return (ddy, dw)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        dy, w = primals
        return _conv_dgrad_op(tangents[0], w, **kwargs) + _conv_dgrad_op(dy, tangents[1], **kwargs)


class ConvWgradOp(Operation):
    """Gradient of conv2d wrt its filter: sum over N and output pixels."""

    partial_policy = "one"

    def kernel(self, x, dy, *, w_shape, stride, padding):
        x4, _ = _fold(x)
        dy4, _ = _fold(dy)
        pt, pb, pl, pr = padding
        R, S, C, F = w_shape
        if _own_kernels(x4):
            return _wgrad_own(x4, dy4, tuple(w_shape), stride, padding)
        xp = TF.pad(x4.permute(0, 3, 1, 2), (pl, pr, pt, pb))
        g = torch.nn.grad.conv2d_weight(xp.float(), (F, C, R, S), dy4.permute(0, 3, 1, 2).float(), stride=stride)
        return g.permute(2, 3, 1, 0).contiguous().to(x.dtype)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        xs = input_shapes[0]
        r = len(xs)
        mx = {i: [f"b{i}"] for i in range(r - 3)}
        mx.update({r - 3: ["bcast_h"], r - 2: ["bcast_w"], r - 1: ["bcast_c"]})
        my = {i: [f"b{i}"] for i in range(r - 3)}
        my.update({r - 3: ["bcast_oh"], r - 2: ["bcast_ow"], r - 1: ["bcast_f"]})
        return OpShardingRule([mx, my], [{0: ["r"], 1: ["s"], 2: ["c"], 3: ["f"]}])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        x, dy = primals
        gx = _conv_dgrad(dy, cot, x_shape=tuple(x._impl.global_shape[-3:]), stride=kwargs["stride"],
                         padding=kwargs["padding"])
        gdy = _conv2d(x, cot, stride=kwargs["stride"], padding=kwargs["padding"])
        return (gx, gdy)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        x, dy = primals
        return _conv_wgrad_op(tangents[0], dy, **kwargs) + _conv_wgrad_op(x, tangents[1], **kwargs)


class Conv2dTransposeOp(Operation):
    def kernel(self, x, w, bias=None, *, stride, padding, **kw):
        return _conv_transpose_fwd(x, w, bias, stride, padding)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        return _conv_rule(input_shapes)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .view import permute

        x, w = primals[0], primals[1]
        # conv_transpose(x, w) = dgrad of a conv with filter w' = w viewed as (R,S,Cout->"C", Cin->"F")
        dx = _conv2d(cot, w, stride=kwargs["stride"], padding=kwargs["padding"])
        dw = _conv_wgrad(cot, x, w_shape=tuple(w._impl.global_shape), stride=kwargs["stride"], padding=kwargs["padding"])
        res = [dx, dw]
        if len(primals) > 2:
            from .reduction import reduce_sum

            res.append(reduce_sum(cot, axis=tuple(range(cot.rank - 1))))
        return tuple(res)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        x, w = primals[0], primals[1]
        t = _conv2d_transpose(tangents[0], w, **kwargs) + _conv2d_transpose(x, tangents[1], **kwargs)
        if len(primals) > 2 and tangents[2] is not None:
            t = t + tangents[2]
        return t


_conv2d, _conv_dgrad_op, _conv_wgrad_op, _conv2d_transpose = Conv2dOp(), ConvDgradOp(), ConvWgradOp(), Conv2dTransposeOp()
Conv2DOp, Conv2DTransposeOp = Conv2dOp, Conv2dTransposeOp      # the reference's spelling (nabla/ops/convolution.py)


def _conv_dgrad(dy, w, *, x_shape, stride, padding):
    return _conv_dgrad_op(dy, w, x_shape=tuple(x_shape), stride=tuple(stride), padding=tuple(padding))


def _conv_wgrad(x, dy, *, w_shape, stride, padding):
    return _conv_wgrad_op(x, dy, w_shape=tuple(w_shape), stride=tuple(stride), padding=tuple(padding))


def _require_positive(value, name: str) -> None:
    if any(int(v) <= 0 for v in value):
        raise ValueError(f"{name} values must be > 0, got {tuple(value)}")


def _require_nonnegative(value, name: str) -> None:
    if any(int(v) < 0 for v in value):
        raise ValueError(f"{name} values must be >= 0, got {tuple(value)}")


def _check(x, w, dilation, groups, name):
    if len(x.shape) < 4 or len(w.shape) != 4:
        raise ValueError(f"{name} expects rank-4 tensors, got x={tuple(x.shape)}, filter={tuple(w.shape)}")
    _require_positive(_two(dilation, "dilation"), "dilation")
    if int(groups) <= 0:
        raise ValueError(f"groups must be > 0, got {int(groups)}")
    if _two(dilation, "dilation") != (1, 1):
        raise ValueError(f"{name} currently supports only dilation=(1, 1)")
    if int(groups) != 1:
        raise ValueError(f"{name} grouped mode (groups={int(groups)}) is not supported: only groups=1")


def _check_bias(bias, c_out: int, name: str):
    bias = ensure_tensor(bias)
    if len(bias.shape) != 1:
        raise ValueError(f"{name} bias must be rank-1 [C_out], got shape={tuple(int(d) for d in bias.shape)}")
    if int(bias.shape[0]) != c_out:
        raise ValueError(f"{name} bias size ({int(bias.shape[0])}) must match filter C_out ({c_out})")
    return bias


def conv2d(x, filter, *, stride=(1, 1), dilation=(1, 1), padding=(0, 0, 0, 0), groups: int = 1, bias=None,
           input_layout=None, filter_layout=None) -> Tensor:
    x, filter = ensure_tensor(x), ensure_tensor(filter)
    if input_layout is not None or filter_layout is not None:
        raise ValueError("conv2d supports only the default NHWC / RSCF layouts")
    _check(x, filter, dilation, groups, "conv2d")
    st, pd = _two(stride, "stride"), _pad4(padding)
    _require_positive(st, "stride")
    _require_nonnegative(pd, "padding")
    if int(x.shape[-1]) != int(filter.shape[2]):
        raise ValueError(f"Input channels ({int(x.shape[-1])}) must match filter channels*groups ({int(filter.shape[2])})")
    if bias is not None:
        bias = _check_bias(bias, int(filter.shape[3]), "conv2d")
        return _conv2d(x, filter, bias, stride=st, padding=pd)
    return _conv2d(x, filter, stride=st, padding=pd)


def conv2d_transpose(x, filter, *, stride=(1, 1), dilation=(1, 1), padding=(0, 0, 0, 0), output_paddings=(0, 0),
                     bias=None, input_layout=None, filter_layout=None) -> Tensor:
    x, filter = ensure_tensor(x), ensure_tensor(filter)
    if input_layout is not None or filter_layout is not None:
        raise ValueError("conv2d_transpose supports only the default NHWC / RSCF layouts")
    _check(x, filter, dilation, 1, "conv2d_transpose")
    if _two(output_paddings, "output_paddings") != (0, 0):
        raise ValueError("conv2d_transpose currently supports only output_paddings=(0, 0)")
    st, pd = _two(stride, "stride"), _pad4(padding)
    _require_positive(st, "stride")
    _require_nonnegative(pd, "padding")
    if int(x.shape[-1]) != int(filter.shape[3]):
        raise ValueError(f"Input channels ({int(x.shape[-1])}) must match filter input channels ({int(filter.shape[3])})")
    if bias is not None:
        return _conv2d_transpose(x, filter, _check_bias(bias, int(filter.shape[2]), "conv2d_transpose"), stride=st, padding=pd)
    return _conv2d_transpose(x, filter, stride=st, padding=pd)
