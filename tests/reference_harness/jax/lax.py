"""``jax.lax`` stand-in: the handful of primitives the reference's tests call directly."""
import math

import torch
import torch.nn.functional as F

from .numpy import _a


def add(x, y):
    return torch.add(_a(x), y)


def mul(x, y):
    return torch.mul(_a(x), y)


def max(x, y):  # noqa: A001
    return torch.maximum(_a(x), _a(y))


def min(x, y):  # noqa: A001
    return torch.minimum(_a(x), _a(y))


def rsqrt(x):
    return torch.rsqrt(_a(x))


def erf(x):
    return torch.erf(_a(x))


def stop_gradient(x):
    return _a(x).detach()


def dynamic_slice(x, start_indices, slice_sizes):
    idx = tuple(slice(int(s), int(s) + int(n)) for s, n in zip(start_indices, slice_sizes))
    return _a(x)[idx]


def dynamic_update_slice(x, update, start_indices):
    out = _a(x).clone()
    idx = tuple(slice(int(s), int(s) + int(n)) for s, n in zip(start_indices, update.shape))
    out[idx] = update
    return out


def _pads(padding, in_sizes, window, strides, dilation=None):
    """Per-dim (lo, hi) from 'VALID' / 'SAME' or an explicit list."""
    if not isinstance(padding, str):
        return [(int(lo), int(hi)) for lo, hi in padding]
    if padding.upper() == "VALID":
        return [(0, 0)] * len(in_sizes)
    out = []
    for i, n in enumerate(in_sizes):
        k = (window[i] - 1) * (dilation[i] if dilation else 1) + 1
        total = builtin_max((math.ceil(n / strides[i]) - 1) * strides[i] + k - n, 0)
        out.append((total // 2, total - total // 2))
    return out


import builtins as _b  # noqa: E402

builtin_max = _b.max


def reduce_window(x, init_value, computation, window_dimensions, window_strides, padding):
    """Windowed sum (``lax.add``) or max (``lax.max``) over every dim of ``x``."""
    x = _a(x)
    pads = _pads(padding, x.shape, window_dimensions, window_strides)
    is_max = computation is max
    fill = -math.inf if is_max else 0.0
    flat = []
    for lo, hi in reversed(pads):
        flat += [lo, hi]
    x = F.pad(x, flat, value=fill)
    for d, (w, s) in enumerate(zip(window_dimensions, window_strides)):
        if w == 1 and s == 1:
            continue
        x = x.unfold(d, w, s)
        x = x.amax(dim=-1) if is_max else x.sum(dim=-1)
    return x


def conv_general_dilated(lhs, rhs, window_strides, padding, lhs_dilation=None, rhs_dilation=None,
                         dimension_numbers=None, feature_group_count=1, **_):
    """2-D convolution for the layouts the tests use: ("NHWC", "HWIO", "NHWC") and ("NCHW", "OIHW", "NCHW")."""
    lhs, rhs = _a(lhs), _a(rhs)
    dn = tuple(dimension_numbers) if dimension_numbers is not None else ("NCHW", "OIHW", "NCHW")
    li, ri, oi = dn
    x = lhs.permute(*[li.index(c) for c in "NCHW"])
    w = rhs.permute(*[ri.index(c) for c in "OIHW"])
    dil = tuple(rhs_dilation) if rhs_dilation is not None else (1, 1)
    if lhs_dilation is not None and tuple(lhs_dilation) != (1, 1):
        # input dilation = transposed convolution: insert zeros between the input elements
        sh, sw = lhs_dilation
        n, c, h, wd = x.shape
        z = x.new_zeros(n, c, (h - 1) * sh + 1, (wd - 1) * sw + 1)
        z[:, :, ::sh, ::sw] = x
        x = z
    pads = _pads(padding, x.shape[2:], w.shape[2:], window_strides, dil)
    x = F.pad(x, [pads[1][0], pads[1][1], pads[0][0], pads[0][1]])
    y = F.conv2d(x, w, stride=tuple(window_strides), dilation=dil, groups=feature_group_count)
    return y.permute(*["NCHW".index(c) for c in oi])
