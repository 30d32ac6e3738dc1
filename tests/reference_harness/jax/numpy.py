"""``jax.numpy`` stand-in on torch: the array functions that the reference's unit tests use to
compute expected values. Arrays are plain CPU ``torch.Tensor`` objects, so they go through
``torch.func`` transforms and DLPack unchanged. Only numpy semantics that torch names differently
are translated (``axis`` / ``keepdims``, default dtypes int32 / float32, ``split`` by count)."""
from __future__ import annotations

import builtins
import math

import numpy as _np
import torch

float16, bfloat16, float32, float64 = torch.float16, torch.bfloat16, torch.float32, torch.float64
int8, int16, int32, int64 = torch.int8, torch.int16, torch.int32, torch.int64
uint8, bool_ = torch.uint8, torch.bool
inf, pi, e, nan, newaxis = math.inf, math.pi, math.e, math.nan, None
ndarray = torch.Tensor

_DT = {"float16": float16, "bfloat16": bfloat16, "float32": float32, "float64": float64, "int8": int8,
       "int16": int16, "int32": int32, "int64": int64, "uint8": uint8, "bool": bool_, float: float32, int: int32,
       bool: bool_, _np.float32: float32, _np.float64: float64, _np.int32: int32, _np.int64: int64, _np.bool_: bool_}


def _dt(dtype):
    if dtype is None or isinstance(dtype, torch.dtype):
        return dtype
    if dtype in _DT:
        return _DT[dtype]
    return _DT[_np.dtype(dtype).name]


def asarray(obj, dtype=None):
    dtype = _dt(dtype)
    if isinstance(obj, torch.Tensor):
        return obj if dtype is None or obj.dtype == dtype else obj.to(dtype)
    if hasattr(obj, "__dlpack__") and not isinstance(obj, _np.ndarray):
        t = torch.from_dlpack(obj)
        return t if dtype is None else t.to(dtype)
    if isinstance(obj, (list, tuple)) and builtins.any(isinstance(o, torch.Tensor) for o in obj):
        t = torch.stack([asarray(o) for o in obj])
        return t if dtype is None else t.to(dtype)
    a = _np.asarray(obj)
    if dtype is None:
        if a.dtype == _np.float64:
            dtype = float32
        elif a.dtype == _np.int64:
            dtype = int32
    t = torch.from_numpy(_np.ascontiguousarray(a)).reshape(a.shape)
    return t.clone() if dtype is None else t.to(dtype)


def array(obj, dtype=None, copy=True):
    t = asarray(obj, dtype)
    return t.clone() if isinstance(obj, torch.Tensor) and t is obj else t


def _a(x):
    return x if isinstance(x, torch.Tensor) else asarray(x)


def _axis(axis):
    return tuple(axis) if isinstance(axis, list) else axis


def from_dlpack(x):
    return torch.from_dlpack(x)


# ---- creation
def _shape(shape):
    return (shape,) if isinstance(shape, int) else tuple(int(s) for s in shape)


def zeros(shape, dtype=None):
    return torch.zeros(_shape(shape), dtype=_dt(dtype) or float32)


def ones(shape, dtype=None):
    return torch.ones(_shape(shape), dtype=_dt(dtype) or float32)


def full(shape, fill_value, dtype=None):
    return torch.full(_shape(shape), fill_value, dtype=_dt(dtype) or (float32 if isinstance(fill_value, float) else None))


def zeros_like(x, dtype=None):
    return torch.zeros_like(_a(x), dtype=_dt(dtype))


def ones_like(x, dtype=None):
    return torch.ones_like(_a(x), dtype=_dt(dtype))


def full_like(x, fill_value, dtype=None):
    return torch.full_like(_a(x), fill_value, dtype=_dt(dtype))


def _count(v):
    # ``x.size`` is an element count in numpy and jax, a bound method on a torch tensor
    return v.__self__.numel() if callable(v) and isinstance(getattr(v, "__self__", None), torch.Tensor) else v


def arange(start, stop=None, step=1, dtype=None):
    start, stop = _count(start), _count(stop)
    if stop is None:
        start, stop = 0, start
    if dtype is None:
        dtype = float32 if builtins.any(isinstance(v, float) for v in (start, stop, step)) else int32
    return torch.arange(start, stop, step, dtype=_dt(dtype))


def linspace(start, stop, num=50, dtype=None):
    return torch.linspace(start, stop, num, dtype=_dt(dtype) or float32)


def eye(n, m=None, dtype=None):
    return torch.eye(n, n if m is None else m, dtype=_dt(dtype) or float32)


def hanning(n):
    return torch.hann_window(n, periodic=False, dtype=float32)


def hamming(n):
    return torch.hamming_window(n, periodic=False, dtype=float32)


def tril(x, k=0):
    return torch.tril(_a(x), diagonal=k)


def triu(x, k=0):
    return torch.triu(_a(x), diagonal=k)


# ---- reductions
def _reduce(fn):
    def f(x, axis=None, keepdims=False, dtype=None):
        x = _a(x)
        axis = _axis(axis)
        if axis == ():
            return x
        if x.dtype == torch.bool and fn in (torch.sum, torch.mean):
            x = x.to(int32)
        out = fn(x) if axis is None else fn(x, dim=axis, keepdim=keepdims)
        if axis is None and keepdims:
            out = out.reshape((1,) * x.dim())
        return out if dtype is None else out.to(_dt(dtype))
    return f


sum = _reduce(torch.sum)
mean = _reduce(torch.mean)
max = amax = _reduce(torch.amax)
min = amin = _reduce(torch.amin)
prod = _reduce(torch.prod)


def all(x, axis=None, keepdims=False):
    x = _a(x)
    return torch.all(x) if axis is None else torch.all(x, dim=axis, keepdim=keepdims)


def any(x, axis=None, keepdims=False):
    x = _a(x)
    return torch.any(x) if axis is None else torch.any(x, dim=axis, keepdim=keepdims)


def argmax(x, axis=None, keepdims=False):
    return torch.argmax(_a(x), dim=axis, keepdim=keepdims).to(int32)


def argmin(x, axis=None, keepdims=False):
    return torch.argmin(_a(x), dim=axis, keepdim=keepdims).to(int32)


def cumsum(x, axis=None):
    x = _a(x)
    return torch.cumsum(x.reshape(-1), 0) if axis is None else torch.cumsum(x, dim=axis)


def cumprod(x, axis=None):
    x = _a(x)
    return torch.cumprod(x.reshape(-1), 0) if axis is None else torch.cumprod(x, dim=axis)


def var(x, axis=None, keepdims=False, ddof=0):
    x = _a(x)
    return torch.var(x, dim=_axis(axis), keepdim=keepdims, correction=ddof)


def std(x, axis=None, keepdims=False, ddof=0):
    return torch.sqrt(var(x, axis, keepdims, ddof))


def logsumexp(x, axis=None, keepdims=False):
    x = _a(x)
    return torch.logsumexp(x, dim=tuple(range(x.dim())) if axis is None else axis, keepdim=keepdims)


# ---- shape
def reshape(x, shape, *more):
    shape = (shape,) + more if isinstance(shape, int) else tuple(shape)
    return _a(x).reshape(shape)


def transpose(x, axes=None):
    x = _a(x)
    return x.permute(*reversed(range(x.dim()))) if axes is None else x.permute(*axes)


def swapaxes(x, a, b):
    return torch.swapaxes(_a(x), a, b)


def moveaxis(x, source, destination):
    return torch.movedim(_a(x), source, destination)


def expand_dims(x, axis):
    x = _a(x)
    axes = (axis,) if isinstance(axis, int) else tuple(axis)
    rank = x.dim() + len(axes)
    for a in sorted(a % rank for a in axes):
        x = x.unsqueeze(a)
    return x


def squeeze(x, axis=None):
    x = _a(x)
    return x.squeeze() if axis is None else x.squeeze(_axis(axis))


def broadcast_to(x, shape):
    return torch.broadcast_to(_a(x), tuple(shape))


def stack(xs, axis=0):
    return torch.stack([_a(x) for x in xs], dim=axis)


def concatenate(xs, axis=0):
    return torch.cat([_a(x) for x in xs], dim=axis)


def split(x, indices_or_sections, axis=0):
    x = _a(x)
    if isinstance(indices_or_sections, int):
        if x.shape[axis] % indices_or_sections:
            raise ValueError("array split does not result in an equal division")
        return list(torch.tensor_split(x, indices_or_sections, dim=axis))
    return list(torch.tensor_split(x, [int(i) for i in indices_or_sections], dim=axis))


def array_split(x, indices_or_sections, axis=0):
    x = _a(x)
    if isinstance(indices_or_sections, int):
        return list(torch.tensor_split(x, indices_or_sections, dim=axis))
    return list(torch.tensor_split(x, [int(i) for i in indices_or_sections], dim=axis))


def flip(x, axis=None):
    x = _a(x)
    return torch.flip(x, dims=tuple(range(x.dim())) if axis is None else ((axis,) if isinstance(axis, int) else tuple(axis)))


def roll(x, shift, axis=None):
    return torch.roll(_a(x), shift, dims=axis)


def tile(x, reps):
    return torch.tile(_a(x), (reps,) if isinstance(reps, int) else tuple(reps))


def repeat(x, repeats, axis=None):
    return torch.repeat_interleave(_a(x), repeats, dim=axis)


def pad(x, pad_width, mode="constant", constant_values=0):
    x = _a(x)
    if isinstance(pad_width, int):
        pad_width = [(pad_width, pad_width)] * x.dim()
    elif isinstance(pad_width[0], int):
        pad_width = [tuple(pad_width)] * x.dim()
    flat = []
    for lo, hi in reversed(list(pad_width)):
        flat += [int(lo), int(hi)]
    if mode == "constant":
        return torch.nn.functional.pad(x, flat, mode="constant", value=constant_values)
    return torch.nn.functional.pad(x, flat, mode={"edge": "replicate", "reflect": "reflect", "wrap": "circular"}[mode])


def take(x, indices, axis=None):
    x = _a(x)
    idx = _a(indices).long()
    if axis is None:
        return x.reshape(-1)[idx]
    return torch.index_select(x, axis, idx.reshape(-1)).reshape(x.shape[:axis] + idx.shape + x.shape[axis % x.dim() + 1:])


def take_along_axis(x, indices, axis):
    return torch.take_along_dim(_a(x), _a(indices).long(), dim=axis)


def where(cond, x=None, y=None):
    cond = _a(cond)
    if x is None:
        return torch.where(cond)
    x, y = _a(x), _a(y)
    if x.dtype != y.dtype:
        dt = torch.promote_types(x.dtype, y.dtype)
        x, y = x.to(dt), y.to(dt)
    return torch.where(cond.bool(), x, y)


def clip(x, a_min=None, a_max=None, *, min=None, max=None):
    return torch.clamp(_a(x), a_min if min is None else min, a_max if max is None else max)


# ---- linear algebra
def matmul(a, b):
    return torch.matmul(_a(a), _a(b))


def dot(a, b):
    a, b = _a(a), _a(b)
    if a.dim() == 0 or b.dim() == 0:
        return a * b
    if b.dim() == 1:
        return torch.tensordot(a, b, dims=([-1], [0]))
    return torch.tensordot(a, b, dims=([-1], [-2]))


def outer(a, b):
    return torch.outer(_a(a).reshape(-1), _a(b).reshape(-1))


def einsum(eq, *xs):
    return torch.einsum(eq, *[_a(x) for x in xs])


def tensordot(a, b, axes=2):
    return torch.tensordot(_a(a), _a(b), dims=axes)


# ---- elementwise
def _binary(fn):
    def f(x, y):
        x = _a(x) if not isinstance(y, torch.Tensor) or isinstance(x, torch.Tensor) else torch.as_tensor(x, dtype=y.dtype)
        y = _a(y) if isinstance(y, torch.Tensor) else torch.as_tensor(y, dtype=x.dtype if x.dtype.is_floating_point or isinstance(y, (int, bool)) else float32)
        return fn(x, y)
    return f


add, subtract, multiply = _binary(torch.add), _binary(torch.sub), _binary(torch.mul)
divide = true_divide = _binary(torch.true_divide)
power = _binary(torch.pow)
maximum, minimum = _binary(torch.maximum), _binary(torch.minimum)
mod = remainder = _binary(torch.remainder)
floor_divide = _binary(torch.floor_divide)
equal, not_equal = _binary(torch.eq), _binary(torch.ne)
less, less_equal, greater, greater_equal = _binary(torch.lt), _binary(torch.le), _binary(torch.gt), _binary(torch.ge)
logical_and, logical_or, logical_xor = _binary(torch.logical_and), _binary(torch.logical_or), _binary(torch.logical_xor)
arctan2 = _binary(torch.atan2)


def logical_not(x):
    return torch.logical_not(_a(x))


def negative(x):
    return torch.neg(_a(x))


def square(x):
    return torch.square(_a(x))


def round(x, decimals=0):
    return torch.round(_a(x), decimals=decimals)


def allclose(a, b, rtol=1e-5, atol=1e-8):
    return bool(torch.allclose(_a(a).double(), _a(b).double(), rtol=rtol, atol=atol))


def isclose(a, b, rtol=1e-5, atol=1e-8):
    return torch.isclose(_a(a), _a(b), rtol=rtol, atol=atol)


def astype(x, dtype):
    return _a(x).to(_dt(dtype))


_ALIASES = {"arccos": "acos", "arcsin": "asin", "arctan": "atan", "arccosh": "acosh", "arcsinh": "asinh",
            "arctanh": "atanh", "absolute": "abs", "fabs": "abs"}


def __getattr__(name):
    """Everything else is elementwise and has the same name in torch (sin, exp, log1p, isnan, ...)."""
    fn = getattr(torch, _ALIASES.get(name, name), None)
    if fn is None or not callable(fn):
        raise AttributeError(f"jax.numpy stand-in has no function {name!r}")

    def f(x, *args, **kwargs):
        return fn(_a(x), *[a if not isinstance(a, (list, _np.ndarray)) else _a(a) for a in args], **kwargs)

    f.__name__ = name
    return f


# ---- methods that jax arrays have and torch tensors lack
class _At:
    def __init__(self, x):
        self.x = x

    def __getitem__(self, idx):
        return _AtIndex(self.x, idx)


def _index(idx):
    def one(i):
        if isinstance(i, torch.Tensor) and i.dtype not in (torch.bool, torch.int64):
            return i.long()
        if isinstance(i, (list, _np.ndarray)):
            return torch.as_tensor(_np.asarray(i)).long()
        return i
    return tuple(one(i) for i in idx) if isinstance(idx, tuple) else one(idx)


class _AtIndex:
    def __init__(self, x, idx):
        self.x, self.idx = x, _index(idx)

    def _value(self, v):
        return v.to(self.x.dtype) if isinstance(v, torch.Tensor) else v

    def set(self, v):
        out = self.x.clone()
        out[self.idx] = self._value(v)
        return out

    def add(self, v):
        out = self.x.clone()
        v = self._value(v)
        idx = self.idx if isinstance(self.idx, tuple) else (self.idx,)
        if builtins.any(isinstance(i, torch.Tensor) for i in idx):
            tgt = out[self.idx]
            out.index_put_(tuple(i for i in idx), torch.broadcast_to(torch.as_tensor(v, dtype=out.dtype), tgt.shape),
                           accumulate=True) if builtins.all(isinstance(i, torch.Tensor) for i in idx) else out.__setitem__(self.idx, tgt + v)
        else:
            out[self.idx] = out[self.idx] + v
        return out

    def multiply(self, v):
        out = self.x.clone()
        out[self.idx] = out[self.idx] * self._value(v)
        return out

    def get(self):
        return self.x[self.idx]


def _install_array_methods():
    T = torch.Tensor
    if not hasattr(T, "astype"):
        T.astype = lambda self, dtype: self.to(_dt(dtype))
    if not hasattr(T, "at"):
        T.at = property(lambda self: _At(self))
    if not hasattr(T, "block_until_ready"):
        T.block_until_ready = lambda self: self
    _orig_getitem = T.__getitem__

    def getitem(self, idx):
        # jax accepts int32 index arrays; torch wants int64
        if isinstance(idx, torch.Tensor) and idx.dtype in (torch.int32, torch.int16, torch.int8):
            idx = idx.long()
        elif isinstance(idx, tuple) and builtins.any(isinstance(i, torch.Tensor) and i.dtype == torch.int32 for i in idx):
            idx = tuple(i.long() if isinstance(i, torch.Tensor) and i.dtype == torch.int32 else i for i in idx)
        return _orig_getitem(self, idx)

    if not getattr(T, "_jax_standin_getitem", False):
        T.__getitem__ = getitem
        T._jax_standin_getitem = True
        # ``np.max(a)`` on a non-ndarray calls ``a.max(axis=None, out=None)``: accept numpy's keywords
        for name, fn in (("max", amax), ("min", amin), ("sum", sum), ("mean", mean), ("prod", prod),
                         ("any", any), ("all", all)):
            setattr(T, name, _numpy_keywords(getattr(T, name), fn))
        for name in ("__radd__", "__rsub__", "__rmul__", "__rtruediv__"):
            setattr(T, name, _reflected(getattr(T, name)))


def _reflected(orig):
    """``ndarray - tensor`` ends in ``tensor.__rsub__(ndarray)`` (torch outranks numpy): take the array."""
    def method(self, other):
        return orig(self, asarray(other) if isinstance(other, _np.ndarray) else other)

    method.__name__ = orig.__name__
    return method


def _numpy_keywords(orig, np_style):
    def method(self, *args, **kwargs):
        if "axis" in kwargs or "out" in kwargs or "keepdims" in kwargs:
            kwargs.pop("out", None)
            kwargs.pop("dtype", None)
            return np_style(self, *args, **kwargs)
        return orig(self, *args, **kwargs)

    method.__name__ = orig.__name__
    return method


_install_array_methods()
