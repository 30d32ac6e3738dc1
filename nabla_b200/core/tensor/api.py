"""User-facing ``Tensor`` (reference: nabla/core/tensor/api.py:48-1521).

A thin facade over ``TensorImpl``. Operations never run here: methods forward to
``nabla_b200.ops`` functions which create promise tensors; data is produced by
``realize()`` / ``realize_all()`` through the graph engine.
"""
from __future__ import annotations

from types import EllipsisType
from typing import Any, Sequence

import numpy as np
import torch

from ...types import CPU, Accelerator, Device, DType, Shape, as_device, as_dtype
from .impl import TensorImpl
from ..common.context import default_device, default_dtype, defaults, defaults_like  # noqa: F401  (re-exported as in the reference)


class Tensor:
    """Multi-dimensional array with lazy evaluation, autodiff hooks and sharding metadata."""

    __slots__ = ("_impl", "__weakref__")
    __array_priority__ = 1000

    def __init__(self, *, buffers=None, value=None, impl: TensorImpl | None = None, is_traced: bool = False):
        if impl is None:
            if buffers is None:
                buffers = value          # the reference's second spelling (a backend value; here a device buffer)
            if buffers is None:
                raise ValueError("Tensor needs `buffers` or `impl`")
            impl = TensorImpl(buffers, is_traced=is_traced)
        self._impl = impl

    # ------------------------------------------------------------ raw state
    @property
    def _buffers(self):
        return self._impl._buffers

    @property
    def buffers(self) -> torch.Tensor | None:
        return self._impl.primary_buffer()

    @property
    def real(self) -> bool:
        return self._impl.is_realized

    # ---- the reference's accessors of the backing storage (nabla/core/tensor/api.py:95-160, 431-439,
    # 617-674). There the storage is a MAX driver buffer or a value of the graph being built; here it
    # is the list of torch tensors of the locally held shards.
    @property
    def driver_tensor(self) -> torch.Tensor:
        if (b := self.buffers) is None:
            raise TypeError("Can't get driver tensor for symbolic tensor")
        return b

    @property
    def values(self) -> list[torch.Tensor]:
        """The locally held shards (realizes the tensor first)."""
        self.hydrate()
        return list(self._impl._buffers)

    @property
    def type(self):
        """(shape, dtype, device) of the global tensor."""
        return tuple(int(d) for d in self._impl.global_shape), self._impl.dtype, self._impl.device

    def hydrate(self) -> "Tensor":
        """Make the data available: realize a promise, leave a realized tensor alone."""
        if not self._impl.is_realized:
            self.realize()
        return self

    @classmethod
    def _create_unsafe(cls, **kwargs: Any) -> "Tensor":
        """Tensor straight from ``TensorImpl`` arguments (no validation)."""
        return cls(impl=TensorImpl(**kwargs))

    @property
    def is_realized(self) -> bool:
        return self._impl.is_realized

    @property
    def is_traced(self) -> bool:
        return self._impl.is_traced

    @is_traced.setter
    def is_traced(self, v: bool) -> None:
        self._impl.is_traced = bool(v)

    @property
    def batch_dims(self) -> int:
        return self._impl.batch_dims

    @batch_dims.setter
    def batch_dims(self, v: int) -> None:
        self._impl.batch_dims = int(v)

    @property
    def op_kwargs(self) -> dict:
        n = self._impl.output_refs
        return dict(n.op_kwargs) if n is not None else {}

    def trace(self) -> "Tensor":
        """Mark this tensor as traced for autograd and return it (reference: api.py:247-250)."""
        self._impl.is_traced = True
        return self

    # ------------------------------------------------------------ autograd flags
    @property
    def requires_grad(self) -> bool:
        return self._impl.requires_grad

    @requires_grad.setter
    def requires_grad(self, v: bool) -> None:
        self._impl.requires_grad = bool(v)
        if v:
            self._impl.is_traced = True

    def requires_grad_(self, value: bool = True) -> "Tensor":
        self.requires_grad = value
        return self

    @property
    def is_leaf(self) -> bool:
        return self._impl.output_refs is None

    def detach(self) -> "Tensor":
        """A tensor sharing this one's data, cut off from the autodiff trace."""
        self.realize()
        impl = TensorImpl(list(self._impl._buffers), shape=self._impl._shape, dtype=self._impl.dtype,
                          device=self._impl.device, sharding=self._impl.sharding, batch_dims=self._impl.batch_dims)
        return Tensor(impl=impl)

    @property
    def grad(self):
        return self._impl.grad

    @grad.setter
    def grad(self, v) -> None:
        self._impl.grad = v

    def backward(self, gradient: "Tensor | None" = None, retain_graph: bool = False, create_graph: bool = False) -> None:
        from ..autograd.backward import backward

        backward(self, gradient, retain_graph=retain_graph, create_graph=create_graph)

    @property
    def tangent(self):
        return self._impl.tangent

    @tangent.setter
    def tangent(self, v) -> None:
        self._impl.tangent = v

    @property
    def dual(self):
        return self._impl.dual

    @dual.setter
    def dual(self, v) -> None:
        self._impl.dual = v

    # ------------------------------------------------------------ sharding
    def shard(self, mesh, dim_specs, replicated_axes=None, partial_sum_axes=None) -> "Tensor":
        from ...ops.communication import shard

        return shard(self, mesh, dim_specs, replicated_axes=replicated_axes, partial_sum_axes=partial_sum_axes)

    def with_sharding(self, mesh, dim_specs, replicated_axes=None) -> "Tensor":
        return self.shard(mesh, dim_specs, replicated_axes=replicated_axes)

    def with_sharding_constraint(self, mesh, dim_specs, replicated_axes=None) -> "Tensor":
        from ..sharding.spec import DimSpec, ShardingSpec

        self._impl.sharding_constraint = ShardingSpec(mesh, [DimSpec.from_raw(d) for d in dim_specs],
                                                      replicated_axes=set(replicated_axes or ()))
        return self

    @property
    def sharding(self):
        return self._impl.sharding

    @sharding.setter
    def sharding(self, v) -> None:
        self._impl.sharding = v

    @property
    def is_sharded(self) -> bool:
        return self._impl.sharding is not None

    @property
    def num_shards(self) -> int:
        return self._impl.num_shards

    # ------------------------------------------------------------ shapes
    @property
    def shape(self) -> Shape:
        """Global logical shape."""
        return Shape(self._impl.global_shape)

    @property
    def global_shape(self) -> Shape:
        """Global shape INCLUDING the leading vmap dims, as in the reference
        (nabla/core/tensor/api.py:416-418); ``shape`` is the logical one."""
        return Shape(self._impl.physical_global_shape)

    @property
    def local_shape(self) -> Shape:
        """Shape of shard 0 including the leading vmap dims (reference: api.py:411-413)."""
        return Shape(self._impl.physical_local_shape(0))

    @property
    def batch_shape(self) -> Shape:
        return Shape(self._impl.batch_shape)

    @property
    def physical_shape(self) -> Shape:
        return Shape(self._impl.physical_local_shape(0))

    @property
    def physical_global_shape(self) -> Shape:
        return Shape(self._impl.physical_global_shape)

    @property
    def global_shape_ints(self) -> tuple[int, ...]:
        return self._impl.global_shape

    @property
    def physical_global_shape_ints(self) -> tuple[int, ...]:
        return self._impl.physical_global_shape

    def physical_local_shape(self, shard_idx: int = 0) -> Shape:
        return Shape(self._impl.physical_local_shape(shard_idx))

    def physical_local_shape_ints(self, shard_idx: int = 0) -> tuple[int, ...]:
        return self._impl.physical_local_shape(shard_idx)

    def logical_local_shape(self, shard_idx: int = 0) -> Shape:
        return Shape(self._impl.logical_local_shape(shard_idx))

    def shard_shape(self, shard_idx: int = 0) -> Shape:
        return Shape(self._impl.logical_local_shape(shard_idx))

    @property
    def rank(self) -> int:
        return len(self._impl.global_shape)

    ndim = rank

    def dim(self) -> int:
        return self.rank

    def size(self, dim: int | None = None):
        s = self._impl.global_shape
        return Shape(s) if dim is None else s[dim]

    @property
    def dtype(self) -> DType:
        return self._impl.dtype

    @property
    def device(self) -> Device:
        return self._impl.device

    def num_elements(self) -> int:
        n = 1
        for d in self._impl.global_shape:
            n *= d
        return n

    numel = num_elements

    def __len__(self) -> int:
        s = self._impl.global_shape
        if not s:
            raise TypeError("len() of a 0-d tensor")
        return s[0]

    # ------------------------------------------------------------ factories
    @classmethod
    def from_dlpack(cls, array: Any) -> "Tensor":
        if isinstance(array, Tensor):
            return array
        if isinstance(array, torch.Tensor):
            t = array
        elif isinstance(array, np.ndarray):
            # np.ascontiguousarray promotes a 0-d array to 1-d: restore the shape
            t = torch.from_numpy(np.ascontiguousarray(array)).reshape(array.shape)
        else:
            t = torch.from_dlpack(array)
        return cls(buffers=[t])

    @classmethod
    def from_torch(cls, t: torch.Tensor) -> "Tensor":
        return cls(buffers=[t])

    @classmethod
    def from_graph_value(cls, value) -> "Tensor":
        """Wrap a value of the execution backend. The reference wraps a node of the MAX graph under
        construction (nabla/core/tensor/api.py:431-434); the values this engine computes with are
        device buffers, so that is what is accepted here."""
        if not isinstance(value, torch.Tensor):
            raise TypeError(f"{value=} must be a tensor or buffer value")
        return cls(buffers=[value])

    @classmethod
    def constant(cls, value, *, dtype=None, device=None) -> "Tensor":
        from ...ops.creation import constant

        return constant(value, dtype=dtype, device=device)

    @classmethod
    def full(cls, shape, value, *, dtype=None, device=None, is_traced: bool = False) -> "Tensor":
        from ...ops.creation import full

        return full(shape, value, dtype=dtype, device=device, is_traced=is_traced)

    @classmethod
    def zeros(cls, shape, *, dtype=None, device=None, is_traced: bool = False) -> "Tensor":
        from ...ops.creation import zeros

        return zeros(shape, dtype=dtype, device=device, is_traced=is_traced)

    @classmethod
    def ones(cls, shape, *, dtype=None, device=None, is_traced: bool = False) -> "Tensor":
        from ...ops.creation import ones

        return ones(shape, dtype=dtype, device=device, is_traced=is_traced)

    @classmethod
    def arange(cls, start=0, stop=None, step=1, *, dtype=None, device=None) -> "Tensor":
        from ...ops.creation import arange

        return arange(start, stop, step, dtype=dtype, device=device)

    @classmethod
    def uniform(cls, shape=(), low=0.0, high=1.0, *, dtype=None, device=None, range=None) -> "Tensor":
        """U(low, high) samples (reference: nabla/core/tensor/api.py:587-598); ``range=(low, high)`` is
        accepted as well."""
        from ...ops.creation import uniform

        if range is not None:
            low, high = range
        elif isinstance(low, (tuple, list)):
            low, high = low
        return uniform(shape, low, high, dtype=dtype, device=device)

    @classmethod
    def gaussian(cls, shape=(), mean=0.0, std=1.0, *, dtype=None, device=None) -> "Tensor":
        from ...ops.creation import gaussian

        return gaussian(shape, mean, std, dtype=dtype, device=device)

    normal = gaussian

    def new_zeros(self, shape, *, dtype=None, device=None) -> "Tensor":
        return Tensor.zeros(shape, dtype=dtype or self.dtype, device=device or self.device)

    def new_ones(self, shape, *, dtype=None, device=None) -> "Tensor":
        return Tensor.ones(shape, dtype=dtype or self.dtype, device=device or self.device)

    def new_full(self, shape, fill_value, *, dtype=None, device=None) -> "Tensor":
        return Tensor.full(shape, fill_value, dtype=dtype or self.dtype, device=device or self.device)

    def new_empty(self, shape, *, dtype=None, device=None) -> "Tensor":
        return self.new_zeros(shape, dtype=dtype, device=device)

    # ------------------------------------------------------------ realization / transfer
    def realize(self) -> "Tensor":
        if not self._impl.is_realized:
            from ..graph.engine import GRAPH

            GRAPH.evaluate(self)
        return self

    def gather(self) -> "Tensor":
        """Resolve pending partial sums and replicate: the result holds the full data."""
        if self._impl.sharding is None:
            return self
        from ...ops.communication import all_reduce, gather_all_axes

        t = self
        if t._impl.sharding.partial_sum_axes:
            t = all_reduce(t, reduce_axes=set(t._impl.sharding.partial_sum_axes))
        if any(d.axes for d in t._impl.sharding.dim_specs):
            t = gather_all_axes(t)
        return t

    def to_torch(self) -> torch.Tensor:
        """The full (gathered) data as a torch tensor on its current device."""
        t = self.gather()
        t.realize()
        return t._impl._buffers[0]

    def to(self, target) -> "Tensor":
        """``to(device)`` moves; ``to(dtype)`` casts."""
        if isinstance(target, (DType, torch.dtype)) or target in (float, int, bool):
            from ...ops.unary import cast

            return cast(self, as_dtype(target))
        from ...ops.communication import to_device

        return to_device(self, as_device(target))

    def cpu(self) -> "Tensor":
        return self.to(CPU())

    def cuda(self, device: int | Device = 0) -> "Tensor":
        return self.to(device if isinstance(device, Device) else Accelerator(int(device)))

    gpu = cuda

    def type_as(self, other: "Tensor") -> "Tensor":
        return self.to(other.dtype)

    def to_numpy(self) -> np.ndarray:
        b = self.to_torch().detach()
        if b.dtype == torch.bfloat16:
            b = b.float()
        return b.cpu().numpy()

    numpy = to_numpy

    @staticmethod
    def to_numpy_all(*tensors: "Tensor") -> tuple[np.ndarray, ...]:
        """Realize all tensors in one batch, then convert."""
        gathered = [t.gather() for t in tensors]
        realize_all(*gathered)
        return tuple(t.to_numpy() for t in gathered)

    def item(self):
        if self.num_elements() != 1:
            raise TypeError("Only single-element tensors can be converted to Python scalars")
        return self.to_torch().reshape(()).item()

    def tolist(self):
        return self.to_numpy().tolist()

    def __array__(self, dtype=None, copy=None):
        a = self.to_numpy()
        return a.astype(dtype) if dtype is not None else a

    def __dlpack__(self, stream=None, **kw):
        return self.to_torch().__dlpack__()

    def __dlpack_device__(self):
        return self.to_torch().__dlpack_device__()

    def __bool__(self) -> bool:
        return bool(self.item())

    def __float__(self) -> float:
        return float(self.item())

    def __int__(self) -> int:
        return int(self.item())

    def __hash__(self) -> int:
        return id(self)

    def __deepcopy__(self, memo) -> "Tensor":
        return self

    def __repr__(self) -> str:
        self.realize()
        content = self._impl.format_metadata(include_data=True)
        if "\n" in content:
            body = "\n".join("  " + l for l in content.split("\n"))
            return f"Tensor(\n{body}\n)"
        return f"Tensor({content})"

    __str__ = __repr__

    def __rich_repr__(self):
        yield "shape", self.shape
        yield "dtype", self.dtype
        yield "device", self.device

    # ------------------------------------------------------------ view helpers (PyTorch-style)
    def reshape(self, *shape) -> "Tensor":
        from ...ops.view import reshape

        return reshape(self, _shape_arg(shape))

    view = reshape

    def squeeze(self, axis=None) -> "Tensor":
        from ...ops.view import squeeze

        if axis is None:
            axis = tuple(i for i, d in enumerate(self._impl.global_shape) if d == 1)
        return squeeze(self, axis=axis)

    def unsqueeze(self, axis: int) -> "Tensor":
        from ...ops.view import unsqueeze

        return unsqueeze(self, axis=axis)

    def swap_axes(self, axis1: int, axis2: int) -> "Tensor":
        from ...ops.view import swap_axes

        return swap_axes(self, axis1, axis2)

    transpose = swap_axes

    def permute(self, *order) -> "Tensor":
        from ...ops.view import permute

        return permute(self, _shape_arg(order))

    def flatten(self, start_dim: int = 0, end_dim: int = -1) -> "Tensor":
        from ...ops.view import flatten

        return flatten(self, start_dim, end_dim)

    def broadcast_to(self, *shape) -> "Tensor":
        from ...ops.view import broadcast_to

        return broadcast_to(self, _shape_arg(shape))

    def expand(self, *shape) -> "Tensor":
        shape = list(_shape_arg(shape))
        cur = self._impl.global_shape
        off = len(shape) - len(cur)
        for i, s in enumerate(shape):
            if s == -1:
                shape[i] = cur[i - off]
        return self.broadcast_to(tuple(shape))

    def flip(self, axis) -> "Tensor":
        from ...ops.view import flip

        return flip(self, axis)

    @property
    def T(self) -> "Tensor":
        if self.rank < 2:
            return self
        return self.swap_axes(-2, -1)

    def gelu(self, approximate: str = "none") -> "Tensor":
        from ...ops.unary import gelu

        return gelu(self, approximate=approximate)

    def cast(self, dtype) -> "Tensor":
        from ...ops.unary import cast

        return cast(self, as_dtype(dtype))

    def softmax(self, axis: int = -1) -> "Tensor":
        from ...ops.unary import softmax

        return softmax(self, axis=axis)

    def logsoftmax(self, axis: int = -1) -> "Tensor":
        from ...ops.unary import logsoftmax

        return logsoftmax(self, axis=axis)

    def sum(self, axis=None, keepdims: bool = False) -> "Tensor":
        from ...ops.reduction import reduce_sum

        return reduce_sum(self, axis=axis, keepdims=keepdims)

    def mean(self, axis=None, keepdims: bool = False) -> "Tensor":
        from ...ops.reduction import mean

        return mean(self, axis=axis, keepdims=keepdims)

    def max(self, axis=None, keepdims: bool = False) -> "Tensor":
        from ...ops.reduction import reduce_max

        return reduce_max(self, axis=axis, keepdims=keepdims)

    def min(self, axis=None, keepdims: bool = False) -> "Tensor":
        from ...ops.reduction import reduce_min

        return reduce_min(self, axis=axis, keepdims=keepdims)

    def argmax(self, axis: int = -1, keepdims: bool = False) -> "Tensor":
        from ...ops.reduction import argmax

        return argmax(self, axis=axis, keepdims=keepdims)

    def argmin(self, axis: int = -1, keepdims: bool = False) -> "Tensor":
        from ...ops.reduction import argmin

        return argmin(self, axis=axis, keepdims=keepdims)

    def cumsum(self, axis: int = -1, exclusive: bool = False, reverse: bool = False) -> "Tensor":
        from ...ops.reduction import cumsum

        return cumsum(self, axis=axis, exclusive=exclusive, reverse=reverse)

    # ------------------------------------------------------------ indexing
    def __getitem__(self, key) -> "Tensor":
        from ...ops import view

        if isinstance(key, Tensor):
            return view.gather(self, key, axis=0)
        start, size, squeeze_axes = _parse_basic_index(self, key)
        res = view.slice_tensor(self, start=tuple(start), size=tuple(size))
        if squeeze_axes:
            res = view.squeeze(res, axis=tuple(squeeze_axes))
        return res

    def __setitem__(self, key, value) -> None:
        updated = _apply_indexed_update(self, key, value, mode="set", inplace=True)
        self._impl = updated._impl

    @property
    def at(self) -> "_TensorAtAccessor":
        return _TensorAtAccessor(self)

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]

    def __pos__(self) -> "Tensor":
        return self

    def __invert__(self) -> "Tensor":
        if self.dtype is DType.bool:
            from ...ops.comparison import logical_not

            return logical_not(self)
        raise NotImplementedError("__invert__ is only supported on bool tensors")


class _TensorAtAccessor:
    def __init__(self, t: Tensor):
        self._t = t

    def __getitem__(self, key) -> "_TensorAtIndexer":
        return _TensorAtIndexer(self._t, key)


class _TensorAtIndexer:
    def __init__(self, t: Tensor, key):
        self._t, self._key = t, key

    def set(self, value) -> Tensor:
        return _apply_indexed_update(self._t, self._key, value, mode="set")

    def add(self, value) -> Tensor:
        return _apply_indexed_update(self._t, self._key, value, mode="add")


def _shape_arg(args) -> tuple[int, ...]:
    if len(args) == 1 and isinstance(args[0], (tuple, list, Shape)):
        args = args[0]
    return tuple(int(a) for a in args)


def _parse_basic_index(x: Tensor, key) -> tuple[list[int], list[int], list[int]]:
    shape = x._impl.global_shape
    if not isinstance(key, tuple):
        key = (key,)
    if any(k is Ellipsis for k in key):
        if sum(1 for k in key if k is Ellipsis) > 1:
            raise ValueError("An index can only have a single ellipsis ('...')")
        i = [j for j, k in enumerate(key) if k is Ellipsis][0]
        key = key[:i] + (slice(None),) * max(0, len(shape) - (len(key) - 1)) + key[i + 1:]
    if len(key) > len(shape):
        raise IndexError(f"too many indices for tensor of rank {len(shape)}")
    start, size, squeeze_axes = [], [], []
    for i, k in enumerate(key):
        n = shape[i]
        if isinstance(k, (int, np.integer)):
            idx = int(k) + n if k < 0 else int(k)
            if not 0 <= idx < n:
                raise IndexError(f"index {k} is out of bounds for axis {i} with size {n}")
            start.append(idx)
            size.append(1)
            squeeze_axes.append(i)
        elif isinstance(k, slice):
            if k.step not in (None, 1):
                raise NotImplementedError("Slicing with step != 1 is not yet supported.")
            s0 = 0 if k.start is None else (k.start + n if k.start < 0 else k.start)
            s1 = n if k.stop is None else (k.stop + n if k.stop < 0 else k.stop)
            s0 = max(0, min(n, s0))
            s1 = max(0, min(n, s1))
            start.append(s0)
            size.append(max(0, s1 - s0))
        else:
            raise TypeError(f"Invalid index type: {type(k)}")
    for i in range(len(start), len(shape)):
        start.append(0)
        size.append(shape[i])
    return start, size, squeeze_axes


def _ensure_like(value, like: Tensor) -> Tensor:
    if isinstance(value, Tensor):
        return value
    from ...ops.creation import constant

    return constant(value, dtype=like.dtype, device=like.device)


def _apply_indexed_update(x: Tensor, key, value, *, mode: str, inplace: bool = False) -> Tensor:
    from ...ops import view

    if isinstance(key, Tensor):
        updates = _ensure_like(value, x)
        tgt = tuple(key._impl.global_shape) + tuple(x._impl.global_shape[1:])
        if tuple(updates._impl.global_shape) != tgt:
            updates = view.broadcast_to(updates, tgt)
        if mode == "add":
            updates = view.gather(x, key, axis=0) + updates
        return view.scatter(x, key, updates, axis=0)
    start, size, squeeze_axes = _parse_basic_index(x, key)
    updates = _ensure_like(value, x)
    if tuple(updates._impl.global_shape) != tuple(size):
        # integer-indexed axes were squeezed away by the user: put them back
        ush = tuple(updates._impl.global_shape)
        kept = tuple(s for i, s in enumerate(size) if i not in squeeze_axes)
        if squeeze_axes and len(ush) <= len(kept):
            updates = view.broadcast_to(updates, kept) if ush != kept else updates
            updates = view.reshape(updates, tuple(size))
        else:
            updates = view.broadcast_to(updates, tuple(size))
    if mode == "add":
        updates = view.slice_tensor(x, start=tuple(start), size=tuple(size)) + updates
    elif mode != "set":
        raise ValueError(f"Unsupported indexed update mode: {mode}")
    return view.slice_update(x, updates, start=tuple(start), size=tuple(size), use_buffer_ops=inplace)


def realize_all(*tensors: Tensor) -> tuple[Tensor, ...]:
    """Realize several tensors with a single graph evaluation (no-op while tracing for compile)."""
    from ... import config

    flat = [t for t in tensors if isinstance(t, Tensor)]
    if config.get_flag("TRACING"):
        return tuple(tensors)
    pending = [t for t in flat if not t._impl.is_realized]
    if pending:
        from ..graph.engine import GRAPH

        GRAPH.evaluate(*pending)
    return tuple(tensors)


# ---------------------------------------------------------------- operator methods
def _install_operators() -> None:
    def binary(name: str, fn_name: str, module: str, reflected: bool = False):
        def method(self, other):
            import importlib

            fn = getattr(importlib.import_module(module, __package__), fn_name)
            if not isinstance(other, (Tensor, int, float, bool, np.ndarray, np.generic, torch.Tensor)):
                return NotImplemented
            return fn(other, self) if reflected else fn(self, other)

        method.__name__ = name
        setattr(Tensor, name, method)

    B, C = "...ops.binary", "...ops.comparison"
    for name, fn in (("add", "add"), ("sub", "sub"), ("mul", "mul"), ("truediv", "div"), ("matmul", "matmul"),
                     ("pow", "pow"), ("mod", "mod")):
        binary(f"__{name}__", fn, B)
        binary(f"__r{name}__", fn, B, reflected=True)
    for name, fn in (("eq", "equal"), ("ne", "not_equal"), ("lt", "less"), ("le", "less_equal"), ("gt", "greater"),
                     ("ge", "greater_equal"), ("and", "logical_and"), ("or", "logical_or"), ("xor", "logical_xor")):
        binary(f"__{name}__", fn, C)

    def unary(name: str, fn_name: str):
        def method(self):
            from ...ops import unary as U

            return getattr(U, fn_name)(self)

        method.__name__ = name
        setattr(Tensor, name, method)

    unary("__neg__", "neg")
    unary("__abs__", "abs")
    for n in ("abs", "exp", "log", "relu", "sigmoid", "sqrt", "tanh", "acos", "atanh", "cos", "erf", "floor",
              "is_inf", "is_nan", "log1p", "rsqrt", "silu", "sin", "trunc", "round", "neg"):
        unary(n, n)


_install_operators()


def __getattr__(name: str):
    # `GRAPH` is importable from here as in the reference (nabla/core/tensor/api.py:44); resolved
    # lazily because the engine module imports this one
    if name == "GRAPH":
        from ..graph.engine import GRAPH

        return GRAPH
    raise AttributeError(name)
