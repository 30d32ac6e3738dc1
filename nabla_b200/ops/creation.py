"""Creation ops (reference: nabla/ops/creation.py:31-663).

``constant`` wraps host data eagerly. ``full/zeros/ones/arange/uniform/gaussian/hann_window``
are lazy ops without tensor inputs. Random ops take ``(seed, counter)`` from the engine at
execution time and derive an independent stream per shard, so replays of a cached plan draw
fresh numbers and shards never repeat each other.
"""
from __future__ import annotations

import numpy as np
import torch

from ..core.common.context import defaults
from ..core.tensor.api import Tensor
from ..types import DType, Shape, as_device, as_dtype
from .base import CreationOperation, Operation, ensure_tensor


def _shape(shape) -> tuple[int, ...]:
    if isinstance(shape, (int, np.integer)):
        return (int(shape),)
    return tuple(int(d) for d in shape)


def constant(value, *, dtype=None, device=None) -> Tensor:
    """A realized tensor holding ``value`` (scalar, nested list, numpy array, torch tensor)."""
    if isinstance(value, Tensor):
        return value
    if isinstance(value, torch.Tensor):
        t = value
    else:
        arr = np.asarray(value)
        if dtype is None and arr.dtype == np.float64:
            arr = arr.astype(np.float32)
        # np.ascontiguousarray promotes a 0-d array to 1-d: restore the shape
        t = torch.from_numpy(np.ascontiguousarray(arr)).reshape(arr.shape)
    dt, dev = defaults(dtype if dtype is not None else DType.from_torch(t.dtype), device)
    t = t.to(device=dev.to_torch(), dtype=dt.to_torch())
    return Tensor(buffers=[t])


class _LocalShapeMixin:
    """Creation ops on a mesh: each shard builds its local piece."""

    def shard_kwargs(self, kwargs, node, shard_idx, device_id):
        out_impl = node.outputs()[0]
        if out_impl is None or out_impl.sharding is None:
            return kwargs
        from ..core.sharding.spec import compute_local_shape, shard_salt

        kw = dict(kwargs)
        kw["shape"] = compute_local_shape(out_impl._shape, out_impl.sharding, device_id)
        kw["_shard"] = shard_salt(out_impl.sharding, device_id)
        return kw


class FullOp(_LocalShapeMixin, CreationOperation):
    def kernel(self, *, shape, value, dtype: DType, device, _shard: int = 0):
        return torch.full(shape, value, dtype=dtype.to_torch(), device=_dev(device))

    def meta_kwargs(self, kwargs):
        return {**kwargs, "device": "meta"}


class ArangeOp(CreationOperation):
    def kernel(self, *, start, stop, step, dtype: DType, device):
        return torch.arange(start, stop, step, dtype=dtype.to_torch(), device=_dev(device))

    def meta_kwargs(self, kwargs):
        return {**kwargs, "device": "meta"}


def _dev(device):
    if isinstance(device, str):
        return torch.device(device)
    return as_device(device).to_torch()


def _generator(device: torch.device, seed: int, counter: int, shard: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((seed * 0x9E3779B97F4A7C15 + counter * 0xD1B54A32D192ED03 + shard * 0x94D049BB133111EB + 1)
                  & 0x7FFFFFFFFFFFFFFF)
    return g


class _RandomOp(_LocalShapeMixin, CreationOperation):
    def meta_kwargs(self, kwargs):
        return {**kwargs, "device": "meta"}

    def execute(self, node):
        from ..core.graph.engine import GRAPH

        self._rng = GRAPH.next_rng()
        return super().execute(node)

    def _gen(self, device, shard):
        if device.type == "meta":
            return None
        seed, counter = getattr(self, "_rng", (0, 0))
        return _generator(device, seed, counter, shard)


def _native_rng(d: torch.device, shape, dtype: DType, shard: int, mode: str, a: float, b: float):
    """Philox kernel on this device's own stream (``native.kernels.rng_state``); None when the
    device is not a GPU or the library is missing."""
    if d.type != "cuda":
        return None
    from ..native import kernels

    if not kernels.has("nb_rng_dev"):
        return None
    td = dtype.to_torch()
    out = kernels.rng_dev(tuple(int(x) for x in shape), td if td in (torch.float32, torch.bfloat16) else torch.float32,
                          d, shard, mode, a, b)
    return out if out.dtype == td else out.to(td)


class UniformOp(_RandomOp):
    def kernel(self, *, shape, low, high, dtype: DType, device, _shard: int = 0):
        d = _dev(device)
        nat = _native_rng(d, shape, dtype, _shard, "uniform", low, high)
        if nat is not None:
            return nat
        g = self._gen(d, _shard)
        u = torch.rand(shape, dtype=torch.float32, device=d, generator=g)
        return (u * (high - low) + low).to(dtype.to_torch())


class GaussianOp(_RandomOp):
    def kernel(self, *, shape, mean, std, dtype: DType, device, _shard: int = 0):
        d = _dev(device)
        nat = _native_rng(d, shape, dtype, _shard, "gaussian", mean, std)
        if nat is not None:
            return nat
        g = self._gen(d, _shard)
        n = torch.randn(shape, dtype=torch.float32, device=d, generator=g)
        return (n * std + mean).to(dtype.to_torch())


class HannWindowOp(CreationOperation):
    def kernel(self, *, window_length, periodic, dtype: DType, device):
        return torch.hann_window(window_length, periodic=periodic, dtype=dtype.to_torch(), device=_dev(device))

    def meta_kwargs(self, kwargs):
        return {**kwargs, "device": "meta"}


class _BandOp(Operation):
    partial_policy = "any"
    upper = True

    def kernel(self, x, *, k: int = 0):
        return torch.triu(x, diagonal=k) if self.upper else torch.tril(x, diagonal=k)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        from ..core.sharding.propagation import OpShardingRule

        rank = len(input_shapes[0])
        m = {i: [f"d{i}"] if i < rank - 2 else [f"bcast_band{i}"] for i in range(rank)}
        return OpShardingRule([dict(m)], [dict(m)])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (type(self)._inst(cot, **kwargs),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return type(self)._inst(tangents[0], **kwargs)


class TriuOp(_BandOp):
    upper = True


class TrilOp(_BandOp):
    upper = False


class ZerosOp(FullOp):
    """`full` with the value fixed to 0 (reference: nabla/ops/creation.py:66)."""

    def kernel(self, *, shape, dtype: DType, device, value=0, _shard: int = 0):
        return super().kernel(shape=shape, value=0, dtype=dtype, device=device, _shard=_shard)


class OnesOp(FullOp):
    """`full` with the value fixed to 1 (reference: nabla/ops/creation.py:81)."""

    def kernel(self, *, shape, dtype: DType, device, value=1, _shard: int = 0):
        return super().kernel(shape=shape, value=1, dtype=dtype, device=device, _shard=_shard)


class ConstantOp:
    """Literal data as a realized tensor (reference: nabla/ops/creation.py:31). Nothing is recorded
    in a trace for it: the tensor is a leaf that already holds its buffer."""

    name = "constant"

    def __call__(self, value, *, dtype=None, device=None) -> Tensor:
        return constant(value, dtype=dtype, device=device)


_full, _arange, _uniform, _gaussian, _hann = FullOp(), ArangeOp(), UniformOp(), GaussianOp(), HannWindowOp()
_triu, _tril = TriuOp(), TrilOp()
TriOp = _BandOp                # the reference's name for the shared base of triu / tril (creation.py:225)
TriuOp._inst, TrilOp._inst = _triu, _tril


def full(shape, value, *, dtype=None, device=None, is_traced: bool = False) -> Tensor:
    dt, dev = defaults(dtype, device)
    if isinstance(value, Tensor):
        from .view import broadcast_to

        out = broadcast_to(value, _shape(shape))
    else:
        out = _full(shape=_shape(shape), value=value, dtype=dt, device=dev)
    if is_traced:
        out.is_traced = True
    return out


def zeros(shape, *, dtype=None, device=None, is_traced: bool = False) -> Tensor:
    return full(shape, 0, dtype=dtype, device=device, is_traced=is_traced)


def ones(shape, *, dtype=None, device=None, is_traced: bool = False) -> Tensor:
    return full(shape, 1, dtype=dtype, device=device, is_traced=is_traced)


def arange(start=0, stop=None, step=1, *, dtype=None, device=None) -> Tensor:
    if stop is None:
        start, stop = 0, start
    if dtype is None and all(isinstance(v, (int, np.integer)) for v in (start, stop, step)):
        from ..core.common.context import get_default_dtype

        dtype = get_default_dtype()
    dt, dev = defaults(dtype, device)
    return _arange(start=start, stop=stop, step=step, dtype=dt, device=dev)


def uniform(shape=(), low: float = 0.0, high: float = 1.0, *, dtype=None, device=None) -> Tensor:
    dt, dev = defaults(dtype, device)
    return _uniform(shape=_shape(shape), low=float(low), high=float(high), dtype=dt, device=dev)


def gaussian(shape=(), mean: float = 0.0, std: float = 1.0, *, dtype=None, device=None) -> Tensor:
    dt, dev = defaults(dtype, device)
    return _gaussian(shape=_shape(shape), mean=float(mean), std=float(std), dtype=dt, device=dev)


normal = gaussian


def hann_window(window_length: int, *, periodic: bool = True, dtype=None, device=None) -> Tensor:
    dt, dev = defaults(dtype, device)
    return _hann(window_length=int(window_length), periodic=bool(periodic), dtype=dt, device=dev)


def triu(x, k: int = 0) -> Tensor:
    return _triu(ensure_tensor(x), k=int(k))


def tril(x, k: int = 0) -> Tensor:
    return _tril(ensure_tensor(x), k=int(k))


def _like(x: Tensor, value) -> Tensor:
    """Filled tensor with the shape, dtype, device, batch dims and sharding of ``x``."""
    im = x._impl
    out = _full(shape=tuple(im._shape), value=value, dtype=im.dtype, device=im.device)
    if im.sharding is not None:
        from .communication import shard

        out = shard(out, im.sharding.mesh, [d.clone() for d in im.sharding.dim_specs],
                    replicated_axes=set(im.sharding.replicated_axes))
    if im.batch_dims:
        out._impl.batch_dims = im.batch_dims
    return out


def zeros_like(x) -> Tensor:
    return _like(ensure_tensor(x), 0)


def ones_like(x) -> Tensor:
    return _like(ensure_tensor(x), 1)


def full_like(x, value) -> Tensor:
    return _like(ensure_tensor(x), value)
