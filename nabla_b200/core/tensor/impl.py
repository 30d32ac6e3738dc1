"""Per-tensor state (reference: nabla/core/tensor/impl.py:42-497).

A ``TensorImpl`` is either *realized* (it owns one ``torch.Tensor`` per locally held shard) or
a *promise*: shape, dtype, device and sharding are known eagerly and ``output_refs`` points at
the ``OpNode`` that will produce the data at ``realize()`` time.

Shapes: the *physical* shape includes ``batch_dims`` leading vmap dimensions; the *logical*
shape is what the user sees. A sharded impl stores the global physical shape; local shapes
follow from the spec (ceil-div chunks).
"""
from __future__ import annotations

from typing import TYPE_CHECKING, Any

import numpy as np
import torch

from ...types import Device, DType, Shape

if TYPE_CHECKING:
    from ..graph.tracing import OpNode
    from ..sharding.spec import ShardingSpec


class TensorImpl:
    __slots__ = ("_buffers", "_shape", "_dtype", "_device", "sharding", "sharding_constraint", "is_traced",
                 "requires_grad", "grad", "tangent", "cotangent", "dual", "batch_dims", "output_refs",
                 "output_index", "_local_shapes", "_keepalive", "__weakref__")

    def __init__(self, buffers: list[torch.Tensor] | torch.Tensor | None = None, *, shape=None, dtype: DType | None = None,
                 device: Device | None = None, sharding: "ShardingSpec | None" = None, batch_dims: int = 0,
                 is_traced: bool = False, bufferss=None, values=None, sharding_constraint=None):
        if buffers is None:
            buffers = bufferss if bufferss is not None else values      # the reference's keyword names
        if isinstance(buffers, torch.Tensor):
            buffers = [buffers]
        self._buffers = buffers
        self.sharding = sharding
        self.sharding_constraint = sharding_constraint
        self.is_traced = is_traced
        self.requires_grad = False
        self.grad = None
        self.tangent = None
        self.cotangent = None
        self.dual = None
        self.batch_dims = batch_dims
        self.output_refs: "OpNode | None" = None
        self.output_index = 0
        self._local_shapes = None
        self._keepalive = None
        if buffers is not None and shape is None:
            b0 = buffers[0]
            if sharding is not None:
                from ..sharding.spec import compute_global_shape

                shapes = [tuple(b.shape) for b in buffers]
                shape = compute_global_shape(shapes[0], sharding,
                                             shapes if len(shapes) == sharding.mesh.size else None)
            else:
                shape = tuple(b0.shape)
            dtype = DType.from_torch(b0.dtype)
            device = Device.from_torch(b0.device)
        self._shape = tuple(int(s) for s in shape)
        self._dtype = dtype
        self._device = device

    # ---- state
    @property
    def is_realized(self) -> bool:
        return self._buffers is not None

    @property
    def is_sharded(self) -> bool:
        return self.sharding is not None

    @property
    def num_shards(self) -> int:
        return self.sharding.mesh.num_local if self.sharding is not None else 1

    @property
    def dtype(self) -> DType:
        return self._dtype

    @property
    def device(self) -> Device:
        return self._device

    # ---- shapes
    @property
    def physical_global_shape(self) -> tuple[int, ...]:
        return self._shape

    @property
    def global_shape(self) -> tuple[int, ...]:
        return self._shape[self.batch_dims:]

    @property
    def batch_shape(self) -> tuple[int, ...]:
        return self._shape[: self.batch_dims]

    def local_shard_ids(self) -> list[int]:
        return self.sharding.mesh.local_ids if self.sharding is not None else [0]

    def physical_local_shape(self, shard_idx: int = 0) -> tuple[int, ...]:
        """Physical shape of the ``shard_idx``-th locally held shard."""
        if self._buffers is not None:
            return tuple(self._buffers[shard_idx].shape)
        if self.sharding is None:
            return self._shape
        if self._local_shapes is None:
            from ..sharding.spec import compute_local_shape

            self._local_shapes = [compute_local_shape(self._shape, self.sharding, d) for d in self.local_shard_ids()]
        return self._local_shapes[shard_idx]

    def logical_local_shape(self, shard_idx: int = 0) -> tuple[int, ...]:
        return self.physical_local_shape(shard_idx)[self.batch_dims:]

    def primary_buffer(self) -> torch.Tensor | None:
        return self._buffers[0] if self._buffers else None

    # ---- graph introspection (reference: nabla/core/tensor/impl.py:157-187, 233-326)
    @property
    def op(self):
        """The operation whose call produced this tensor (None for leaves)."""
        return self.output_refs.op if self.output_refs is not None else None

    @property
    def op_kwargs(self) -> dict | None:
        return self.output_refs.op_kwargs if self.output_refs is not None else None

    @property
    def op_name(self) -> str | None:
        return self.output_refs.op.name if self.output_refs is not None else None

    @property
    def parents(self) -> list["TensorImpl"]:
        """Tensor arguments of the producing op call, in argument order ([] for leaves)."""
        return list(self.output_refs.input_impls()) if self.output_refs is not None else []

    @property
    def is_leaf(self) -> bool:
        """True when no recorded op produced this tensor (inputs, constants, detached results)."""
        return self.output_refs is None

    @property
    def ndim(self) -> int:
        return len(self._shape) - self.batch_dims

    @property
    def physical_shape(self) -> tuple[int, ...]:
        """Shape of the first locally held shard, batch dims included."""
        return self.physical_local_shape(0)

    @property
    def local_shape(self) -> tuple[int, ...]:
        return self.physical_local_shape(0)

    @property
    def logical_shape(self) -> tuple[int, ...]:
        """Shape of the first locally held shard without the batch dims."""
        return self.logical_local_shape(0)

    def physical_local_shape_ints(self, shard_idx: int = 0) -> tuple[int, ...]:
        return tuple(int(d) for d in self.physical_local_shape(shard_idx))

    @property
    def physical_global_shape_ints(self) -> tuple[int, ...]:
        return tuple(int(d) for d in self._shape)

    @property
    def global_shape_ints(self) -> tuple[int, ...]:
        return tuple(int(d) for d in self._shape[self.batch_dims:])

    def get_unrealized_shape(self) -> tuple[int, ...]:
        return self.global_shape

    def get_unrealized_dtype(self) -> DType:
        return self._dtype

    def get_realized_shape(self) -> tuple[int, ...]:
        if self._buffers is None:
            raise RuntimeError("tensor is not realized")
        return self.global_shape

    def get_realized_dtype(self) -> DType:
        if self._buffers is None:
            raise RuntimeError("tensor is not realized")
        return self._dtype

    @property
    def primary_value(self) -> torch.Tensor | None:
        """The first local buffer (the reference returns its driver buffer / graph value here)."""
        return self.primary_buffer()

    # ---- formatting: f32[8,4](<dp, *> | partial={'tp'})(local=[4,4])
    @staticmethod
    def _fmt_shape(shape, batch_dims: int) -> str:
        shape = [int(d) for d in shape]
        if batch_dims > 0:
            b = ",".join(str(d) for d in shape[:batch_dims])
            r = ",".join(str(d) for d in shape[batch_dims:])
            return f"[{b} | {r}]"
        return "[" + ",".join(str(d) for d in shape) + "]"

    @staticmethod
    def _fmt_factors(sharding) -> str:
        if sharding is None:
            return ""
        fs = ["*" if not d.axes else ", ".join(d.axes) for d in sharding.dim_specs]
        par = ""
        if sharding.partial_sum_axes:
            par = " | partial={" + ", ".join(f"'{a}'" for a in sorted(sharding.partial_sum_axes)) + "}"
        return f"(<{', '.join(fs)}>{par})"

    def format_metadata(self, include_data: bool = False) -> str:
        dt = self._dtype.short if self._dtype is not None else "?"
        gl = self._fmt_shape(self._shape, self.batch_dims)
        if self.sharding is not None:
            loc = self._fmt_shape(self.physical_local_shape(0), self.batch_dims)
            header = f"{dt}{gl}{self._fmt_factors(self.sharding)}(local={loc})"
        else:
            header = f"{dt}{gl}"
        if not include_data:
            return header
        if self._buffers is None:
            return f"[unrealized] : {header}"
        opts = dict(edgeitems=3, threshold=6, max_line_width=1000, precision=4, suppress_small=True)

        def arr(b):
            b = b.detach().cpu()
            if b.dtype == torch.bfloat16:
                b = b.float()
            return np.array2string(b.numpy(), **opts)

        if self.sharding is not None:
            parts = []
            for i, b in zip(self.local_shard_ids(), self._buffers):
                prefix = f"shard({i}): "
                lines = arr(b).split("\n")
                parts.append("\n".join([prefix + lines[0]] + [" " * len(prefix) + l for l in lines[1:]]))
            block = "\n".join("  " + l for l in "\n".join(parts).split("\n"))
            data = f"[\n{block}\n]"
        else:
            data = arr(self._buffers[0])
        return f"{data} : {header}"

    def __repr__(self) -> str:
        return self.format_metadata(include_data=True)

    # ---- compat with the reference's attribute names
    @property
    def shape(self) -> Shape:
        return Shape(self.global_shape)
