"""Interleaved-complex views (reference: nabla/ops/view/complex.py:18-102): a real tensor whose
last dimension is 2 (re, im) seen as complex and back."""
from __future__ import annotations

import torch

from ...core.tensor.api import Tensor
from ..base import Operation, ensure_tensor


class AsInterleavedComplexOp(Operation):
    def kernel(self, x):
        if x.shape[-1] != 2:
            raise ValueError("as_interleaved_complex needs a trailing dimension of size 2")
        return torch.view_as_complex(x.contiguous())

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        from ...core.sharding.propagation import OpShardingRule

        r = len(input_shapes[0])
        return OpShardingRule([{i: [f"d{i}"] if i < r - 1 else ["bcast_c"] for i in range(r)}],
                              [{i: [f"d{i}"] for i in range(r - 1)}])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (view_as_real_interleaved(cot),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return as_interleaved_complex(tangents[0])


class ViewAsRealInterleavedOp(Operation):
    def kernel(self, x):
        return torch.view_as_real(x)

    def sharding_rule(self, input_shapes, output_shapes, **kw):
        from ...core.sharding.propagation import OpShardingRule

        r = len(input_shapes[0])
        return OpShardingRule([{i: [f"d{i}"] for i in range(r)}],
                              [{**{i: [f"d{i}"] for i in range(r)}, r: ["ri"]}])

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (as_interleaved_complex(cot),)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return view_as_real_interleaved(tangents[0])


_as_c, _as_r = AsInterleavedComplexOp(), ViewAsRealInterleavedOp()


def as_interleaved_complex(x) -> Tensor:
    return _as_c(ensure_tensor(x))


def view_as_real_interleaved(x) -> Tensor:
    return _as_r(ensure_tensor(x))
