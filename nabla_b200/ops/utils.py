"""Op helpers: un-broadcasting and the custom-kernel entry point
(reference: nabla/ops/utils.py:765-824, nabla/core/autograd/backward.py:31-54)."""
from __future__ import annotations

from typing import Any, Sequence

from ..core.tensor.api import Tensor


def reduce_to_shape(x: Tensor, shape: Sequence[int]) -> Tensor:
    """Sum ``x`` over the dimensions that numpy broadcasting added to reach ``x.shape`` from
    ``shape`` (used to map cotangents back onto broadcast operands)."""
    from .reduction import reduce_sum

    shape = tuple(int(s) for s in shape)
    cur = tuple(x._impl.global_shape)
    if cur == shape:
        return x
    extra = len(cur) - len(shape)
    if extra > 0:
        x = reduce_sum(x, axis=tuple(range(extra)), keepdims=False)
        cur = tuple(x._impl.global_shape)
    axes = tuple(i for i, (c, s) in enumerate(zip(cur, shape)) if s == 1 and c != 1)
    if axes:
        x = reduce_sum(x, axis=axes, keepdims=True)
    if tuple(x._impl.global_shape) != shape:
        from .view import reshape

        x = reshape(x, shape)
    return x


def call_custom_kernel(func_name: str, kernel_path: Any, values, out_types, device=None, **kwargs):
    """Run a registered custom CUDA (or host) kernel as one op.

    Signature kept from the reference (nabla/ops/utils.py:765-824), where ``kernel_path`` is a
    directory of Mojo kernels. Here ``kernel_path`` may be a ``.cu`` file (compiled with nvcc
    for sm_100a on first use), a built ``.so`` or ``None`` when ``func_name`` was registered
    with ``nabla_b200.ops.custom.register_kernel``. ``out_types`` describes the outputs:
    ``(shape, dtype)`` pairs or Tensors to imitate.
    """
    from .custom import call_custom_kernel as impl

    return impl(func_name, kernel_path, values, out_types, device=device, **kwargs)
