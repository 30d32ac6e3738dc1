"""nabla_b200: a Blackwell-native (B200 / sm_100a) framework with the capabilities and public
API of nabla-ml/nabla: lazy tensors with eager shape inference, trace-based autodiff
(grad / vjp / jvp / jacobians), vmap, compile, DeviceMesh + factor-based sharding propagation
with deferred partial sums, nn modules, optimizers, LoRA / QLoRA fine-tuning and custom
kernels, on PyTorch tensors with hand-written tcgen05 / TMA CUDA kernels for the hot ops.

The reference gates its import on the MAX runtime (nabla/__init__.py:9-19); this package only
needs torch.
"""
from __future__ import annotations

from importlib import metadata  # noqa: F401  (the reference exposes it the same way)

from . import config, nn, testing
from .core import (GRAPH, PyTreeDef, Tensor, TensorImpl, default_device, default_dtype, defaults, defaults_like,
                   is_tensor, realize_all, register_pytree_node, tensor_leaves, traced, tree_flatten, tree_leaves,
                   tree_map, tree_structure, tree_unflatten, untraced, with_batch_dims)
from .core.autograd import forward
from .core.autograd.backward import backward
from .core.graph.engine import clear_cache, get_cache_stats, reset_cache_stats, seed
from .core.graph.tracing import trace
from .core.sharding.spec import (DeviceMesh, DimSpec, P, PartitionSpec, ShardingSpec, compute_local_shape,
                                 get_num_shards)
from .ops.base import BinaryOperation, CreationOperation, Operation, ReduceOperation, UnaryOperation
from .ops.binary import add, div, matmul, mod, mul, outer, pow, sub
from .ops.communication import (accelerator, all_gather, all_reduce, all_to_all, axis_index, cpu, distributed_broadcast,
                                gather_all_axes, gpu, pmean, ppermute, reduce_scatter, reshard, shard, to_device,
                                transfer_to)
from .ops.comparison import (equal, greater, greater_equal, less, less_equal, logical_and, logical_not, logical_or,
                             logical_xor, not_equal)
from .ops.control_flow import cond, scan, where, while_loop
from .ops.convolution import conv2d, conv2d_transpose
from .ops.creation import (arange, constant, full, full_like, gaussian, hann_window, normal, ones, ones_like, tril,
                           triu, uniform, zeros, zeros_like)
from .ops.custom import register_kernel
from .ops.multi_output import chunk, minmax, split, unbind
from .ops.pooling import avg_pool2d, max_pool2d
from .ops.reduction import (argmax, argmin, cumsum, mean, mean_physical, reduce_max, reduce_min, reduce_sum,
                            reduce_sum_physical)
from .ops.unary import (abs, acos, atanh, cast, cos, erf, exp, floor, gelu, is_inf, is_nan, log, log1p, logsoftmax,
                        neg, relu, round, rsqrt, sigmoid, silu, sin, softmax, sqrt, tanh, trunc)
from .ops.utils import call_custom_kernel
from .ops.view import (as_interleaved_complex, broadcast_batch_dims, broadcast_to, broadcast_to_physical, concatenate,
                       decr_batch_dims, flatten, flip, gather, incr_batch_dims, move_axis_from_batch_dims,
                       move_axis_to_batch_dims, moveaxis, moveaxis_physical, pad, permute, rebind, reshape, scatter,
                       scatter_add, slice_tensor, slice_update, squeeze, squeeze_physical, stack, swap_axes, take,
                       transpose, unsqueeze, unsqueeze_physical, view_as_real_interleaved)
from .transforms.compile import CompilationStats, CompiledFunction, compile
from .transforms.grad import grad, value_and_grad
from .transforms.jacfwd import jacfwd
from .transforms.jacrev import jacrev
from .transforms.jvp import _clear_jvp_cache, jvp
from .transforms.shard_map import shard_map
from .transforms.vjp import vjp
from .transforms.vmap import vmap
from .types import CPU, Accelerator, Device, Dim, DType, Shape, StaticDim, SymbolicDim, accelerator_count

sum = reduce_sum
max = reduce_max
min = reduce_min

__version__ = "0.1.0"


def _clear_caches() -> None:
    """Drop the plan cache and shape-inference cache (tests call this between cases)."""
    from .ops.base import _META_CACHE

    GRAPH.clear_all()
    _META_CACHE.clear()


def driver_tensor_type(t: Tensor):
    """(shape, dtype, device) triple of a tensor's primary buffer."""
    return tuple(t._impl.physical_local_shape(0)), t.dtype, t.device
