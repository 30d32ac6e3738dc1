from .base import (AxisOp, BinaryOperation, CollectiveOperation, CreationOperation, Operation, ReduceOperation,
                   ShapeOp, UnaryOperation, ensure_tensor)
from .binary import add, div, matmul, mod, mul, outer, pow, sub
from .comparison import (equal, greater, greater_equal, less, less_equal, logical_and, logical_not, logical_or,
                         logical_xor, not_equal)
from .creation import (arange, constant, full, full_like, gaussian, hann_window, normal, ones, ones_like, tril, triu,
                       uniform, zeros, zeros_like)
from .multi_output import chunk, minmax, split, unbind
from .reduction import (argmax, argmin, cumsum, mean, mean_physical, reduce_max, reduce_min, reduce_sum,
                        reduce_sum_physical)
from .unary import (abs, acos, atanh, cast, cos, erf, exp, floor, gelu, is_inf, is_nan, log, log1p, logsoftmax, neg,
                    relu, round, rsqrt, sigmoid, silu, sin, softmax, sqrt, tanh, trunc)
from .utils import call_custom_kernel, reduce_to_shape
from .view import *  # noqa: F401,F403
from .view import gather, scatter, take
from .communication import (accelerator, all_gather, all_reduce, all_to_all, cpu, distributed_broadcast, gpu, ppermute,
                            reduce_scatter, reshard, shard, to_device, transfer_to)
from .control_flow import cond, scan, where, while_loop
from .convolution import conv2d, conv2d_transpose
from .pooling import avg_pool2d, max_pool2d
from .utils import _clear_hashable_cache, _get_tensor_hash, _make_hashable  # noqa: F401

# class names of the reference's op hierarchy (nabla/ops/__init__.py:6-14)
BinaryOp, UnaryOp, ReduceOp, CreationOp, CollectiveOp = (BinaryOperation, UnaryOperation, ReduceOperation,
                                                         CreationOperation, CollectiveOperation)
