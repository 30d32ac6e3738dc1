from .common import *  # noqa: F401,F403
from .common.context import _in_running_loop  # noqa: F401
from .graph import (GRAPH, ComputeGraph, OpNode, Trace, apply_to_operations, driver_tensor_type,
                    get_all_impls_topological, get_operations_topological, print_trace_graph, trace)
from .tensor import Tensor, TensorImpl, realize_all
