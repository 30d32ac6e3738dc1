from .engine import GRAPH, ComputeGraph, clear_cache, get_cache_stats, reset_cache_stats, seed
from .tracing import OpNode, Trace, trace
from .utils import apply_to_operations, get_all_impls_topological, get_operations_topological, print_trace_graph


def driver_tensor_type(t):
    """(shape, dtype, device) of a realized buffer: what the engine needs to know about an input
    (reference: nabla/core/graph/engine.py:91, which returns the MAX graph tensor type of a driver
    buffer; the buffers here are torch tensors)."""
    from ...types import as_dtype

    return tuple(int(d) for d in t.shape), as_dtype(t.dtype), t.device
