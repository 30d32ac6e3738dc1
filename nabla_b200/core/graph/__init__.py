from .engine import GRAPH, ComputeGraph, clear_cache, driver_tensor_type, get_cache_stats, reset_cache_stats, seed
from .tracing import OpNode, Trace, trace
from .utils import apply_to_operations, get_all_impls_topological, get_operations_topological, print_trace_graph
