from .engine import GRAPH, ComputeGraph, clear_cache, get_cache_stats, reset_cache_stats, seed
from .tracing import OpNode, Trace, trace
from .utils import print_trace_graph
