from .backward import BackwardEngine, backward, backward_on_trace, suppress_tracing
from .forward import ForwardEngine, forward_on_trace
