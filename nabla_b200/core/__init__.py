from .common import *  # noqa: F401,F403
from .graph import GRAPH, OpNode, Trace, trace
from .tensor import Tensor, TensorImpl, realize_all
