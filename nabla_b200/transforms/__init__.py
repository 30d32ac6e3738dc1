from .compile import CompilationStats, CompiledFunction, compile
from .grad import grad, value_and_grad
from .jacfwd import jacfwd
from .jacrev import jacrev
from .jvp import _clear_jvp_cache, jvp
from .shard_map import shard_map
from .vjp import vjp
from .vmap import vmap
