"""``jax.tree_util`` stand-in."""
from .tree import flatten as tree_flatten  # noqa: F401
from .tree import leaves as tree_leaves  # noqa: F401
from .tree import map as tree_map  # noqa: F401
from .tree import unflatten as tree_unflatten  # noqa: F401
