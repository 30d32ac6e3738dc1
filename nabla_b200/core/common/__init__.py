from .context import (default_device, default_dtype, defaults, defaults_like, get_default_device,
                      get_default_dtype, set_default_device)
from .pytree import (PyTreeDef, is_tensor, register_pytree_node, tensor_leaves, traced, tree_flatten,
                     tree_leaves, tree_map, tree_structure, tree_unflatten, untraced, with_batch_dims)
