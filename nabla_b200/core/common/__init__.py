from .context import (_in_running_loop, default_device, default_dtype, defaults, defaults_like, get_default_device,
                      get_default_dtype, set_default_device)
from .pytree import (tree_flatten_full, tree_flatten_with_names, tree_unflatten_full, PyTreeDef, is_tensor, register_pytree_node, tensor_leaves, traced, tree_flatten,
                     tree_leaves, tree_map, tree_structure, tree_unflatten, untraced, with_batch_dims)
