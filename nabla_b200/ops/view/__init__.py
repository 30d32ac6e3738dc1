from .axes import (flip, moveaxis, permute, squeeze, squeeze_physical, swap_axes, transpose, unsqueeze,
                   unsqueeze_physical)
from .batch import (broadcast_batch_dims, decr_batch_dims, incr_batch_dims, move_axis_from_batch_dims,
                    move_axis_to_batch_dims, moveaxis_physical)
from .complex import as_interleaved_complex, view_as_real_interleaved
from .indexing import gather, scatter, scatter_add, take
from .shape import (broadcast_to, broadcast_to_physical, concatenate, flatten, pad, rebind, reshape, slice_tensor,
                    slice_update, slice_update_inplace, stack)
from .axes import SqueezePhysicalOp, UnsqueezePhysicalOp  # noqa: F401,E402
