from .collectives import (accelerator, all_gather, all_reduce, all_to_all, axis_index, broadcast, cpu,
                          distributed_broadcast, gather_all_axes, gpu, pmean, ppermute, reduce_scatter, reshard,
                          reshard_tensor, reshard_to_spec, relabel_spec, shard, to_device, transfer_to)
