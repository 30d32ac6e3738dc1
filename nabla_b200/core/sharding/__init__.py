from .propagation import (OpShardingRule, OpShardingRuleTemplate, elementwise_rule, infer_from_rule,
                          propagate_sharding, required_input_specs)
from .spec import (DeviceMesh, DimSpec, P, PartitionSpec, ShardingSpec, compute_global_shape,
                   compute_local_shape, compute_local_slices, get_num_shards, needs_reshard, parse_sub_axis)
