"""Communication ops. Functions (``all_reduce``, ``shard``, ...) are the public API; the ``*_op``
names are the op objects behind them, for code that inspects or extends ops
(reference: nabla/ops/communication/__init__.py)."""
from ..base import CollectiveOperation
from .collectives import (accelerator, all_gather, all_reduce, all_to_all, axis_index, broadcast, cpu,
                          distributed_broadcast, gather_all_axes, gpu, pmean, ppermute, reduce_scatter, reshard,
                          reshard_tensor, reshard_to_spec, relabel_spec, shard, to_device, transfer_to)
from .collectives import (_all_gather_op as all_gather_op, _all_reduce_op as all_reduce_op,
                          _gather_all_op as gather_all_axes_op, _ppermute_op as ppermute_op,
                          _reduce_scatter_op as reduce_scatter_op, _shard_op as shard_op)


class _ComposedOp:
    """Callable stand-in with a ``name`` for collectives that this framework builds from other ops
    (a re-layout, or all-reduce + scale) instead of a dedicated op class."""

    def __init__(self, name: str, fn):
        self.name = name
        self._fn = fn
        self.__doc__ = fn.__doc__

    def __call__(self, *args, **kwargs):
        return self._fn(*args, **kwargs)

    def __repr__(self) -> str:
        return f"<composed op {self.name}>"


class PMeanOp(_ComposedOp):
    """all-reduce followed by a scale by 1 / group size."""


class AllToAllOp(_ComposedOp):
    """a change of layout: the split axis becomes replicated and the concat axis sharded."""


class DistributedBroadcastOp(_ComposedOp):
    """replication of one rank's value over the mesh."""


class AxisIndexOp(_ComposedOp):
    """a constant per device: its coordinate along a mesh axis."""


pmean_op = PMeanOp("pmean", pmean)
all_to_all_op = AllToAllOp("all_to_all", all_to_all)
distributed_broadcast_op = DistributedBroadcastOp("distributed_broadcast", distributed_broadcast)
axis_index_op = AxisIndexOp("axis_index", axis_index)


def create_replicated_spec(mesh, rank: int):
    """Fully replicated sharding spec of a rank-``rank`` tensor on ``mesh``
    (reference: nabla/ops/communication/shard.py:356-368)."""
    from ...core.sharding.spec import DimSpec, ShardingSpec

    return ShardingSpec(mesh, [DimSpec([]) for _ in range(rank)])
from .collectives import (AllGatherOp, AllReduceOp, GatherAllAxesOp, PPermuteOp, ReduceScatterOp, RelabelOp, ShardOp,  # noqa: F401,E402
                          TransferOp)

# The reference keeps every collective in a module named like its function (`.shard`, `.all_reduce`, ...).
# Those module paths exist here as thin re-exports; they are loaded now, and the function names are
# bound again afterwards, because loading a submodule binds its name on the package.
import importlib as _importlib  # noqa: E402

for _m in ("all_gather", "all_reduce", "all_to_all", "axis_index", "base", "broadcast", "p_permute", "reduce_scatter",
           "reshard", "shard", "transfer"):
    _importlib.import_module(__name__ + "." + _m)      # (`from . import shard` would just return the function)
del _m
from .collectives import (all_gather, all_reduce, all_to_all, axis_index, broadcast, reduce_scatter, reshard,  # noqa: F401,E402,F811
                          shard)
