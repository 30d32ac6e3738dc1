"""Import path of the reference (nabla/ops/communication/shard.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import ShardOp, create_replicated_spec, shard, broadcast  # noqa: F401

__all__ = ['ShardOp', 'create_replicated_spec', 'shard', 'broadcast']
