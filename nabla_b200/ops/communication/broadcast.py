"""Import path of the reference (nabla/ops/communication/broadcast.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import DistributedBroadcastOp, distributed_broadcast  # noqa: F401

__all__ = ['DistributedBroadcastOp', 'distributed_broadcast']
