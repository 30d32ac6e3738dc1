"""Import path of the reference (nabla/ops/communication/reshard.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import reshard, reshard_tensor, create_replicated_spec  # noqa: F401

__all__ = ['reshard', 'reshard_tensor', 'create_replicated_spec']
