"""Import path of the reference (nabla/ops/communication/base.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import CollectiveOperation  # noqa: F401

__all__ = ['CollectiveOperation']
