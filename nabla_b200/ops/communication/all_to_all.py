"""Import path of the reference (nabla/ops/communication/all_to_all.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import AllToAllOp, all_to_all  # noqa: F401

__all__ = ['AllToAllOp', 'all_to_all']
