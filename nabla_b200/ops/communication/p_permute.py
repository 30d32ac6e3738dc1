"""Import path of the reference (nabla/ops/communication/p_permute.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import PPermuteOp, ppermute  # noqa: F401

__all__ = ['PPermuteOp', 'ppermute']
