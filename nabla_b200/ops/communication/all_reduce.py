"""Import path of the reference (nabla/ops/communication/all_reduce.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import AllReduceOp, PMeanOp, all_reduce, pmean  # noqa: F401

__all__ = ['AllReduceOp', 'PMeanOp', 'all_reduce', 'pmean']
