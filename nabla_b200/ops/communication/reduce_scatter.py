"""Import path of the reference (nabla/ops/communication/reduce_scatter.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import ReduceScatterOp, reduce_scatter  # noqa: F401

__all__ = ['ReduceScatterOp', 'reduce_scatter']
