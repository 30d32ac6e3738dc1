"""Import path of the reference (nabla/ops/communication/all_gather.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import AllGatherOp, GatherAllAxesOp, all_gather, gather_all_axes  # noqa: F401

__all__ = ['AllGatherOp', 'GatherAllAxesOp', 'all_gather', 'gather_all_axes']
