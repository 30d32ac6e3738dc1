"""Import path of the reference (nabla/ops/communication/axis_index.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import AxisIndexOp, axis_index  # noqa: F401

__all__ = ['AxisIndexOp', 'axis_index']
