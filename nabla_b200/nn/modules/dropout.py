"""Import path of the reference (nabla/nn/modules/dropout.py); the layers of this package live in
``layers.py`` and are re-exported here."""
from .layers import Dropout  # noqa: F401

__all__ = ['Dropout']
