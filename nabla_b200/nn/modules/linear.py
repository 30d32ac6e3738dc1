"""Import path of the reference (nabla/nn/modules/linear.py); the layers of this package live in
``layers.py`` and are re-exported here."""
from .layers import Linear  # noqa: F401

__all__ = ['Linear']
