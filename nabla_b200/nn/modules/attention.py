"""Import path of the reference (nabla/nn/modules/attention.py); the layers of this package live in
``layers.py`` and are re-exported here."""
from .layers import MultiHeadAttention  # noqa: F401

__all__ = ['MultiHeadAttention']
