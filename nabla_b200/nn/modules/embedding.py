"""Import path of the reference (nabla/nn/modules/embedding.py); the layers of this package live in
``layers.py`` and are re-exported here."""
from .layers import Embedding  # noqa: F401

__all__ = ['Embedding']
