"""Import path of the reference (nabla/nn/modules/transformer.py); the layers of this package live in
``layers.py`` and are re-exported here."""
from .layers import TransformerEncoderLayer, TransformerDecoderLayer  # noqa: F401

__all__ = ['TransformerEncoderLayer', 'TransformerDecoderLayer']
