"""Import path of the reference (nabla/nn/modules/layernorm.py); the layers of this package live in
``layers.py`` and are re-exported here."""
from .layers import LayerNorm  # noqa: F401

__all__ = ['LayerNorm']
