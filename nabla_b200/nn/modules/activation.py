"""Import path of the reference (nabla/nn/modules/activation.py); the layers of this package live in
``layers.py`` and are re-exported here."""
from .layers import ReLU, GELU, Sigmoid, Tanh, SiLU, Softmax  # noqa: F401

__all__ = ['ReLU', 'GELU', 'Sigmoid', 'Tanh', 'SiLU', 'Softmax']
