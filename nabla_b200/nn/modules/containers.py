"""Import path of the reference (nabla/nn/modules/containers.py); the layers of this package live in
``layers.py`` and are re-exported here."""
from .layers import Sequential  # noqa: F401

__all__ = ['Sequential']
