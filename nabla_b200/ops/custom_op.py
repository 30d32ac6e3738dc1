"""Older import path of the custom-kernel entry point (``from nabla.ops.custom_op import
call_custom_kernel`` in the reference's earlier tests); the implementation lives in ``ops/custom.py``."""
from .utils import call_custom_kernel  # noqa: F401
