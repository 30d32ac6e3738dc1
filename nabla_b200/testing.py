from .core.testing import assert_allclose, batch_realize  # noqa: F401
