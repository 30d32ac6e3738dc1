from nabla_b200.types import DType  # noqa: F401
