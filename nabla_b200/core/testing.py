"""Test helpers (reference: nabla/core/testing.py:76-133): batch realization and
``assert_allclose`` across nabla / torch / numpy pytrees."""
from __future__ import annotations

from typing import Any

import numpy as np

from .common import pytree
from .tensor.api import Tensor, realize_all


def batch_realize(*trees: Any) -> None:
    ts = [t for tr in trees for t in pytree.tensor_leaves(tr)]
    realize_all(*ts)


def _to_numpy(x: Any) -> np.ndarray:
    import torch

    if isinstance(x, Tensor):
        return x.to_numpy()
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu()
        return (x.float() if x.dtype == torch.bfloat16 else x).numpy()
    return np.asarray(x)


def assert_allclose(actual: Any, expected: Any, rtol: float = 1e-5, atol: float = 1e-8, err_msg: str = "", *,
                    equal_nan: bool = False, realize: bool = True) -> None:
    """Leaf-by-leaf numerical comparison of two pytrees of tensors / arrays. ``realize=False`` skips
    the batched evaluation for callers that already did it (reference: nabla/core/testing.py:59-82)."""
    la = pytree.tree_leaves(actual)
    le = pytree.tree_leaves(expected)
    if len(la) != len(le):
        raise AssertionError(f"pytree leaf count differs: {len(la)} vs {len(le)} {err_msg}")
    if realize:
        batch_realize(actual, expected)
    for a, e in zip(la, le):
        np.testing.assert_allclose(_to_numpy(a), _to_numpy(e), rtol=rtol, atol=atol, err_msg=err_msg, equal_nan=equal_nan)
