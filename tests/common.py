"""Shared helpers: torch/numpy oracles and tolerant comparison."""
import numpy as np
import torch

import nabla_b200 as nb


def T(a, dtype=None):
    """numpy/torch -> nabla tensor."""
    if isinstance(a, torch.Tensor):
        t = a.detach().clone()
    else:
        t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return nb.Tensor.from_torch(t)


def close(actual, expected, rtol=1e-5, atol=1e-5, msg=""):
    a = actual.to_numpy() if isinstance(actual, nb.Tensor) else np.asarray(actual)
    e = expected.detach().cpu().float().numpy() if isinstance(expected, torch.Tensor) else np.asarray(expected)
    assert a.shape == e.shape, f"{msg} shape {a.shape} vs {e.shape}"
    np.testing.assert_allclose(a.astype(np.float64), e.astype(np.float64), rtol=rtol, atol=atol, err_msg=msg)


def rand(*shape, seed=0, positive=False, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape) * 7 + len(shape))
    x = torch.randn(*shape, generator=g) * scale
    if positive:
        x = x.abs() + 0.5
    return x
