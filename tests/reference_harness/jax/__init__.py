"""Stand-in for the parts of ``jax`` that the reference's unit tests use as their ORACLE, built on
``torch.func``. It exists so that those test files can run unchanged where jax is not installed:
the package under test never imports it. Arrays are CPU ``torch.Tensor`` objects."""
from __future__ import annotations

import torch
from torch import func as _func

from . import dlpack, lax, nn, random, tree, tree_util  # noqa: F401
from . import numpy  # noqa: F401

Array = torch.Tensor


class _Config:
    def update(self, *a, **k):
        pass


config = _Config()


def clear_caches():
    pass


def devices(*a, **k):
    return ["cpu"]


def _argnums(argnums):
    return argnums if isinstance(argnums, int) else tuple(argnums)


def _arrays(tree_):
    """numpy arrays and Python scalars are arrays to jax; torch.func wants tensors."""
    import numpy as np

    def one(x):
        if isinstance(x, (np.ndarray, np.generic, float)):
            return numpy.asarray(x)
        return x

    return tree.map(one, tree_)


def _with_arrays(transform):
    def wrapped(*args, **kwargs):
        return transform(*_arrays(list(args)), **kwargs)

    return wrapped


def grad(fun, argnums=0, has_aux=False):
    return _with_arrays(_func.grad(fun, argnums=_argnums(argnums), has_aux=has_aux))


def value_and_grad(fun, argnums=0, has_aux=False):
    inner = _func.grad_and_value(fun, argnums=_argnums(argnums), has_aux=has_aux)

    def wrapped(*args, **kwargs):
        g, v = inner(*_arrays(list(args)), **kwargs)
        return v, g

    return wrapped


def vjp(fun, *primals, has_aux=False):
    res = _func.vjp(fun, *_arrays(list(primals)), has_aux=has_aux)
    out, pull = res[0], res[1]

    def pullback(ct):
        r = pull(_arrays(ct))
        return r if isinstance(r, tuple) else (r,)

    return (out, pullback, res[2]) if has_aux else (out, pullback)


def jvp(fun, primals, tangents, has_aux=False):
    return _func.jvp(fun, tuple(_arrays(list(primals))), tuple(_arrays(list(tangents))), has_aux=has_aux)


def jacrev(fun, argnums=0, has_aux=False):
    return _with_arrays(_func.jacrev(fun, argnums=_argnums(argnums), has_aux=has_aux))


def jacfwd(fun, argnums=0, has_aux=False):
    return _with_arrays(_func.jacfwd(fun, argnums=_argnums(argnums), has_aux=has_aux))


def hessian(fun, argnums=0):
    return _with_arrays(_func.hessian(fun, argnums=_argnums(argnums)))


def vmap(fun, in_axes=0, out_axes=0, axis_name=None, axis_size=None, spmd_axis_name=None):
    if isinstance(in_axes, list):
        in_axes = tuple(in_axes)
    return _with_arrays(_func.vmap(fun, in_dims=in_axes, out_dims=out_axes))


def jit(fun=None, **kwargs):
    if fun is None:
        return lambda f: f
    return fun


def tree_map(f, tree_, *rest):
    return tree.map(f, tree_, *rest)
