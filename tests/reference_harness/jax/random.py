"""``jax.random`` stand-in: keys are integers, draws come from a torch generator seeded by the key.
The values differ from jax's; the tests only need them deterministic per key."""
import torch

from .numpy import _dt, float32


def PRNGKey(seed):
    return int(seed) & 0x7FFFFFFF


key = PRNGKey


def _gen(k):
    g = torch.Generator()
    g.manual_seed(int(k))
    return g


def split(k, num=2):
    return [(int(k) * 1000003 + 7919 * (i + 1)) & 0x7FFFFFFF for i in range(num)]


def fold_in(k, data):
    return (int(k) * 1000003 + int(data)) & 0x7FFFFFFF


def _shape(shape):
    return (shape,) if isinstance(shape, int) else tuple(int(s) for s in shape)


def normal(k, shape=(), dtype=float32):
    return torch.randn(_shape(shape), generator=_gen(k), dtype=_dt(dtype))


def uniform(k, shape=(), dtype=float32, minval=0.0, maxval=1.0):
    return torch.rand(_shape(shape), generator=_gen(k), dtype=_dt(dtype)) * (maxval - minval) + minval


def randint(k, shape, minval, maxval, dtype=torch.int32):
    return torch.randint(int(minval), int(maxval), _shape(shape), generator=_gen(k), dtype=_dt(dtype))


def choice(k, a, shape=(), replace=True, p=None):
    a = torch.arange(a) if isinstance(a, int) else a
    idx = torch.randint(0, a.shape[0], _shape(shape), generator=_gen(k))
    return a[idx]


def bernoulli(k, p=0.5, shape=()):
    return torch.rand(_shape(shape), generator=_gen(k)) < p


def permutation(k, x):
    n = x if isinstance(x, int) else x.shape[0]
    perm = torch.randperm(n, generator=_gen(k))
    return perm.to(torch.int32) if isinstance(x, int) else x[perm]
