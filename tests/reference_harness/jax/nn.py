"""``jax.nn`` stand-in."""
import torch
import torch.nn.functional as F

from .numpy import _a


def relu(x):
    return torch.relu(_a(x))


def sigmoid(x):
    return torch.sigmoid(_a(x))


def silu(x):
    return F.silu(_a(x))


swish = silu


def gelu(x, approximate=True):
    return F.gelu(_a(x), approximate="tanh" if approximate else "none")


def softmax(x, axis=-1):
    return torch.softmax(_a(x), dim=axis)


def log_softmax(x, axis=-1):
    return torch.log_softmax(_a(x), dim=axis)


def softplus(x):
    return F.softplus(_a(x))


def tanh(x):
    return torch.tanh(_a(x))


def one_hot(x, num_classes, dtype=torch.float32):
    return F.one_hot(_a(x).long(), num_classes).to(dtype)


def logsumexp(x, axis=None, keepdims=False):
    from .numpy import logsumexp as f

    return f(x, axis, keepdims)
