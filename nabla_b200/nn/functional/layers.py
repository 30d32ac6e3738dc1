"""Functional layers (reference: nabla/nn/functional/layers.py:30-153).

Each function has two implementations with identical results: ``*_reference`` composes
primitive ops exactly like the reference, and the default entry point dispatches to the fused
operation (``nabla_b200.ops.fused``) when ``use_fused`` says so: tensors on a GPU, or
``NABLA_B200_FUSED=1``. Fused and reference paths are cross-checked in the tests.
"""
from __future__ import annotations

import math
import os

from ...core.tensor.api import Tensor
from ...ops import fused
from ...ops.binary import matmul
from ...ops.comparison import greater
from ...ops.control_flow import where
from ...ops.creation import full, ones, tril, uniform
from ...ops.reduction import mean
from ...ops.unary import cast, rsqrt, softmax
from ...ops.view import gather, swap_axes


def use_fused(*tensors: Tensor) -> bool:
    mode = os.environ.get("NABLA_B200_FUSED", "auto")
    if mode in ("0", "off", "false"):
        return False
    for t in tensors:
        if t is None:
            continue
        if t._impl.batch_dims:
            return False
    if mode in ("1", "on", "true"):
        return True
    return any(t is not None and t._impl.device.label == "gpu" for t in tensors)


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None, activation: str | None = None) -> Tensor:
    """``x @ weight + bias`` with ``weight`` of shape (in, out); ``activation`` in
    {None, 'relu', 'gelu', 'gelu_tanh', 'silu'} is fused into the GEMM epilogue on GPU."""
    if use_fused(x, weight):
        return fused.linear(x, weight, bias, activation=activation)
    out = matmul(x, weight)
    if bias is not None:
        out = out + bias
    if activation is not None:
        from ...ops import unary

        out = {"relu": unary.relu, "gelu": unary.gelu, "silu": unary.silu,
               "gelu_tanh": lambda t: unary.gelu(t, approximate="tanh")}[activation](out)
    return out


def layer_norm_reference(x, weight=None, bias=None, eps: float = 1e-5, axis=-1) -> Tensor:
    mu = mean(x, axis=axis, keepdims=True)
    centered = x - mu
    var = mean(centered * centered, axis=axis, keepdims=True)
    out = centered * rsqrt(var + eps)
    if weight is not None:
        out = out * weight
    if bias is not None:
        out = out + bias
    return out


def layer_norm(x: Tensor, weight: Tensor | None = None, bias: Tensor | None = None, eps: float = 1e-5,
               axis: int | tuple[int, ...] = -1) -> Tensor:
    last = axis in (-1, x.rank - 1) or axis == (-1,) or axis == (x.rank - 1,)
    if last and use_fused(x) and x.rank >= 2:
        return fused.layer_norm(x, weight, bias, eps)
    return layer_norm_reference(x, weight, bias, eps, axis)


def dropout(x: Tensor, p: float = 0.5, training: bool = True) -> Tensor:
    if not training or p <= 0.0:
        return x
    if p >= 1.0:
        return x * 0.0
    if use_fused(x):
        return fused.dropout_fused(x, p)
    mask = cast(greater(uniform(tuple(x._impl.global_shape), 0.0, 1.0, dtype=x.dtype, device=x.device), p), x.dtype)
    return x * mask * (1.0 / (1.0 - p))


def embedding(indices: Tensor, weight: Tensor) -> Tensor:
    """Rows of ``weight`` (vocab, dim) selected by integer ``indices``."""
    return gather(weight, indices, axis=0)


def scaled_dot_product_attention_reference(query, key, value, attn_mask=None, dropout_p: float = 0.0,
                                           is_causal: bool = False, training: bool = True, scale=None) -> Tensor:
    d_k = int(query.shape[-1])
    sc = scale if scale is not None else 1.0 / math.sqrt(d_k)
    scores = matmul(query, swap_axes(key, -2, -1)) * sc
    if is_causal:
        sq, sk = int(query.shape[-2]), int(key.shape[-2])
        causal = tril(ones((sq, sk), dtype=query.dtype, device=query.device))
        neg = full((sq, sk), -1e9, dtype=query.dtype, device=query.device)
        scores = where(greater(causal, 0.0), scores, neg)
    if attn_mask is not None:
        scores = scores + attn_mask
    weights = softmax(scores, axis=-1)
    if dropout_p > 0.0 and training:
        weights = dropout(weights, p=dropout_p, training=True)
    return matmul(weights, value)


def scaled_dot_product_attention(query: Tensor, key: Tensor, value: Tensor, attn_mask: Tensor | None = None,
                                 dropout_p: float = 0.0, is_causal: bool = False, training: bool = True,
                                 scale: float | None = None) -> Tensor:
    """softmax(q k^T / sqrt(d) [+ causal] [+ mask]) v on ``(..., seq, d)`` operands. On GPU this
    is one flash-style kernel that never materialises the (seq_q, seq_k) scores."""
    drop = dropout_p if training else 0.0
    if use_fused(query, key, value) and drop == 0.0 and query.rank >= 3:
        return fused.scaled_dot_product_attention(query, key, value, attn_mask, causal=is_causal, scale=scale)
    return scaled_dot_product_attention_reference(query, key, value, attn_mask, dropout_p, is_causal, training, scale)
