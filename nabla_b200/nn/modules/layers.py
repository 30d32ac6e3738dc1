"""Layers (reference: nabla/nn/modules/{linear,activation,containers,dropout,embedding,
layernorm,attention,transformer}.py). ``Linear.weight`` is (in_features, out_features) and
``Linear.bias`` is (1, out_features), as in the reference."""
from __future__ import annotations

from typing import Any

from ...core.tensor.api import Tensor
from ...ops import unary
from ...ops.creation import gaussian, ones, zeros
from ...ops.view import reshape, swap_axes
from ...types import DType
from .. import functional as F
from .base import Module


def _param(t: Tensor) -> Tensor:
    t.realize()
    t.requires_grad = True
    return t


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, dtype=DType.float32, device=None):
        super().__init__()
        self.in_features, self.out_features = int(in_features), int(out_features)
        self.weight = _param(F.xavier_normal((in_features, out_features), dtype=dtype, device=device))
        self.bias = _param(zeros((1, out_features), dtype=dtype, device=device)) if bias else None

    def forward(self, x: Tensor) -> Tensor:
        return F.linear(x, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class ReLU(Module):
    def forward(self, x):
        return unary.relu(x)


class GELU(Module):
    def __init__(self, approximate: str = "none"):
        super().__init__()
        self.approximate = approximate

    def forward(self, x):
        return unary.gelu(x, approximate=self.approximate)


class Sigmoid(Module):
    def forward(self, x):
        return unary.sigmoid(x)


class Tanh(Module):
    def forward(self, x):
        return unary.tanh(x)


class SiLU(Module):
    def forward(self, x):
        return unary.silu(x)


class Softmax(Module):
    def __init__(self, axis: int = -1):
        super().__init__()
        self.axis = axis

    def forward(self, x):
        return unary.softmax(x, axis=self.axis)

    def extra_repr(self):
        return f"axis={self.axis}"


class Sequential(Module):
    def __init__(self, *args: Any):
        super().__init__()
        if len(args) == 1 and isinstance(args[0], dict):
            for k, m in args[0].items():
                setattr(self, k, m)
            self._order = tuple(args[0].keys())
        else:
            for i, m in enumerate(args):
                setattr(self, str(i), m)
            self._order = tuple(str(i) for i in range(len(args)))

    def forward(self, x):
        for k in self._order:
            x = self._modules[k](x)
        return x

    def __len__(self):
        return len(self._order)

    def __getitem__(self, i):
        return self._modules[self._order[i]]

    def __iter__(self):
        return (self._modules[k] for k in self._order)


class Dropout(Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        if not 0.0 <= p < 1.0:
            raise ValueError(f"dropout probability must be in [0, 1), got {p}")
        self.p = float(p)

    def forward(self, x):
        return F.dropout(x, self.p, training=self._training)

    def extra_repr(self):
        return f"p={self.p}"


class Embedding(Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, *, dtype=DType.float32, device=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim = int(num_embeddings), int(embedding_dim)
        self.weight = _param(gaussian((num_embeddings, embedding_dim), 0.0, 1.0, dtype=dtype, device=device))

    def forward(self, indices):
        return F.embedding(indices, self.weight)

    def extra_repr(self):
        return f"num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim}"


class LayerNorm(Module):
    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True, *, dtype=DType.float32,
                 device=None):
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(int(d) for d in normalized_shape)
        self.eps = float(eps)
        self.elementwise_affine = bool(elementwise_affine)
        if elementwise_affine:
            self.weight = _param(ones(self.normalized_shape, dtype=dtype, device=device))
            self.bias = _param(zeros(self.normalized_shape, dtype=dtype, device=device))
        else:
            self.weight = None
            self.bias = None

    def forward(self, x):
        n = len(self.normalized_shape)
        axis = -1 if n == 1 else tuple(range(-n, 0))
        return F.layer_norm(x, self.weight, self.bias, eps=self.eps, axis=axis)

    def extra_repr(self):
        return f"normalized_shape={self.normalized_shape}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"


class MultiHeadAttention(Module):
    """Multi-head attention with separate q/k/v/out projections on (batch, seq, d_model)."""

    def __init__(self, d_model: int, num_heads: int, dropout: float = 0.0, bias: bool = True, *, dtype=DType.float32,
                 device=None):
        super().__init__()
        if d_model % num_heads != 0:
            raise ValueError(f"d_model ({d_model}) must be divisible by num_heads ({num_heads})")
        self.d_model, self.num_heads, self.head_dim = int(d_model), int(num_heads), d_model // num_heads
        self.dropout_p = float(dropout)
        self.q_proj = Linear(d_model, d_model, bias=bias, dtype=dtype, device=device)
        self.k_proj = Linear(d_model, d_model, bias=bias, dtype=dtype, device=device)
        self.v_proj = Linear(d_model, d_model, bias=bias, dtype=dtype, device=device)
        self.out_proj = Linear(d_model, d_model, bias=bias, dtype=dtype, device=device)

    def _heads(self, x: Tensor, batch: int, seq: int) -> Tensor:
        return swap_axes(reshape(x, (batch, seq, self.num_heads, self.head_dim)), 1, 2)

    def forward(self, query: Tensor, key: Tensor | None = None, value: Tensor | None = None,
                attn_mask: Tensor | None = None, is_causal: bool = False) -> Tensor:
        key = query if key is None else key
        value = key if value is None else value
        b, sq = int(query.shape[0]), int(query.shape[1])
        sk = int(key.shape[1])
        q = self._heads(self.q_proj(query), b, sq)
        k = self._heads(self.k_proj(key), b, sk)
        v = self._heads(self.v_proj(value), b, sk)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, dropout_p=self.dropout_p,
                                           is_causal=is_causal, training=self._training)
        o = reshape(swap_axes(o, 1, 2), (b, sq, self.d_model))
        return self.out_proj(o)

    def extra_repr(self):
        return f"d_model={self.d_model}, num_heads={self.num_heads}, dropout={self.dropout_p}"


class TransformerEncoderLayer(Module):
    """Pre-norm block: x + MHA(LN(x)); x + FFN(LN(x)) with a GELU feed-forward."""

    def __init__(self, d_model: int, num_heads: int, dim_feedforward: int = 2048, dropout: float = 0.1, *,
                 dtype=DType.float32, device=None):
        super().__init__()
        self.self_attn = MultiHeadAttention(d_model, num_heads, dropout=dropout, dtype=dtype, device=device)
        self.linear1 = Linear(d_model, dim_feedforward, dtype=dtype, device=device)
        self.linear2 = Linear(dim_feedforward, d_model, dtype=dtype, device=device)
        self.norm1 = LayerNorm(d_model, dtype=dtype, device=device)
        self.norm2 = LayerNorm(d_model, dtype=dtype, device=device)
        self.dropout1 = Dropout(dropout)        # after the attention, after the feed-forward: the
        self.dropout2 = Dropout(dropout)        # reference's layout (nabla/nn/modules/transformer.py:60-82)

    def forward(self, src: Tensor, src_mask: Tensor | None = None, is_causal: bool = False) -> Tensor:
        h = self.norm1(src)
        x = src + self.dropout1(self.self_attn(h, h, h, attn_mask=src_mask, is_causal=is_causal))
        h = self.norm2(x)
        ff = self.linear2(F.linear(h, self.linear1.weight, self.linear1.bias, activation="gelu"))
        return x + self.dropout2(ff)


class TransformerDecoderLayer(Module):
    """Pre-norm decoder block: (optionally causal) self-attention, cross-attention, GELU feed-forward."""

    def __init__(self, d_model: int, num_heads: int, dim_feedforward: int = 2048, dropout: float = 0.1, *,
                 dtype=DType.float32, device=None):
        super().__init__()
        self.self_attn = MultiHeadAttention(d_model, num_heads, dropout=dropout, dtype=dtype, device=device)
        self.cross_attn = MultiHeadAttention(d_model, num_heads, dropout=dropout, dtype=dtype, device=device)
        self.linear1 = Linear(d_model, dim_feedforward, dtype=dtype, device=device)
        self.linear2 = Linear(dim_feedforward, d_model, dtype=dtype, device=device)
        self.norm1 = LayerNorm(d_model, dtype=dtype, device=device)
        self.norm2 = LayerNorm(d_model, dtype=dtype, device=device)
        self.norm3 = LayerNorm(d_model, dtype=dtype, device=device)
        self.dropout1 = Dropout(dropout)
        self.dropout2 = Dropout(dropout)
        self.dropout3 = Dropout(dropout)

    def forward(self, tgt: Tensor, memory: Tensor, tgt_mask: Tensor | None = None, memory_mask: Tensor | None = None,
                is_causal: bool = False, tgt_is_causal: bool | None = None) -> Tensor:
        """Pre-norm decoder layer. ``is_causal`` masks the self-attention causally (default off, as in
        the reference, nabla/nn/modules/transformer.py:124-131); ``tgt_is_causal`` is an older name for it."""
        if tgt_is_causal is not None:
            is_causal = tgt_is_causal
        h = self.norm1(tgt)
        x = tgt + self.dropout1(self.self_attn(h, h, h, attn_mask=tgt_mask, is_causal=is_causal))
        h = self.norm2(x)
        x = x + self.dropout2(self.cross_attn(h, memory, memory, attn_mask=memory_mask))
        h = self.norm3(x)
        ff = self.linear2(F.linear(h, self.linear1.weight, self.linear1.bias, activation="gelu"))
        return x + self.dropout3(ff)
