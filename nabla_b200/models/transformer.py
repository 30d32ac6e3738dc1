"""Decoder-only pre-LayerNorm transformer (the dp x tp benchmark model).

Parameters are a plain pytree of Tensors; tensor parallelism is expressed only through their
shardings (Megatron layout): ``wqkv``/``w1``/``lm_head`` are column-parallel ``P(None, 'tp')``,
``wo``/``w2`` row-parallel ``P('tp', None)``, the batch is ``P('dp', None)``. The sharding
propagation inserts the collectives. ``wqkv`` columns are ordered (head, {q,k,v}, head_dim) so
that splitting the column dim splits heads.

With ``SeqParallel`` the LayerNorm / residual regions keep the tokens split over the tensor-
parallel axis as well (activations ``P('dp', 'tp', None)``): the row-parallel projections end in
a reduce-scatter instead of an all-reduce, the column-parallel ones start with an all-gather,
and no elementwise work is replicated over the tensor-parallel group. Both collectives fuse
with their GEMM (``csrc/gemm_tcgen05.cu``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

from ..core.tensor.api import Tensor
from ..nn import functional as F
from ..ops import fused
from ..ops.creation import arange, gaussian, ones, zeros
from ..ops.view import gather, reshape
from ..types import DType


@dataclass
class TransformerConfig:
    n_layers: int = 24
    d_model: int = 2048
    n_heads: int = 16
    d_ff: int = 8192
    vocab: int = 32000
    max_seq: int = 2048
    dtype: DType = DType.bfloat16
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def num_params(self) -> int:
        d, f, v = self.d_model, self.d_ff, self.vocab
        per_layer = 4 * d * d + 4 * d + 2 * d * f + f + d + 4 * d
        return self.n_layers * per_layer + 2 * v * d + self.max_seq * d + 2 * d

    def flops_per_token(self, seq: int) -> float:
        """Training FLOPs per token: 6 x matmul parameters + causal attention."""
        d, f, v = self.d_model, self.d_ff, self.vocab
        mm = self.n_layers * (4 * d * d + 2 * d * f) + v * d
        attn = self.n_layers * 2 * seq * d      # QK^T and PV, causal halves the 4*s*d
        return 6.0 * mm + 3.0 * attn


@dataclass(frozen=True)
class SeqParallel:
    """Where the token dimension is split between the tensor-parallel regions."""
    mesh: Any
    dp_axis: str | None = "dp"
    tp_axis: str = "tp"

    def tokens_split(self, x: Tensor) -> Tensor:      # (B, S, D) -> P(dp, tp, None)
        return x.shard(self.mesh, (self.dp_axis, self.tp_axis, None))

    def tokens_whole(self, x: Tensor) -> Tensor:      # (B, S, D) -> P(dp, None, None)
        return x.shard(self.mesh, (self.dp_axis, None, None))


def init_params(cfg: TransformerConfig, mesh=None, tp_axis: str | None = "tp", device=None) -> dict[str, Any]:
    """Random-normal weights (std ``init_std``), zero biases, unit LayerNorm gains."""
    dt = cfg.dtype
    d, f, v = cfg.d_model, cfg.d_ff, cfg.vocab

    def col(t):   # split output features
        return t.shard(mesh, (None, tp_axis)) if mesh is not None and tp_axis else t

    def row(t):   # split input features
        return t.shard(mesh, (tp_axis, None)) if mesh is not None and tp_axis else t

    def vec_col(t):
        return t.shard(mesh, (tp_axis,)) if mesh is not None and tp_axis else t

    def rep(t):
        return t.shard(mesh, tuple(None for _ in t.shape)) if mesh is not None else t

    def w(shape, std=cfg.init_std):
        return gaussian(shape, 0.0, std, dtype=dt, device=device)

    layers = []
    out_std = cfg.init_std / math.sqrt(2 * cfg.n_layers)
    for _ in range(cfg.n_layers):
        layers.append({
            "ln1_g": rep(ones((d,), dtype=dt, device=device)), "ln1_b": rep(zeros((d,), dtype=dt, device=device)),
            "wqkv": col(w((d, 3 * d))), "bqkv": vec_col(zeros((3 * d,), dtype=dt, device=device)),
            "wo": row(w((d, d), out_std)), "bo": rep(zeros((d,), dtype=dt, device=device)),
            "ln2_g": rep(ones((d,), dtype=dt, device=device)), "ln2_b": rep(zeros((d,), dtype=dt, device=device)),
            "w1": col(w((d, f))), "b1": vec_col(zeros((f,), dtype=dt, device=device)),
            "w2": row(w((f, d), out_std)), "b2": rep(zeros((d,), dtype=dt, device=device)),
        })
    return {
        "tok_emb": rep(w((v, d))), "pos_emb": rep(w((cfg.max_seq, d))),
        "layers": layers,
        "lnf_g": rep(ones((d,), dtype=dt, device=device)), "lnf_b": rep(zeros((d,), dtype=dt, device=device)),
        "lm_head": col(w((d, v))),
    }


def init_lora(params: dict[str, Any], cfg: TransformerConfig, rank: int = 16, init_std: float = 0.02, mesh=None,
              tp_axis: str | None = "tp") -> list[dict[str, Any]]:
    """Rank-``rank`` adapters (A ~ N(0, init_std), B = 0) on the q/k/v (packed) and o projections of
    every layer. With a mesh the adapters follow their frozen weight's split: for the column-parallel
    ``wqkv`` B is split over ``tp_axis``, for the row-parallel ``wo`` A is."""
    from ..nn.finetune.lora import init_lora_adapter

    out = []
    for L in params["layers"]:
        qkv = init_lora_adapter(L["wqkv"], rank, init_std)
        o = init_lora_adapter(L["wo"], rank, init_std)
        if mesh is not None and tp_axis:
            qkv = {"A": qkv["A"].shard(mesh, (None, None)), "B": qkv["B"].shard(mesh, (None, tp_axis))}
            o = {"A": o["A"].shard(mesh, (tp_axis, None)), "B": o["B"].shard(mesh, (None, None))}
        out.append({"qkv": qkv, "o": o})
    return out


def _lora_linear(x: Tensor, w: Tensor, b: Tensor | None, ad: dict[str, Tensor] | None, alpha: float) -> Tensor:
    y = F.linear(x, w, b)
    if ad is None:
        return y
    A, B = ad["A"], ad["B"]
    return y + ((x @ A) @ B) * (alpha / float(int(A.shape[1])))


def block(x: Tensor, p: dict[str, Tensor], cfg: TransformerConfig, sp: SeqParallel | None = None,
          lora: dict[str, Any] | None = None, lora_alpha: float = 16.0) -> Tensor:
    if lora is not None:
        h = F.layer_norm(x, p["ln1_g"], p["ln1_b"])
        qkv = _lora_linear(h, p["wqkv"], p["bqkv"], lora["qkv"], lora_alpha)
        a = fused.packed_self_attention(qkv, cfg.head_dim, causal=True)
        x = x + _lora_linear(a, p["wo"], p["bo"], lora["o"], lora_alpha)
        h = F.layer_norm(x, p["ln2_g"], p["ln2_b"])
        m = F.linear(h, p["w1"], p["b1"], activation="gelu")
        return x + F.linear(m, p["w2"], p["b2"])
    if sp is None:
        h = F.layer_norm(x, p["ln1_g"], p["ln1_b"])
        qkv = F.linear(h, p["wqkv"], p["bqkv"])
        a = fused.packed_self_attention(qkv, cfg.head_dim, causal=True)
        x = x + F.linear(a, p["wo"], p["bo"])
        h = F.layer_norm(x, p["ln2_g"], p["ln2_b"])
        m = F.linear(h, p["w1"], p["b1"], activation="gelu")
        return x + F.linear(m, p["w2"], p["b2"])
    # tokens split over tp outside the projections: gather -> column-parallel -> row-parallel -> scatter
    h = sp.tokens_whole(F.layer_norm(x, p["ln1_g"], p["ln1_b"]))
    qkv = F.linear(h, p["wqkv"], p["bqkv"])
    a = fused.packed_self_attention(qkv, cfg.head_dim, causal=True)
    x = x + (sp.tokens_split(F.linear(a, p["wo"])) + p["bo"])
    h = sp.tokens_whole(F.layer_norm(x, p["ln2_g"], p["ln2_b"]))
    m = F.linear(h, p["w1"], p["b1"], activation="gelu")
    return x + (sp.tokens_split(F.linear(m, p["w2"])) + p["b2"])


def forward(params: dict[str, Any], tokens: Tensor, cfg: TransformerConfig, sp: SeqParallel | None = None,
            lora: list[dict[str, Any]] | None = None) -> Tensor:
    """tokens (B, S) int64 -> logits (B, S, vocab)."""
    S = int(tokens.shape[1])
    x = gather(params["tok_emb"], tokens, axis=0)
    pos = params["pos_emb"]
    if int(pos.shape[0]) != S:
        pos = pos[:S]
    x = x + pos
    if sp is not None:
        x = sp.tokens_split(x)
    for li, p in enumerate(params["layers"]):
        x = block(x, p, cfg, sp, lora[li] if lora is not None else None)
    x = F.layer_norm(x, params["lnf_g"], params["lnf_b"])
    if sp is not None:
        x = sp.tokens_whole(x)
    return F.linear(x, params["lm_head"])


def loss_fn(params: dict[str, Any], tokens: Tensor, targets: Tensor, cfg: TransformerConfig,
            sp: SeqParallel | None = None, lora: list[dict[str, Any]] | None = None) -> Tensor:
    """Mean next-token cross-entropy over all positions (fp32 scalar)."""
    from ..ops.reduction import reduce_sum

    logits = forward(params, tokens, cfg, sp, lora)
    rows = fused.cross_entropy_rows(logits, targets)
    n = int(tokens.shape[0]) * int(tokens.shape[1])
    return reduce_sum(rows) * (1.0 / n)


def place_params(params: dict[str, Any], mesh, tp_axis: str = "tp") -> dict[str, Any]:
    """Lay an unsharded parameter tree out on ``mesh`` (Megatron column/row split over ``tp_axis``)."""
    out = {k: v for k, v in params.items() if k != "layers"}
    out["lm_head"] = params["lm_head"].shard(mesh, (None, tp_axis))
    out["layers"] = []
    for L in params["layers"]:
        out["layers"].append({**L, "wqkv": L["wqkv"].shard(mesh, (None, tp_axis)), "bqkv": L["bqkv"].shard(mesh, (tp_axis,)),
                              "wo": L["wo"].shard(mesh, (tp_axis, None)), "w1": L["w1"].shard(mesh, (None, tp_axis)),
                              "b1": L["b1"].shard(mesh, (tp_axis,)), "w2": L["w2"].shard(mesh, (tp_axis, None))})
    return out


def torch_reference_forward(params: dict[str, Any], tokens, cfg: TransformerConfig):
    """Plain PyTorch fp32 implementation of the same architecture (test oracle)."""
    import torch
    import torch.nn.functional as TF

    def t(x):
        return torch.from_numpy(x.to_numpy()).float()

    x = t(params["tok_emb"])[tokens] + t(params["pos_emb"])[: tokens.shape[1]]
    B, S, d = x.shape
    H, hd = cfg.n_heads, cfg.head_dim
    for p in params["layers"]:
        h = TF.layer_norm(x, (d,), t(p["ln1_g"]), t(p["ln1_b"]))
        qkv = (h @ t(p["wqkv"]) + t(p["bqkv"])).view(B, S, H, 3, hd)
        q, k, v = (qkv[:, :, :, i].transpose(1, 2) for i in range(3))
        a = TF.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, d)
        x = x + a @ t(p["wo"]) + t(p["bo"])
        h = TF.layer_norm(x, (d,), t(p["ln2_g"]), t(p["ln2_b"]))
        x = x + TF.gelu(h @ t(p["w1"]) + t(p["b1"])) @ t(p["w2"]) + t(p["b2"])
    x = TF.layer_norm(x, (d,), t(params["lnf_g"]), t(params["lnf_b"]))
    return x @ t(params["lm_head"])
