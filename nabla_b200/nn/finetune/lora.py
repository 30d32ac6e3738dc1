"""LoRA helpers (reference: nabla/nn/finetune/lora.py:16-127)."""
from __future__ import annotations

from typing import Any

from ...core.common.pytree import tree_map
from ...core.tensor.api import Tensor
from ...ops.creation import gaussian, zeros


def init_lora_adapter(weight: Tensor, rank: int, init_std: float = 0.01, dtype=None) -> dict[str, Tensor]:
    """``{'A': (in, rank) ~ N(0, init_std), 'B': (rank, out) = 0}`` for a frozen (in, out) weight."""
    if len(weight.shape) != 2:
        raise ValueError("init_lora_adapter expects a 2D weight tensor")
    if rank <= 0:
        raise ValueError("rank must be > 0")
    fin, fout = int(weight.shape[0]), int(weight.shape[1])
    dt = dtype or weight.dtype
    return {"A": gaussian((fin, rank), mean=0.0, std=init_std, dtype=dt, device=weight.device),
            "B": zeros((rank, fout), dtype=dt, device=weight.device)}


def lora_delta(adapter: dict[str, Tensor], alpha: float = 1.0) -> Tensor:
    """``(alpha / rank) * A @ B`` of shape (in, out)."""
    A, B = adapter["A"], adapter["B"]
    return (A @ B) * (alpha / float(int(A.shape[1])))


def lora_linear(x: Tensor, frozen_weight: Tensor, adapter: dict[str, Tensor], alpha: float = 1.0) -> Tensor:
    """``x @ W + (alpha/r) (x @ A) @ B``. The low-rank path is applied as two thin GEMMs, which
    equals the reference's ``x @ (A @ B)`` but never forms the dense (in, out) delta."""
    A, B = adapter["A"], adapter["B"]
    scale = alpha / float(int(A.shape[1]))
    return (x @ frozen_weight) + ((x @ A) @ B) * scale


def merge_lora_weight(frozen_weight: Tensor, adapter: dict[str, Tensor], alpha: float = 1.0) -> Tensor:
    return frozen_weight + lora_delta(adapter, alpha=alpha)


def unmerge_lora_weight(merged_weight: Tensor, adapter: dict[str, Tensor], alpha: float = 1.0) -> Tensor:
    return merged_weight - lora_delta(adapter, alpha=alpha)


def tree_lora_delta(adapters: Any, alpha: float = 1.0, *, is_leaf: Any = None) -> Any:
    def is_adapter(x):
        return (isinstance(x, dict) and "A" in x and "B" in x) or (is_leaf is not None and is_leaf(x))

    def f(leaf):
        if isinstance(leaf, dict) and "A" in leaf and "B" in leaf:
            return lora_delta(leaf, alpha=alpha)
        return leaf

    return tree_map(f, adapters, is_leaf=is_adapter)
