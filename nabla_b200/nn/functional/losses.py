"""Losses (reference: nabla/nn/functional/losses.py:14-77)."""
from __future__ import annotations

from ...core.tensor.api import Tensor
from ...ops import fused
from ...ops.comparison import equal
from ...ops.creation import arange
from ...ops.reduction import mean, reduce_sum
from ...ops.unary import cast, logsoftmax
from ...ops.view import unsqueeze


def mse_loss(predictions: Tensor, targets: Tensor) -> Tensor:
    diff = predictions - targets
    return mean(diff * diff)


def _one_hot(indices: Tensor, num_classes: int, dtype=None) -> Tensor:
    classes = arange(0, num_classes, 1, dtype=indices.dtype, device=indices.device)
    mask = equal(unsqueeze(indices, -1), classes)
    return cast(mask, dtype) if dtype is not None else mask


def cross_entropy_loss_reference(logits: Tensor, targets: Tensor, axis: int = -1) -> Tensor:
    log_probs = logsoftmax(logits, axis=axis)
    if len(targets.shape) < len(logits.shape):
        targets = _one_hot(targets, num_classes=int(logits.shape[axis]), dtype=logits.dtype)
    return -reduce_sum(targets * log_probs) / float(int(logits.shape[0]))


def cross_entropy_loss(logits: Tensor, targets: Tensor, axis: int = -1) -> Tensor:
    """Sum of per-position cross-entropies divided by ``logits.shape[0]`` (the reference's
    convention). ``targets``: one-hot like ``logits`` or integer class indices."""
    from .layers import use_fused

    int_targets = len(targets.shape) < len(logits.shape)
    last = axis in (-1, logits.rank - 1)
    if int_targets and last and use_fused(logits):
        rows = fused.cross_entropy_rows(logits, targets)
        return reduce_sum(rows) / float(int(logits.shape[0]))
    return cross_entropy_loss_reference(logits, targets, axis)
