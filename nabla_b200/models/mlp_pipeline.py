"""GPipe-style pipeline parallel MLP (the GPipe and PP x DP configurations; reference recipe:
examples/07_mlp_pipeline_parallel.ipynb, examples/08_mlp_pp_dp_training.ipynb).

Per-stage weights are stacked on a leading axis split over the ``stage`` mesh axis;
``vmap(stage_fn, spmd_axis_name='stage')`` runs all stages at once on their own devices;
``ppermute`` shifts activations one stage down the pipe each tick; micro-batches are injected
at stage 0 with ``where`` masks and collected from the last stage. ``grad`` differentiates
through the whole unrolled schedule (the VJP of ``ppermute`` is the inverse shift).
"""
from __future__ import annotations

from typing import Any

import numpy as np

from ..core.tensor.api import Tensor
from ..ops.binary import matmul
from ..ops.communication import ppermute, shard
from ..ops.control_flow import where
from ..ops.creation import constant, zeros
from ..ops.reduction import mean, reduce_sum
from ..ops.unary import cast, relu
from ..types import DType
from ..ops.view import broadcast_to, reshape, stack, unsqueeze
from ..transforms.vmap import vmap


def place_stage_params(t: Tensor, mesh, stage_axis: str = "stage") -> Tensor:
    """Split the leading (stage) dimension over the stage axis of the mesh."""
    return shard(t, mesh, (stage_axis,) + (None,) * (t.rank - 1))


def _stage_fn(x, w, b):
    return relu(matmul(x, w) + b)


def _stage_fn2(x, w1, b1, w2, b2):
    """Two Linear + relu per stage (the PP x DP configuration)."""
    return relu(matmul(relu(matmul(x, w1) + b1), w2) + b2)


def _stage_mask(n_stages: int, index: int, like: Tensor, mesh, stage_axis: str) -> Tensor:
    """(S,1,1) boolean selecting one stage, laid out over the stage axis."""
    m = np.zeros((n_stages, 1, 1), dtype=bool)
    m[index] = True
    return shard(constant(m, device=like.device), mesh, (stage_axis, None, None))


def _perm(mesh, stage_axis: str) -> list[tuple[int, int]]:
    """i -> i+1 along the stage axis inside every replica group (no wrap-around)."""
    n = mesh.get_axis_size(stage_axis)
    perm = []
    for d in range(mesh.size):
        c = mesh.get_coordinate(d, stage_axis)
        if c + 1 < n:
            group = mesh.group_of(d, [stage_axis])
            perm.append((d, group[c + 1]))
    return perm


def gpipe_forward(w, b, xs: Tensor, mesh, stage_axis: str = "stage", dp_axis: str | None = None) -> Tensor:
    """Run ``xs`` (micro_batches, batch, dim) through the S-stage pipe; returns the last stage's
    outputs, shape (micro_batches, batch, dim). ``w`` / ``b`` are the stacked (S, ...) stage
    parameters, or pairs ``(w1, w2)`` / ``(b1, b2)`` for stages of two Linear + relu."""
    S = mesh.get_axis_size(stage_axis)
    MB, B, D = (int(d) for d in xs.shape)
    two = isinstance(w, (tuple, list))
    if two:
        step2 = vmap(_stage_fn2, in_axes=(0, 0, 0, 0, 0), spmd_axis_name=stage_axis, mesh=mesh)
        step = lambda x_, w_, b_: step2(x_, w[0], unsqueeze(b[0], axis=1), w[1], unsqueeze(b[1], axis=1))
    else:
        step = vmap(_stage_fn, in_axes=(0, 0, 0), spmd_axis_name=stage_axis, mesh=mesh)
    state_spec = (stage_axis, dp_axis, None)
    state = shard(zeros((S, B, D), dtype=xs.dtype, device=xs.device), mesh, state_spec)
    first = _stage_mask(S, 0, xs, mesh, stage_axis)
    last = _stage_mask(S, S - 1, xs, mesh, stage_axis)
    perm = _perm(mesh, stage_axis)
    zero_x = zeros((B, D), dtype=xs.dtype, device=xs.device)
    outs = []
    for t in range(MB + S - 1):
        fresh = xs[t] if t < MB else zero_x
        fresh = shard(broadcast_to(unsqueeze(fresh, axis=0), (S, B, D)), mesh, state_spec)
        inp = where(first, fresh, state)
        computed = step(inp, w, None if two else unsqueeze(b, axis=1))
        if t >= S - 1:
            # the last stage's row, extracted by masking and summing over the stage axis
            outs.append(reduce_sum(where(last, computed, zeros_like_state(computed)), axis=0))
        state = ppermute(computed, perm)
    return stack(outs, axis=0)


def zeros_like_state(t: Tensor) -> Tensor:
    from ..ops.creation import zeros_like

    return zeros_like(t)


def gpipe_loss(w, b, xs: Tensor, ys: Tensor, mesh, stage_axis: str = "stage",
               dp_axis: str | None = None) -> Tensor:
    """Mean squared error of the pipe's outputs against ``ys`` (micro_batches, batch, dim).

    The outputs never leave the last stage and no tick does any loss arithmetic: every stage keeps
    what it computed in the ticks that matter (t >= S - 1) and, after the last tick, ONE masked
    difference against the targets, one square and one reduction over the stacked
    (S, micro_batches, batch, dim) tensor give the loss (fp32 accumulation). A tick is therefore the
    stage's GEMM, the input select and the ``ppermute`` shift, nothing else, where the reference
    recipe (examples/07_mlp_pipeline_parallel.ipynb) sums a masked (S, batch, dim) tensor over the
    stage axis every tick."""
    S = mesh.get_axis_size(stage_axis)
    MB, B, D = (int(d) for d in xs.shape)
    two = isinstance(w, (tuple, list))
    if two:
        step2 = vmap(_stage_fn2, in_axes=(0, 0, 0, 0, 0), spmd_axis_name=stage_axis, mesh=mesh)
        step = lambda x_, w_, b_: step2(x_, w[0], unsqueeze(b[0], axis=1), w[1], unsqueeze(b[1], axis=1))
    else:
        step = vmap(_stage_fn, in_axes=(0, 0, 0), spmd_axis_name=stage_axis, mesh=mesh)
    state_spec = (stage_axis, dp_axis, None)
    state = shard(zeros((S, B, D), dtype=xs.dtype, device=xs.device), mesh, state_spec)
    first = _stage_mask(S, 0, xs, mesh, stage_axis)
    perm = _perm(mesh, stage_axis)
    zero_x = zeros((B, D), dtype=xs.dtype, device=xs.device)
    kept = []
    for t in range(MB + S - 1):
        fresh = xs[t] if t < MB else zero_x
        fresh = shard(broadcast_to(unsqueeze(fresh, axis=0), (S, B, D)), mesh, state_spec)
        inp = where(first, fresh, state)
        computed = step(inp, w, None if two else unsqueeze(b, axis=1))
        if t >= S - 1:
            kept.append(computed)
        if t + 1 < MB + S - 1:
            state = ppermute(computed, perm)
    all_spec = (stage_axis, None, dp_axis, None)
    got = shard(stack(kept, axis=1), mesh, all_spec)                                   # (S, MB, B, D)
    want = shard(broadcast_to(unsqueeze(ys, axis=0), (S, MB, B, D)), mesh, all_spec)
    m = np.zeros((S, 1, 1, 1), dtype=bool)
    m[S - 1] = True
    last = shard(constant(m, device=xs.device), mesh, (stage_axis, None, None, None))
    d = cast(where(last, got - want, zeros_like_state(got)), DType.float32)
    e = reduce_sum(reduce_sum(reduce_sum(d * d, axis=3), axis=2), axis=1)              # (S,), one value per stage
    return reduce_sum(e, axis=0) * (1.0 / float(MB * B * D))
