"""Deterministic replay check: run the same step several times from the same state and compare bits.

The kernels of this package talk to each other through flags in peer memory, side streams and (in
the release configuration) first-come-first-served job counters. A missing wait or a buffer that
is reused too early shows up as a result that differs from run to run, rarely and only under
load. ``replay_check`` makes that visible and repeatable:

* every run starts from a private deep copy of the arguments (donated / in-place updated state
  included), with the random seed put back to the same value;
* the runs execute under ``config.deterministic()``, which removes every *intended* source of
  run-to-run variation (atomics, in-switch sums, dynamic job order, side streams), so that any
  difference that is left is a bug;
* the outputs (and, optionally, the arguments after the call, which is where in-place optimizer
  updates land) are compared bit for bit with those of the first run.

With more than one rank each rank compares its own shards, and the result is combined over the
process group, so every rank returns the same ``ok``.

The reference has no counterpart (its only concurrency hardening is ContextVar isolation of the
graph and the flags, nabla/core/graph/engine.py:922-1012); this is one of the substitutes for a
race detector, next to the debug-build index checks of ``csrc/nb_debug.cuh``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from .. import config
from ..core.common import pytree
from ..core.graph.engine import GRAPH
from ..core.tensor.api import Tensor
from ..core.tensor.impl import TensorImpl


@dataclass
class Mismatch:
    run: int                 # index of the run that differed from run 0
    leaf: str                # path of the leaf in (outputs, arguments-after-the-call)
    shard: int               # local shard index
    n_diff: int              # number of differing elements
    first_index: int         # flat index of the first differing element
    max_abs_diff: float


@dataclass
class ReplayReport:
    runs: int
    leaves: int
    ok: bool                               # combined over all ranks
    mismatches: list[Mismatch] = field(default_factory=list)   # of this rank

    def __bool__(self) -> bool:
        return self.ok

    def summary(self) -> str:
        if self.ok:
            return f"replay ok: {self.runs} runs, {self.leaves} leaves identical"
        lines = [f"replay differs: {len(self.mismatches)} leaf/run pairs on this rank"]
        for m in self.mismatches[:8]:
            lines.append(f"  run {m.run} {m.leaf}[shard {m.shard}]: {m.n_diff} elements differ, first at {m.first_index}, "
                         f"max |diff| {m.max_abs_diff:.3e}")
        return "\n".join(lines)


def _is_tensor(x: Any) -> bool:
    return isinstance(x, Tensor)


def _copy_leaf(x: Any) -> Any:
    """Private copy of a leaf: same values, sharding and autograd flags, own storage."""
    if isinstance(x, Tensor):
        x.realize()
        src = x._impl
        impl = TensorImpl([b.clone() for b in src._buffers], shape=src._shape, dtype=src.dtype, device=src.device,
                          sharding=src.sharding, batch_dims=src.batch_dims)
        impl.requires_grad = src.requires_grad
        impl.is_traced = src.is_traced
        return Tensor(impl=impl)
    if isinstance(x, torch.Tensor):
        return x.clone()
    return x


def _snapshot(tree: Any) -> list[tuple[str, list[torch.Tensor]]]:
    """(path, [clone of every local shard]) for every tensor leaf of ``tree``."""
    leaves, names, _ = pytree.tree_flatten_with_names(tree, is_leaf=_is_tensor)
    out = []
    for name, leaf in zip(names, leaves):
        if isinstance(leaf, Tensor):
            leaf.realize()
            out.append((name, [b.detach().clone() for b in leaf._impl._buffers]))
        elif isinstance(leaf, torch.Tensor):
            out.append((name, [leaf.detach().clone()]))
    return out


def _bits(t: torch.Tensor) -> torch.Tensor:
    """The tensor's bytes as integers, so that NaNs compare equal to themselves and -0.0 differs from 0.0."""
    t = t.contiguous()
    if t.dtype == torch.bool:
        return t.view(torch.uint8).view(-1)
    width = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
    return t.view(width).view(-1)


def _compare(run: int, ref: list, got: list, sink: list[Mismatch]) -> None:
    for (name, a_shards), (_, b_shards) in zip(ref, got):
        for k, (a, b) in enumerate(zip(a_shards, b_shards)):
            if a.shape != b.shape or a.dtype != b.dtype:
                sink.append(Mismatch(run, name, k, max(a.numel(), b.numel()), 0, float("inf")))
                continue
            if a.numel() == 0:
                continue
            ne = _bits(a) != _bits(b)
            n = int(ne.sum().item())
            if n:
                first = int(torch.nonzero(ne)[0].item())
                d = (a.double() - b.double()).abs()
                d = d[torch.isfinite(d)]
                sink.append(Mismatch(run, name, k, n, first, float(d.max().item()) if d.numel() else float("nan")))


def _combine_over_ranks(ok: bool) -> bool:
    try:
        import torch.distributed as dist
    except Exception:   # pragma: no cover
        return ok
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return ok
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    flag = torch.tensor([0 if ok else 1], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return int(flag.item()) == 0


def _reseed(seed: int) -> None:
    """Put the host-side and every device-resident random stream back to (seed, 0 draws). The device
    states are rewritten in place, so a captured CUDA graph that reads them restarts its stream too."""
    GRAPH.set_seed(seed)
    if torch.cuda.is_available():
        from ..native import kernels

        for dev in list(kernels._rng_states):
            kernels.rng_state(dev)


def replay_check(fn: Callable, *args, repeats: int = 3, seed: int | None = None, check_args: bool = True,
                 deterministic: bool = True, **kwargs) -> ReplayReport:
    """Call ``fn(*args, **kwargs)`` ``repeats`` times, each time on a private copy of the arguments and
    from the same random seed, and compare the results bit for bit with the first run.

    ``fn`` is usually a compiled training step (its donated arguments are why every run gets its own
    copy). ``check_args=True`` also compares the arguments after the call (state that a plain function
    updates in place), except those a compiled function was given with ``donate_argnums``. ``deterministic=False`` runs the release configuration instead, which
    is allowed to differ in the last bit where it uses atomics or in-switch sums: useful to measure how
    much, not as a pass/fail test. The caller's own arguments are never modified."""
    if repeats < 2:
        raise ValueError("replay_check needs at least two runs")
    base_seed = GRAPH.seed if seed is None else int(seed)
    donated = set(getattr(fn, "donate_argnums", ()) or ())
    ref = None
    mismatches: list[Mismatch] = []
    n_leaves = 0
    for run in range(repeats):
        a = pytree.tree_map(_copy_leaf, args, is_leaf=_is_tensor)
        kw = pytree.tree_map(_copy_leaf, kwargs, is_leaf=_is_tensor)
        _reseed(base_seed)
        with config.deterministic(deterministic):
            out = fn(*a, **kw)
        # a donated argument belongs to the function after the call (its contents are unspecified:
        # updated in place on one path, copied into a captured graph's own memory on another)
        kept = tuple(x for i, x in enumerate(a) if i not in donated)
        snap = _snapshot({"out": out, "args": (kept, kw)} if check_args else {"out": out})
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if ref is None:
            ref = snap
            n_leaves = len(snap)
        else:
            _compare(run, ref, snap, mismatches)
    ok = _combine_over_ranks(not mismatches)
    return ReplayReport(runs=repeats, leaves=n_leaves, ok=ok, mismatches=mismatches)
