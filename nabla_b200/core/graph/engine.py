"""Lazy evaluation engine (reference: nabla/core/graph/engine.py:119-1012).

``GRAPH.evaluate(*tensors)`` realizes promise tensors: it collects the unrealized producer
subgraph, orders it topologically, looks up / builds an execution *plan* keyed by the
structural hash of that subgraph (op identities, static arguments, input signatures), and runs
the plan step by step on torch buffers — hand-written CUDA kernels for the hot ops on GPU.
A plan may fuse neighbouring nodes (``matmul -> add(bias) -> relu/gelu`` into one GEMM
epilogue). Buffers of intermediates are released as soon as their last consumer has run,
because executed untraced nodes drop their references immediately.

The reference compiles each new subgraph with MAX and caches the executable; here the cached
object is the fused schedule, and the counters (`get_cache_stats`) keep the same meaning.
"""
from __future__ import annotations

import os
import time
from contextvars import ContextVar
from typing import Any

import torch

from ..tensor.impl import TensorImpl
from .tracing import OpNode, topo_nodes

DEBUG = os.environ.get("NABLA_DEBUG", "0") == "1"
DEBUG_CACHE = os.environ.get("NABLA_DEBUG_CACHE", "0") == "1"

_GRAPH_CACHE: dict[Any, "Plan"] = {}
_STATS = {"hits": 0, "misses": 0, "invalidations": 0, "evaluations": 0, "nodes_executed": 0}


def get_cache_stats() -> dict:
    s = dict(_STATS)
    total = s["hits"] + s["misses"]
    s["hit_rate"] = s["hits"] / total if total else 0.0
    s["size"] = len(_GRAPH_CACHE)
    return s


def reset_cache_stats() -> None:
    for k in _STATS:
        _STATS[k] = 0


def clear_cache() -> None:
    if _GRAPH_CACHE:
        _STATS["invalidations"] += len(_GRAPH_CACHE)
    _GRAPH_CACHE.clear()


def _freeze(v: Any) -> Any:
    if isinstance(v, (str, int, float, bool, type(None), bytes)):
        return v
    if isinstance(v, (tuple, list)):
        return tuple(_freeze(x) for x in v)
    if isinstance(v, dict):
        return tuple((k, _freeze(x)) for k, x in sorted(v.items(), key=lambda kv: str(kv[0])))
    if isinstance(v, (set, frozenset)):
        return tuple(sorted((_freeze(x) for x in v), key=repr))
    if hasattr(v, "effect_signature"):
        return v.effect_signature()
    if isinstance(v, torch.Tensor):
        return ("tensor", id(v))
    try:
        hash(v)
        return v
    except TypeError:
        return repr(v)


def _leaf_signature(impl: TensorImpl) -> tuple:
    sh = impl.sharding.effect_signature() if impl.sharding is not None else None
    return (impl._shape, impl._dtype, sh, impl.batch_dims)


def structural_key(nodes: list[OpNode], targets: list[TensorImpl]) -> tuple:
    """Hashable identity of a subgraph: same key <=> same schedule is valid."""
    pos: dict[int, tuple[int, int]] = {}
    parts = []
    for ni, n in enumerate(nodes):
        ins = []
        for a in n.arg_leaves:
            if isinstance(a, TensorImpl):
                p = pos.get(id(a))
                ins.append(p if p is not None else _leaf_signature(a))
            else:
                ins.append(("s", _freeze(a)))
        if n._hash is None:
            n._hash = (n.op.name, _freeze(n.kwargs))
        parts.append((n._hash, tuple(ins)))
        for oi, r in enumerate(n.out_refs):
            o = r()
            if o is not None:
                pos[id(o)] = (ni, oi)
    tg = tuple(pos.get(id(t), ("leaf",)) for t in targets)
    return (tuple(parts), tg)


class Plan:
    """Cached schedule for one subgraph structure: a list of steps, each a tuple
    ``(kind, node_indices)`` where ``kind`` is 'op' (run the node's op) or the name of a
    fused pattern handled by ``nabla_b200.core.graph.fusion``."""

    __slots__ = ("steps", "num_nodes")

    def __init__(self, steps, num_nodes):
        self.steps = steps
        self.num_nodes = num_nodes


# evaluation counter of the current context (the reference's `_GRAPH_EPOCH`, engine.py:30): bumped
# together with `ComputeGraph.epoch`, so code that only has the context can tell two evaluations apart
_GRAPH_EPOCH: ContextVar[int] = ContextVar("nabla_graph_epoch", default=0)


class ComputeGraph:
    """Owner of evaluation state: epoch counter and RNG (seed, counter)."""

    def __init__(self, context=None, seed: int = 0) -> None:
        # (`context` is the reference's MLIR context: there is none here, the argument is accepted and unused)
        # a fresh graph starts a new epoch of its context (the reference's constructor does the same,
        # nabla/core/graph/engine.py), so `epoch` is positive from the start
        self.epoch = _GRAPH_EPOCH.get() + 1
        _GRAPH_EPOCH.set(self.epoch)
        self.seed = int(seed)
        self.rng_counter = 0
        self.seed_epoch = 0          # bumped by set_seed: device-resident stream states re-read (seed, counter)
        # attributes of the reference's graph object (nabla/core/graph/engine.py). There `graph` is the
        # MAX graph under construction and `sources` / `unrealized` its inputs and pending outputs;
        # evaluation here walks the trace from the requested tensors, so these only identify the
        # context's graph object and stay empty.
        self.graph = self
        self.sources: dict = {}
        self.unrealized: dict = {}

    # ---- RNG: counter-based, carried by the engine across evaluations
    def set_seed(self, seed: int) -> None:
        self.seed = int(seed)
        self.rng_counter = 0
        self.seed_epoch += 1

    def next_rng(self) -> tuple[int, int]:
        c = self.rng_counter
        self.rng_counter += 1
        return self.seed, c

    # ---- evaluation
    def evaluate(self, tensor=None, *extra_outputs, return_model: bool = False) -> None:
        tensors = (() if tensor is None else (tensor,)) + tuple(extra_outputs)
        targets: list[TensorImpl] = []
        seen: set[int] = set()
        for t in tensors:
            impl = t._impl if hasattr(t, "_impl") else t
            if isinstance(impl, TensorImpl) and not impl.is_realized and id(impl) not in seen:
                seen.add(id(impl))
                targets.append(impl)
        if not targets:
            return
        t0 = time.perf_counter() if DEBUG else 0.0
        nodes = topo_nodes(targets, lambda impl: impl.is_realized)
        _STATS["evaluations"] += 1
        from . import fusion

        plan = None
        if fusion.enabled():
            key = structural_key(nodes, targets)
            plan = _GRAPH_CACHE.get(key)
            if plan is None:
                _STATS["misses"] += 1
                plan = fusion.build_plan(nodes, targets)
                _GRAPH_CACHE[key] = plan
                if DEBUG_CACHE:
                    print(f"[nabla cache] miss: {len(nodes)} nodes -> {len(plan.steps)} steps; {get_cache_stats()}")
            else:
                _STATS["hits"] += 1
                if DEBUG_CACHE:
                    print(f"[nabla cache] hit; {get_cache_stats()}")
        t1 = time.perf_counter() if DEBUG else 0.0
        self._run(nodes, plan)
        self.epoch += 1
        _GRAPH_EPOCH.set(_GRAPH_EPOCH.get() + 1)
        for t in targets:
            if not t.is_realized:
                raise RuntimeError("evaluate() finished but a target tensor is still unrealized")
        if DEBUG:
            t2 = time.perf_counter()
            print(f"[nabla] evaluate: {len(nodes)} nodes, plan {1e3 * (t1 - t0):.2f} ms, run {1e3 * (t2 - t1):.2f} ms")

    def _run(self, nodes: list[OpNode], plan: Plan | None) -> None:
        _STATS["nodes_executed"] += len(nodes)
        if plan is None:
            for i in range(len(nodes)):
                node = nodes[i]
                nodes[i] = None
                run_node(node)
            return
        from . import fusion

        for kind, idxs in plan.steps:
            if kind == "op":
                node = nodes[idxs[0]]
                nodes[idxs[0]] = None
                run_node(node)
            else:
                group = [nodes[i] for i in idxs]
                for i in idxs:
                    nodes[i] = None
                fusion.run_fused(kind, group)

    def clear_all(self) -> None:
        clear_cache()
        self.epoch += 1
        _GRAPH_EPOCH.set(_GRAPH_EPOCH.get() + 1)


def store_outputs(node: OpNode, outs: list[list[torch.Tensor]]) -> None:
    """Attach produced shard buffers to the node's live outputs and drop the producer link
    of untraced outputs (which frees upstream intermediates by reference counting)."""
    for i, ref in enumerate(node.out_refs):
        impl = ref()
        if impl is None:
            continue
        impl._buffers = outs[i]
        if not impl.is_traced:
            impl.output_refs = None


def run_node(node: OpNode) -> None:
    outs = node.op.execute(node)
    store_outputs(node, outs)


_UNSET = object()
# per-context graph. Three states: never set in this context (the process-wide graph is used), set
# to a graph (`GRAPH.use`), or set to None, which asks for a fresh graph on the next access: a server
# does that on a copied context so that each request handler gets its own (reference: engine.py:922).
_GRAPH_VAR: ContextVar = ContextVar("nabla_graph", default=_UNSET)
_CURRENT_GRAPH = _GRAPH_VAR          # the reference's name for the per-context graph variable
_DEFAULT_GRAPH = ComputeGraph()


def _get_current_graph() -> ComputeGraph:
    """The graph of the current context (reference: nabla/core/graph/engine.py, same name)."""
    g = _GRAPH_VAR.get()
    if g is _UNSET:
        return _DEFAULT_GRAPH
    if g is None:
        g = ComputeGraph()
        _GRAPH_VAR.set(g)
    return g


class _GraphProxy:
    """ContextVar-backed proxy: each context (thread / asyncio task that copied its context)
    may install its own ``ComputeGraph``; otherwise the process-wide one is used."""

    def _get(self) -> ComputeGraph:
        return _get_current_graph()

    def __getattr__(self, name):
        return getattr(self._get(), name)

    def __setattr__(self, name, value):
        setattr(self._get(), name, value)

    def use(self, graph: ComputeGraph):
        return _GRAPH_VAR.set(graph)


GRAPH = _GraphProxy()


def seed(value: int) -> None:
    """Set the global RNG seed used by ``uniform`` / ``gaussian`` / ``dropout``."""
    GRAPH.set_seed(value)


def driver_tensor_type(t):
    """(shape, dtype, device) of a realized buffer: what the engine needs to know about an input
    (reference: nabla/core/graph/engine.py:91, which returns the MAX graph tensor type of a driver
    buffer; the buffers here are torch tensors)."""
    from ...types import as_dtype

    return tuple(int(d) for d in t.shape), as_dtype(t.dtype), t.device
