"""``compile`` (reference: nabla/transforms/compile.py:40-602).

The first call with a new signature runs the Python function ONCE on placeholder tensors,
recording a private graph of ``OpNode``s; later calls skip the Python function and the op
pipeline (no shape inference, no sharding propagation): they bind the new input buffers to
the placeholders and replay the recorded, fused schedule, freeing every intermediate right
after its last use. With ``cuda_graph=True`` the replay is captured into a CUDA graph so a
launch-bound step costs one graph launch.

``donate_argnums=(i, ...)`` hands the buffers of those arguments to the function: optimizer-step
ops that are the last reader of a donated parameter / moment update it in place, so the returned
parameters ARE the argument's buffers (no 3x parameter-size allocation per step, and under
``cuda_graph=True`` no copy in or out: feed the returned tree back in). The caller must not use
a donated argument after the call. Outputs of a CUDA-graph replay that do not alias a donated
input are copied out of the graph's memory; those that do are returned as they are.

Cache key = (pytree structure, per-tensor (shape, dtype, sharding signature), static values);
dimensions named in ``dynamic_dims={arg_idx: {dim_idx: "name"}}`` enter the key as ``"$name"``
so all sizes share one entry. The first call of such an entry traces the Python function twice,
once on the real inputs and once, without executing anything, on placeholders whose named
dimensions are doubled; every integer that differs between the two recordings (reshape targets,
slice bounds, creation shapes...) is an affine function of the named sizes. A later call with
new sizes does not run the Python function: the recorded node list is instantiated for the new
sizes (shape-valued arguments evaluated from those functions, output shapes re-inferred node by
node) and planned again (reference: one executable with SymbolicDim inputs,
nabla/transforms/compile.py:276-301). ``stats.retraces`` counts real re-runs of the Python
function, ``stats.respecialisations`` the instantiations.

``cond`` / ``while_loop`` inside the function become recorded nodes that decide again on every
replay (``ops/control_flow.py``); a schedule that contains one is replayed without CUDA-graph
capture. Random ops read a stream position that lives on the device, so replays (captured or not)
draw fresh numbers.
"""
from __future__ import annotations

import time
import weakref
from collections import OrderedDict
from fractions import Fraction
from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from .. import config
from ..core.common import pytree
from ..core.graph import fusion
from ..core.graph.engine import GRAPH, _STATS, store_outputs
from ..core.graph.tracing import OpNode, topo_nodes
from ..core.tensor.api import Tensor
from ..core.tensor.impl import TensorImpl


import os as _os

_NVTX = _os.environ.get("NABLA_B200_NVTX", "0") == "1"
_SPEC_SIG: dict[int, tuple] = {}      # id(ShardingSpec) -> (spec, effect signature)


@dataclass
class CompilationStats:
    hits: int = 0
    misses: int = 0
    fallbacks: int = 0
    retraces: int = 0
    respecialisations: int = 0       # new sizes of a dynamic_dims entry served without re-running the function
    compile_time_s: float = 0.0
    replay_time_s: float = 0.0
    graph_nodes: int = 0
    graph_steps: int = 0
    cuda_graphs: int = 0
    launches_per_graph: int = 0      # this package's kernels inside the last captured CUDA graph

    cache_size: int = 0              # entries in the LRU cache of the owning CompiledFunction

    # the reference's field names (nabla/transforms/compile.py:48-58), in milliseconds
    @property
    def total_compile_time_ms(self) -> float:
        return self.compile_time_s * 1e3

    @property
    def total_cached_exec_time_ms(self) -> float:
        return self.replay_time_s * 1e3

    @property
    def hit_rate(self) -> float:
        t = self.hits + self.misses
        return self.hits / t if t else 0.0

    def __repr__(self) -> str:
        return (f"CompilationStats(hits={self.hits}, misses={self.misses}, fallbacks={self.fallbacks}, "
                f"hit_rate={self.hit_rate:.1%}, compile_time={self.compile_time_s * 1e3:.2f}ms, "
                f"nodes={self.graph_nodes}, steps={self.graph_steps})")


def _static_values_agree(base: "_Recorded", probe: "_Recorded") -> bool:
    """Only INTEGERS may move with a dynamic size (they are re-evaluated affinely). A float, a string
    or a constant tensor whose VALUE differs between the two recordings was computed from the size
    in Python (``1.0 / n``, an index table built from ``n``): such a function is recorded per size."""
    def same(a, b) -> bool:
        if isinstance(a, TensorImpl) or isinstance(b, TensorImpl):
            if not (isinstance(a, TensorImpl) and isinstance(b, TensorImpl)):
                return False
            if a is b or a._buffers is None or b._buffers is None or a.output_refs is not None or b.output_refs is not None:
                return True                     # the same captured tensor, or a value computed inside the recording
            if len(a._buffers) != len(b._buffers):
                return False
            if any(x.device.type == "meta" or y.device.type == "meta" for x, y in zip(a._buffers, b._buffers)):
                return True                     # an input placeholder of the shape-only recording
            return all(x.shape == y.shape and x.dtype == y.dtype and bool(torch.equal(x, y))
                       for x, y in zip(a._buffers, b._buffers))
        if isinstance(a, bool) or isinstance(a, (float, str)) or a is None:
            return type(a) is type(b) and (a == b or (isinstance(a, float) and a != a and b != b))
        if isinstance(a, (tuple, list)):
            return isinstance(b, (tuple, list)) and len(a) == len(b) and all(same(x, y) for x, y in zip(a, b))
        if isinstance(a, dict):
            return isinstance(b, dict) and a.keys() == b.keys() and all(same(a[k], b[k]) for k in a)
        return True                             # integers (handled affinely) and opaque objects

    for n0, n1 in zip(base.nodes, probe.nodes):
        if len(n0.arg_leaves) != len(n1.arg_leaves):
            return False
        if not all(same(a, b) for a, b in zip(n0.arg_leaves, n1.arg_leaves)) or not same(n0.kwargs, n1.kwargs):
            return False
    return True


def _integers_on_a_line(base: "_Recorded", p2: "_Recorded", p3: "_Recorded", name: str) -> bool:
    """Every integer argument (and output extent) of the three recordings moves linearly with the
    size called ``name``: v3 - v0 == (v2 - v0) * (s3 - s0) / (s2 - s0)."""
    s0, s2, s3 = base.sizes[name], p2.sizes[name], p3.sizes[name]

    def ok(a, b, c) -> bool:
        if isinstance(a, bool) or not isinstance(a, int):
            if isinstance(a, (tuple, list)):
                return isinstance(b, (tuple, list)) and isinstance(c, (tuple, list)) and len(a) == len(b) == len(c) \
                    and all(ok(x, y, z) for x, y, z in zip(a, b, c))
            if isinstance(a, dict):
                return isinstance(b, dict) and isinstance(c, dict) and a.keys() == b.keys() == c.keys() \
                    and all(ok(a[k], b[k], c[k]) for k in a)
            return True
        if not (isinstance(b, int) and isinstance(c, int)):
            return False
        return (c - a) * (s2 - s0) == (b - a) * (s3 - s0)

    for n0, n2, n3 in zip(base.nodes, p2.nodes, p3.nodes):
        if not (len(n0.arg_leaves) == len(n2.arg_leaves) == len(n3.arg_leaves)):
            return False
        if not all(ok(a, b, c) for a, b, c in zip(n0.arg_leaves, n2.arg_leaves, n3.arg_leaves)):
            return False
        if not ok(n0.kwargs, n2.kwargs, n3.kwargs):
            return False
        for o0, o2, o3 in zip(n0.outputs(), n2.outputs(), n3.outputs()):
            if o0 is not None and not ok(tuple(o0._shape), tuple(o2._shape) if o2 is not None else None,
                                         tuple(o3._shape) if o3 is not None else None):
                return False
    return True


class _NotAffine(Exception):
    """A recorded integer does not follow an affine function of the named sizes."""


class _Recorded:
    """One specialisation: placeholder impls, ordered nodes, fused steps, output recipe."""

    def __init__(self):
        self.targets: list[TensorImpl] = []
        self.keep_alive: list[TensorImpl] = []
        self.placeholders: list[TensorImpl] = []
        self.nodes: list[OpNode] = []
        self.keep: list[list[TensorImpl]] = []      # strong refs to every node's outputs
        self.steps: list = []
        self.free_after: list[list[TensorImpl]] = []
        self.out_impls: list[TensorImpl | None] = []
        self.out_static: list[Any] = []
        self.out_treedef = None
        self.cuda_graph = None
        self.arena_blocks: dict[int, tuple] = {}    # gathered tensors living in a symmetric arena
        self.arena_ok: set[int] = set()             # ids of impls that may live there (never returned)
        self.donated: list[bool] = []               # per placeholder
        self.out_cached: list | None = None         # Tensor objects of outputs that alias donated inputs
        self.static_inputs: list[list[torch.Tensor]] | None = None
        self.static_outputs: list[list[torch.Tensor]] | None = None
        self.side_steps: set[int] = set()           # optimizer updates that run on a side stream, under the backward
        self.host_sync = False                      # holds a node that reads a device value on the host
        self.sizes: dict[str, int] = {}             # value of every named dynamic dimension in this recording


def _first_tensor(tree: Any):
    """First Tensor found in a pytree (depth first), without flattening the whole tree."""
    if isinstance(tree, Tensor):
        return tree
    if isinstance(tree, dict):
        for v in tree.values():
            t = _first_tensor(v)
            if t is not None:
                return t
    elif isinstance(tree, (list, tuple)):
        for v in tree:
            t = _first_tensor(v)
            if t is not None:
                return t
    return None


def _normalize_step_scalars(tree: Any, depth: int = 0) -> Any:
    """Optimizer state dicts carry ``step`` as a python int that changes every call; turn it
    into a 0-d tensor so the cache key stays stable (reference: compile.py:138-170). Only the
    argument itself and its direct children are inspected: that is where optimizer states live,
    and walking a whole parameter tree on every call would cost more than the replay."""
    if isinstance(tree, dict):
        step = tree.get("step")
        if isinstance(step, (int, float)) and not isinstance(step, bool) and \
                ("m" in tree or "v" in tree or "momentum_buffers" in tree):
            from ..ops.creation import constant
            from ..types import DType

            first = _first_tensor(tree)
            out = dict(tree)
            out["step"] = constant(float(step), dtype=DType.float32, device=first.device if first is not None else None)
            return out
        if depth < 1:
            return {k: _normalize_step_scalars(v, depth + 1) for k, v in tree.items()}
        return tree
    if depth < 1 and isinstance(tree, (list, tuple)) and not hasattr(tree, "_fields"):
        return type(tree)(_normalize_step_scalars(v, depth + 1) for v in tree)
    return tree


class CompiledFunction:
    def __init__(self, fn: Callable, *, fullgraph: bool = False, max_cache_size: int = 64,
                 dynamic_dims: dict[int, dict[int, str]] | None = None, cuda_graph: bool = False,
                 donate_argnums: tuple[int, ...] | int = ()):
        self.fn = fn
        self.donate_argnums = (donate_argnums,) if isinstance(donate_argnums, int) else tuple(donate_argnums)
        self.fullgraph = fullgraph
        self.max_cache_size = int(max_cache_size)
        self.dynamic_dims = dynamic_dims or {}
        self.use_cuda_graph = bool(cuda_graph)
        self.profile_ops = False        # set True to time every step of the replay with CUDA events
        self.op_profile: dict[str, list] = {}
        self._cache: "OrderedDict[Any, dict[Any, _Recorded]]" = OrderedDict()
        self._stats = CompilationStats()
        self.__name__ = getattr(fn, "__name__", "compiled")
        self.__doc__ = getattr(fn, "__doc__", None)

    @property
    def stats(self) -> CompilationStats:
        return self._stats

    def clear_cache(self) -> None:
        self._cache.clear()

    def release(self) -> None:
        """Drop every recorded schedule together with its CUDA graphs and the buffers they own.
        Call it (then synchronise) before tearing down a process group whose collectives were
        captured, so that no graph outlives the communicator it launches into."""
        for entry in self._cache.values():
            for rec in entry.values():
                if not isinstance(rec, _Recorded):
                    continue
                rec.cuda_graph = None
                rec.static_inputs = rec.static_outputs = rec.out_cached = None
                for ph in rec.placeholders:
                    ph._buffers = None
                for outs in rec.keep:
                    for o in outs:
                        o._buffers = None
        self._cache.clear()

    def dump_plan(self, file=None) -> str:
        """Text listing of every recorded schedule: one line per step with its kind (``op`` or
        the name of a fused step), the op names it covers and the output shapes."""
        lines = []
        for entry in self._cache.values():
            for rec in entry.values():
                if not isinstance(rec, _Recorded):
                    continue
                lines.append(f"plan: {len(rec.nodes)} nodes, {len(rec.steps)} steps, "
                             f"{sum(rec.donated)} donated inputs, cuda_graph={rec.cuda_graph is not None}")
                for si, (kind, idxs) in enumerate(rec.steps):
                    names = "+".join(rec.nodes[i].op.name for i in idxs)
                    outs = [tuple(o._shape) for o in rec.keep[idxs[-1]]] if idxs[-1] < len(rec.keep) else []
                    lines.append(f"  {si:5d} {kind:20s} {names:40s} -> {outs}")
        text = "\n".join(lines)
        if file is not None:
            print(text, file=file)
        return text

    # ---- keys
    def _extract_sharding_key(self, sharding) -> Any:
        """Hashable identity of a sharding for the cache key: mesh, per-dimension axes, and the
        explicitly replicated and partial-sum axes, so a replicated input and one with a pending
        reduction never share a plan (reference: nabla/transforms/compile.py:270-274)."""
        return None if sharding is None else sharding.effect_signature()

    def _signature(self, t: Tensor, arg_idx: int | None) -> tuple[tuple, tuple]:
        im = t._impl
        shape = tuple(im._shape)
        dyn = self.dynamic_dims.get(arg_idx) if arg_idx is not None else None
        sp = im.sharding
        if sp is None:
            sh = None
        else:
            # the signature of a spec object never changes; the memo keeps the object alive so its id stays its own
            hit = _SPEC_SIG.get(id(sp))
            if hit is None or hit[0] is not sp:
                hit = (sp, sp.effect_signature())
                _SPEC_SIG[id(sp)] = hit
            sh = hit[1]
        rest = (im.dtype, sh, im.batch_dims, im.device)
        conc = (shape,) + rest
        if not dyn:
            return conc, conc
        sym = tuple(f"${dyn[i - im.batch_dims]}" if (i - im.batch_dims) in dyn else d for i, d in enumerate(shape))
        return (sym,) + rest, conc

    def _keys(self, args, kwargs):
        # one flatten per top-level argument: gives the leaves, the structure and each leaf's owner
        leaves: list = []
        owner: list[int | None] = []
        tds = []
        for i, a in enumerate(args):
            lv, td_a = pytree.tree_flatten(a)
            tds.append(td_a)
            leaves += lv
            owner += [i] * len(lv)
        lv, td_k = pytree.tree_flatten(kwargs)
        leaves += lv
        owner += [None] * len(lv)
        td = (tuple(tds), td_k)
        sym, conc = [], []
        for leaf, ow in zip(leaves, owner):
            if isinstance(leaf, Tensor):
                s, c = self._signature(leaf, ow)
                sym.append(s)
                conc.append(c)
            else:
                from ..core.graph.engine import _freeze

                f = ("static", _freeze(leaf))
                sym.append(f)
                conc.append(f)
        self._last_owner = owner
        # a plan (and above all a captured CUDA graph) freezes the kernel variants that were chosen
        # while it was recorded, so deterministic-replay mode gets entries of its own
        return (td, tuple(sym), config.is_deterministic()), tuple(conc), leaves, td

    # ---- call
    def __call__(self, *args, **kwargs):
        args = tuple(_normalize_step_scalars(a) for a in args)
        kwargs = {k: _normalize_step_scalars(v) for k, v in kwargs.items()}
        key, conc, leaves, td = self._keys(args, kwargs)
        pending = [t for t in leaves if isinstance(t, Tensor) and not t._impl.is_realized]
        if pending:
            GRAPH.evaluate(*pending)
        entry = self._cache.get(key)
        if entry is None:
            self._stats.misses += 1
            entry = {}
            self._cache[key] = entry
            while len(self._cache) > self.max_cache_size:
                self._cache.popitem(last=False)
            self._stats.cache_size = len(self._cache)
        else:
            self._cache.move_to_end(key)
            self._stats.hits += 1
        rec = entry.get(conc)
        if rec is None:
            t0 = time.perf_counter()
            sym = entry.get("__symbolic__")
            if sym is not None and sym is not False:
                # a new size of a dynamic_dims entry: instantiate the recorded node list, no Python re-run
                try:
                    rec, result = self._respecialise(sym, leaves)
                    self._stats.respecialisations += 1
                    entry[conc] = rec
                    self._stats.compile_time_s += time.perf_counter() - t0
                    return result
                except _NotAffine:
                    entry["__symbolic__"] = False
            if any(isinstance(r, _Recorded) for r in entry.values()):
                self._stats.retraces += 1
            try:
                rec, result = self._trace(leaves, td)
            except Exception:
                self._stats.fallbacks += 1
                raise
            entry[conc] = rec
            if self.dynamic_dims and sym is None:
                entry["__symbolic__"] = self._probe(rec, leaves, td)
            self._stats.compile_time_s += time.perf_counter() - t0
            return result
        t0 = time.perf_counter()
        out = self._replay(rec, [l for l in leaves if isinstance(l, Tensor)])
        self._stats.replay_time_s += time.perf_counter() - t0
        return out

    # ---- trace
    def _dyn_names(self, li: int, im: TensorImpl) -> dict[int, str]:
        """{physical dim index: name} of the named dynamic dimensions of leaf ``li``."""
        owner = getattr(self, "_last_owner", [])
        ow = owner[li] if li < len(owner) else None
        dyn = self.dynamic_dims.get(ow) if ow is not None else None
        return {d + im.batch_dims: n for d, n in dyn.items()} if dyn else {}

    def _record(self, leaves: list, td, scale: dict[str, int] | None = None) -> _Recorded:
        """Run the Python function once on placeholders and keep the node list. With ``scale``
        ({name: factor}) the placeholders are shape-only (meta buffers) and the named dimensions are
        multiplied: nothing can execute, the recording only serves to see which integers move."""
        rec = _Recorded()
        ph_leaves = []
        owner = getattr(self, "_last_owner", [None] * len(leaves))
        for li, l in enumerate(leaves):
            if isinstance(l, Tensor):
                im = l._impl
                shape = list(im._shape)
                names = self._dyn_names(li, im)
                for d, name in names.items():
                    rec.sizes[name] = int(shape[d]) * (scale.get(name, 1) if scale else 1)
                    shape[d] = rec.sizes[name]
                if scale is None:
                    bufs = list(im._buffers)
                else:
                    from ..core.sharding.spec import compute_local_shape

                    ids = im.sharding.mesh.local_ids if im.sharding is not None else [0]
                    bufs = [torch.empty(compute_local_shape(shape, im.sharding, i) if im.sharding is not None else shape,
                                        dtype=im.dtype.to_torch(), device="meta") for i in ids]
                ph = TensorImpl(bufs, shape=tuple(shape), dtype=im.dtype, device=im.device,
                                sharding=im.sharding, batch_dims=im.batch_dims, is_traced=False)
                ph.requires_grad = im.requires_grad
                ph.is_traced = im.requires_grad
                rec.placeholders.append(ph)
                rec.donated.append(owner[li] in self.donate_argnums if owner[li] is not None else False)
                ph_leaves.append(Tensor(impl=ph))
            else:
                ph_leaves.append(l)
        tds, td_k = td
        p_args, pos = [], 0
        for t_ in tds:
            p_args.append(pytree.tree_unflatten(t_, ph_leaves[pos: pos + t_.num_leaves]))
            pos += t_.num_leaves
        p_kwargs = pytree.tree_unflatten(td_k, ph_leaves[pos:])
        with config.tracing(True), config.eager_max_graph(False), config.capturable_trace(self.use_cuda_graph):
            result = self.fn(*p_args, **p_kwargs)
        out_leaves, out_td = pytree.tree_flatten(result)
        rec.out_treedef = out_td
        targets = []
        for o in out_leaves:
            if isinstance(o, Tensor):
                rec.out_impls.append(o._impl)
                rec.out_static.append(None)
                if not o._impl.is_realized:
                    targets.append(o._impl)
            else:
                rec.out_impls.append(None)
                rec.out_static.append(o)
        rec.nodes = topo_nodes(targets, lambda impl: impl.is_realized)
        rec.keep = [[o for o in n.outputs() if o is not None] for n in rec.nodes]
        rec.targets = targets
        return rec

    def _plan(self, rec: _Recorded) -> None:
        """Fused schedule, liveness and in-place marking of a recorded node list."""
        nodes, targets = rec.nodes, rec.targets
        rec.host_sync = any(getattr(n.op, "host_sync", False) for n in nodes)
        plan = fusion.build_plan(nodes, targets) if fusion.enabled() else None
        rec.steps = plan.steps if plan is not None else [("op", (i,)) for i in range(len(nodes))]
        if any(rec.donated):
            rec.steps = _optimizer_steps_last(rec.steps, nodes)
            rec.steps = _bucket_small_all_reduces(rec.steps, nodes)
        # liveness: free an intermediate after the last step that reads it
        out_ids = {id(i) for i in rec.out_impls if i is not None}
        produced = {id(o): o for outs in rec.keep for o in outs}
        last_use: dict[int, int] = {}
        ph_ids = {id(p) for p in rec.placeholders}
        ph_last_use: dict[int, int] = {}
        for si, (kind, idxs) in enumerate(rec.steps):
            for ni in idxs:
                for a in nodes[ni].input_impls():
                    if id(a) in produced:
                        last_use[id(a)] = si
                    elif id(a) in ph_ids:
                        ph_last_use[id(a)] = si
                for o in rec.keep[ni]:
                    last_use.setdefault(id(o), si)
        if any(rec.donated):
            _mark_inplace_updates(rec, ph_last_use)
            _fuse_dp_grad_updates(rec)
            if _os.environ.get("NABLA_B200_EARLY_OPTIMIZER", "1") != "0":
                last_use = _hoist_optimizer_steps(rec, last_use, produced)
        rec.free_after = [[] for _ in rec.steps]
        side_inputs = {id(a) for si in rec.side_steps for ni in rec.steps[si][1] for a in nodes[ni].input_impls()}
        for k, si in last_use.items():
            if k not in out_ids:
                # what a side-stream step reads stays allocated until the streams join (end of the schedule)
                rec.free_after[len(rec.steps) - 1 if k in side_inputs else si].append(produced[k])
        self._stats.graph_nodes = len(nodes)
        self._stats.graph_steps = len(rec.steps)

    def _trace(self, leaves: list, td) -> tuple[_Recorded, Any]:
        rec = self._record(leaves, td)
        self._plan(rec)
        self._run(rec)
        return rec, self._collect(rec)

    # ---- dynamic dimensions
    def _probe(self, rec: _Recorded, leaves: list, td):
        """Second, shape-only recording with every named dimension doubled (one recording per name).
        Returns the symbolic description used by ``_respecialise`` or False when the function cannot
        be described that way (it needs data while tracing, or its structure depends on the size)."""
        names = sorted(rec.sizes)
        if not names:
            return False
        probes = {}
        try:
            for name in names:
                other = self._record(leaves, td, scale={name: 2})
                if len(other.nodes) != len(rec.nodes) or any(a.op is not b.op for a, b in zip(other.nodes, rec.nodes)):
                    return False
                if not _static_values_agree(rec, other):
                    return False
                # two recordings always lie on a line; a third one says whether the integers really do
                third = self._record(leaves, td, scale={name: 3})
                if len(third.nodes) != len(rec.nodes) or any(a.op is not b.op for a, b in zip(third.nodes, rec.nodes)) \
                        or not _static_values_agree(rec, third) or not _integers_on_a_line(rec, other, third, name):
                    return False
                probes[name] = other
        except Exception:
            return False
        return {"base": rec, "probes": probes}

    def _respecialise(self, sym: dict, leaves: list) -> tuple["_Recorded", Any]:
        """Instantiate the base recording for the sizes of ``leaves``: same nodes, integers that moved
        between the base and the probe recordings re-evaluated, output shapes re-inferred."""
        base: _Recorded = sym["base"]
        tensors = [(li, l) for li, l in enumerate(leaves) if isinstance(l, Tensor)]
        sizes: dict[str, int] = {}
        for (li, l) in tensors:
            for d, name in self._dyn_names(li, l._impl).items():
                v = int(l._impl._shape[d])
                if sizes.setdefault(name, v) != v:
                    raise ValueError(f"dynamic dimension '{name}' has two different sizes in one call ({sizes[name]}, {v})")
        env = [(base.sizes[n], sym["probes"][n].sizes[n], sizes[n], sym["probes"][n]) for n in sorted(base.sizes)]

        def value(path_get, v0):
            """Integer at the same place in every recording -> its value for the new sizes."""
            out = Fraction(v0)
            for s0, s1, s_new, probe in env:
                v1 = path_get(probe)
                if type(v1) is not type(v0) and not (isinstance(v1, int) and isinstance(v0, int)):
                    raise _NotAffine()
                if v1 != v0:
                    out += Fraction(v1 - v0, s1 - s0) * (s_new - s0)
            if out.denominator != 1:
                raise _NotAffine()
            return int(out)

        def subst(x0, getter):
            """Rebuild a (nested) static argument, re-evaluating the integers that moved."""
            if isinstance(x0, bool) or x0 is None or isinstance(x0, (str, float)):
                return x0
            if isinstance(x0, int):
                return value(getter, x0)
            if isinstance(x0, (tuple, list)):
                for _, _, _, probe in env:
                    x1 = getter(probe)
                    if not isinstance(x1, (tuple, list)) or len(x1) != len(x0):
                        raise _NotAffine()
                return type(x0)(subst(v, (lambda i: lambda r: getter(r)[i])(i)) for i, v in enumerate(x0)) \
                    if not hasattr(x0, "_fields") else x0
            if isinstance(x0, dict):
                return {k: subst(v, (lambda k: lambda r: getter(r)[k])(k)) for k, v in x0.items()}
            return x0

        new = _Recorded()
        new.sizes = sizes
        new.donated = list(base.donated)
        new.out_static = list(base.out_static)
        new.out_treedef = base.out_treedef
        mapping: dict[int, TensorImpl] = {}
        for ph0, (li, l) in zip(base.placeholders, tensors):
            im = l._impl
            ph = TensorImpl(list(im._buffers), shape=im._shape, dtype=im.dtype, device=im.device, sharding=im.sharding,
                            batch_dims=im.batch_dims, is_traced=False)
            ph.requires_grad = ph0.requires_grad
            ph.is_traced = ph0.is_traced
            new.placeholders.append(ph)
            mapping[id(ph0)] = ph
        for ni, n0 in enumerate(base.nodes):
            leaves_new = []
            for ai, a in enumerate(n0.arg_leaves):
                if isinstance(a, TensorImpl):
                    leaves_new.append(mapping.get(id(a), a))         # constants captured by the trace stay as they are
                else:
                    leaves_new.append(subst(a, (lambda ni, ai: lambda r: r.nodes[ni].arg_leaves[ai])(ni, ai)))
            kw = subst(n0.kwargs, (lambda ni: lambda r: r.nodes[ni].kwargs)(ni))
            okw = kw if n0.op_kwargs is n0.kwargs else subst(n0.op_kwargs, (lambda ni: lambda r: r.nodes[ni].op_kwargs)(ni))
            node = OpNode(n0.op, leaves_new, n0.arg_treedef, kw, okw)
            node.out_treedef = n0.out_treedef
            outs0 = n0.outputs()
            ins = [a for a in leaves_new if isinstance(a, TensorImpl)]
            if getattr(n0.op, "host_sync", False):
                # control-flow nodes keep the structure of their state: shapes follow the matching inputs
                metas = None
            else:
                fake = [Tensor(impl=a) if isinstance(a, TensorImpl) else a for a in leaves_new]
                metas, _ = n0.op.infer_outputs([(a._shape, a.dtype.to_torch()) for a in ins], fake, n0.arg_treedef, kw)
            for oi, o0 in enumerate(outs0):
                if o0 is None:
                    node.out_refs.append(lambda: None)
                    continue
                if metas is not None:
                    shape = tuple(int(x) for x in metas[oi][0])
                else:
                    shape = subst(tuple(int(x) for x in o0._shape), (lambda ni, oi: lambda r: tuple(int(x) for x in r.nodes[ni].outputs()[oi]._shape))(ni, oi))
                impl = TensorImpl(None, shape=shape, dtype=o0.dtype, device=o0.device, sharding=o0.sharding,
                                  batch_dims=o0.batch_dims, is_traced=o0.is_traced)
                impl.output_refs = node
                impl.output_index = oi
                node.out_refs.append(weakref.ref(impl))
                mapping[id(o0)] = impl
                new.keep_alive.append(impl)
            new.nodes.append(node)
        new.keep = [[o for o in n.outputs() if o is not None] for n in new.nodes]
        new.out_impls = [mapping.get(id(i), i) if i is not None else None for i in base.out_impls]
        new.targets = [mapping[id(t)] for t in base.targets]
        self._plan(new)
        self._run(new)
        return new, self._collect(new)

    # ---- execution of a recorded graph
    def _run(self, rec: _Recorded) -> None:
        nodes = rec.nodes
        _STATS["nodes_executed"] += len(nodes)
        if self.profile_ops and not torch.cuda.is_current_stream_capturing():
            return self._run_profiled(rec)
        nvtx = _NVTX and torch.cuda.is_available()
        side = cur = None
        # Measured on the 24-layer benchmark step (1 GPU, power-capped at 1 kW): 155.8 ms with the updates
        # on the side stream, 155.2 ms without: the step is energy bound, so hiding the AdamW kernels
        # buys nothing there. The side stream is therefore opt-in; the early placement stays.
        if rec.side_steps and _os.environ.get("NABLA_B200_OPTIMIZER_STREAM", "0") == "1" \
                and not config.is_deterministic() and torch.cuda.is_available() \
                and rec.placeholders and rec.placeholders[0].device.label == "gpu":
            cur = torch.cuda.current_stream()
            side = _optimizer_stream(cur.device)
        for si, (kind, idxs) in enumerate(rec.steps):
            if nvtx:       # one range per plan step (NABLA_B200_NVTX=1), visible in timeline profilers
                torch.cuda.nvtx.range_push(kind if kind != "op" else nodes[idxs[0]].op.name)
            if kind == "op":
                n = nodes[idxs[0]]
                if side is not None and si in rec.side_steps:
                    # in-place parameter update whose inputs are final and whose parameter nobody reads
                    # any more in this step: it runs beside the rest of the backward pass
                    side.wait_stream(cur)
                    with torch.cuda.stream(side):
                        outs = n.op.execute(n)
                else:
                    outs = n.op.execute(n)
                for i, ref in enumerate(n.out_refs):
                    o = ref()
                    if o is not None:
                        o._buffers = outs[i]
            else:
                fusion.run_fused(kind, [nodes[i] for i in idxs], keep_graph=True, arena_blocks=rec.arena_blocks)
            if nvtx:
                torch.cuda.nvtx.range_pop()
            for dead in rec.free_after[si]:
                dead._buffers = None
                blk = rec.arena_blocks.pop(id(dead), None)
                if blk is not None:
                    blk[0].free(blk[1])
            if side is not None and si == len(rec.steps) - 2:
                cur.wait_stream(side)          # join before the last step's frees and before anything is returned
        if side is not None:
            cur.wait_stream(side)
        self._release_arena(rec)

    @staticmethod
    def _release_arena(rec: _Recorded) -> None:
        """Results that are handed to the caller must not stay in the symmetric arena."""
        for impl in rec.out_impls:
            blk = rec.arena_blocks.pop(id(impl), None) if impl is not None else None
            if blk is not None:
                impl._buffers = [b.clone() for b in impl._buffers]
                blk[0].free(blk[1])

    def _run_profiled(self, rec: _Recorded) -> None:
        """Same as ``_run`` with a CUDA event pair around every step; device time per step kind
        accumulates in ``self.op_profile`` ({name: [calls, ms]}), read it after a synchronize."""
        nodes = rec.nodes
        marks = []
        for si, (kind, idxs) in enumerate(rec.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if kind == "op":
                n = nodes[idxs[0]]
                outs = n.op.execute(n)
                for i, ref in enumerate(n.out_refs):
                    o = ref()
                    if o is not None:
                        o._buffers = outs[i]
                name = n.op.name
            else:
                fusion.run_fused(kind, [nodes[i] for i in idxs], keep_graph=True, arena_blocks=rec.arena_blocks)
                name = kind + ":" + nodes[idxs[-1]].op.name
            e1.record()
            marks.append((name, e0, e1))
            for dead in rec.free_after[si]:
                dead._buffers = None
                blk = rec.arena_blocks.pop(id(dead), None)
                if blk is not None:
                    blk[0].free(blk[1])
        torch.cuda.synchronize()
        for name, e0, e1 in marks:
            ent = self.op_profile.setdefault(name, [0, 0.0])
            ent[0] += 1
            ent[1] += e0.elapsed_time(e1)

    def _collect(self, rec: _Recorded) -> Any:
        outs = []
        for impl, static in zip(rec.out_impls, rec.out_static):
            if impl is None:
                outs.append(static)
                continue
            new = TensorImpl(list(impl._buffers), shape=impl._shape, dtype=impl.dtype, device=impl.device,
                             sharding=impl.sharding, batch_dims=impl.batch_dims)
            outs.append(Tensor(impl=new))
        # drop our references to output buffers produced by nodes (placeholders are re-bound per call)
        ph = {id(p) for p in rec.placeholders}
        for impl in rec.out_impls:
            if impl is not None and id(impl) not in ph and impl.output_refs is not None:
                impl._buffers = None
        return pytree.tree_unflatten(rec.out_treedef, outs)

    def _replay(self, rec: _Recorded, tensors: list[Tensor]) -> Any:
        if self.use_cuda_graph and not rec.host_sync and tensors and tensors[0]._impl.device.label == "gpu":
            return self._replay_cuda_graph(rec, tensors)
        for ph, t in zip(rec.placeholders, tensors):
            ph._buffers = t._impl._buffers
        try:
            self._run(rec)
            return self._collect(rec)
        finally:
            for ph in rec.placeholders:
                ph._buffers = None

    def _replay_cuda_graph(self, rec: _Recorded, tensors: list[Tensor]) -> Any:
        if rec.cuda_graph is None:
            # the graph owns its inputs: replays read (and, for donated arguments, update) them
            rec.static_inputs = [[b.clone() for b in t._impl._buffers] for t in tensors]
            for ph, bufs in zip(rec.placeholders, rec.static_inputs):
                ph._buffers = bufs
            torch.cuda.synchronize()
            torch.cuda.empty_cache()      # the graph gets its own pool; hand cached blocks back first
            g = torch.cuda.CUDAGraph()
            try:
                from ..native import total_launches

                n0 = total_launches()
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    self._run(rec)
                    rec.static_outputs = [list(i._buffers) if i is not None else None for i in rec.out_impls]
            except Exception as e:
                import warnings

                warnings.warn(f"CUDA graph capture failed ({type(e).__name__}: {e}); replaying without a graph")
                self._stats.fallbacks += 1
                self.use_cuda_graph = False
                for ph in rec.placeholders:
                    ph._buffers = None
                return self._replay(rec, tensors)
            rec.cuda_graph = g
            self._stats.cuda_graphs += 1
            self._stats.launches_per_graph = total_launches() - n0
            # only the graph's copies of DONATED arguments may be handed back as results: the caller gave
            # those buffers up. The static copy of any other argument is overwritten by the next
            # call's copy-in, so a result that aliases it is cloned out below.
            rec.static_ptrs = {b.data_ptr() for bufs, d in zip(rec.static_inputs, rec.donated) if d for b in bufs}
        for bufs, t in zip(rec.static_inputs, tensors):
            for dst, src in zip(bufs, t._impl._buffers):
                if dst.data_ptr() != src.data_ptr():
                    dst.copy_(src)
        rec.cuda_graph.replay()
        if rec.out_cached is None:
            # results that live entirely in a donated input's buffers are the same storage on
            # every replay: their Tensor objects are built once and handed back as they are
            rec.out_cached = []
            for impl, bufs in zip(rec.out_impls, rec.static_outputs):
                if impl is not None and all(b.data_ptr() in rec.static_ptrs for b in bufs):
                    rec.out_cached.append(Tensor(impl=TensorImpl(list(bufs), shape=impl._shape, dtype=impl.dtype,
                                                                device=impl.device, sharding=impl.sharding,
                                                                batch_dims=impl.batch_dims)))
                else:
                    rec.out_cached.append(None)
        outs = []
        for impl, static, bufs, cached in zip(rec.out_impls, rec.out_static, rec.static_outputs, rec.out_cached):
            if impl is None:
                outs.append(static)
            elif cached is not None:
                outs.append(cached)
            else:
                res = [b if b.data_ptr() in rec.static_ptrs else b.clone() for b in bufs]
                new = TensorImpl(res, shape=impl._shape, dtype=impl.dtype, device=impl.device,
                                 sharding=impl.sharding, batch_dims=impl.batch_dims)
                outs.append(Tensor(impl=new))
        return pytree.tree_unflatten(rec.out_treedef, outs)


_OPT_STREAMS: dict = {}


def _optimizer_stream(device) -> "torch.cuda.Stream":
    st = _OPT_STREAMS.get(device)
    if st is None:
        st = torch.cuda.Stream(device=device)
        _OPT_STREAMS[device] = st
    return st


def _hoist_optimizer_steps(rec: "_Recorded", last_use: dict[int, int], produced: dict[int, TensorImpl]) -> dict[int, int]:
    """Move every in-place optimizer update from the tail of the schedule to right behind the step
    that makes it runnable: its gradient (and every other input) exists and no later step reads the
    parameter / moments it overwrites. Each parameter is then updated as soon as its gradient is
    final (reference: the update follows the partial-sum all-reduce of the gradient,
    nabla/core/autograd/backward.py:72-80 + nn/optim/functional.py:116-162), and because such an
    update touches nothing the rest of the backward pass uses, ``_run`` can issue it on a side stream
    (``NABLA_B200_OPTIMIZER_STREAM=1``) so that the bandwidth-bound AdamW kernels run under the
    tensor-core work of the earlier layers; its gradient is freed right after it either way.

    Only plain local updates move (kind 'op', already marked in place); updates fused with a
    collective stay in the tail, in program order on the main stream, because their device-side
    barriers share the group's workspace with the fused GEMM kernels. Returns ``last_use`` re-keyed
    to the new step indices; ``rec.steps`` and ``rec.side_steps`` are updated."""
    nodes, steps = rec.nodes, rec.steps
    movable = [si for si, (kind, idxs) in enumerate(steps)
               if kind == "op" and getattr(nodes[idxs[0]].op, "inplace_inputs", None) and nodes[idxs[0]].kwargs.get("inplace")]
    if not movable:
        return last_use
    mov = set(movable)
    producer: dict[int, int] = {}
    for si, (kind, idxs) in enumerate(steps):
        for ni in idxs:
            for o in rec.keep[ni]:
                producer[id(o)] = si
    readers: dict[int, int] = {}            # impl id -> last NON-movable step that reads it
    for si, (kind, idxs) in enumerate(steps):
        if si in mov:
            continue
        for ni in idxs:
            for a in nodes[ni].input_impls():
                readers[id(a)] = si
    after: dict[int, list[int]] = {}
    for si in movable:
        n = nodes[steps[si][1][0]]
        ready = -1
        for a in n.input_impls():
            ready = max(ready, producer.get(id(a), -1), readers.get(id(a), -1))
        ready = min(ready, si)              # never later than where it already was
        after.setdefault(ready, []).append(si)
    order: list[int] = list(after.get(-1, []))
    for si in range(len(steps)):
        if si in mov:
            continue
        order.append(si)
        order += after.get(si, [])
    new_index = {old: new for new, old in enumerate(order)}
    rec.steps = [steps[o] for o in order]
    # an update that ends up last has nothing to run beside
    rec.side_steps = {new_index[si] for si in movable if new_index[si] < len(order) - 1}
    return _recompute_last_use(rec)


def _recompute_last_use(rec: "_Recorded") -> dict[int, int]:
    produced = {id(o) for outs in rec.keep for o in outs}
    last: dict[int, int] = {}
    for si, (kind, idxs) in enumerate(rec.steps):
        for ni in idxs:
            for a in rec.nodes[ni].input_impls():
                if id(a) in produced:
                    last[id(a)] = si
            for o in rec.keep[ni]:
                last.setdefault(id(o), si)
    return last


def _optimizer_steps_last(steps: list, nodes: list[OpNode]) -> list:
    """Move in-place-capable update ops whose results feed no other node to the end of the
    schedule, so that they are the last readers of the parameters they overwrite."""
    consumed = set()
    for n in nodes:
        for a in n.input_impls():
            consumed.add(id(a))
    head, tail = [], []
    for st in steps:
        kind, idxs = st
        n = nodes[idxs[0]]
        if kind == "op" and getattr(n.op, "inplace_inputs", None) and \
                not any(o is not None and id(o) in consumed for o in n.outputs()):
            tail.append(st)
        else:
            head.append(st)
    return head + tail


def _bucket_small_all_reduces(steps: list, nodes: list[OpNode], max_elems: int = 1 << 20) -> list:
    """Gradients of small parameters (biases, LayerNorm gains) each need their own all-reduce
    before the optimizer: hundreds of launches that move a few KB. Those whose only reader is an
    optimizer step at the end of the schedule are taken out of line and reduced together, one
    flat buffer per (axes, dtype), right before the optimizer steps."""
    readers: dict[int, list[int]] = {}
    for ni, n in enumerate(nodes):
        for a in n.input_impls():
            readers.setdefault(id(a), []).append(ni)
    tail_nodes = set()
    tail_start = len(steps)
    for si in range(len(steps) - 1, -1, -1):
        kind, idxs = steps[si]
        if kind == "op" and getattr(nodes[idxs[0]].op, "inplace_inputs", None):
            tail_nodes.add(idxs[0])
            tail_start = si
        else:
            break
    if not tail_nodes:
        return steps
    groups: dict[tuple, list[int]] = {}
    for si, (kind, idxs) in enumerate(steps[:tail_start]):
        if kind != "op":
            continue
        n = nodes[idxs[0]]
        if n.op.name != "all_reduce" or n.kwargs.get("reduce_op", "sum") != "sum":
            continue
        x = n.input_impls()[0]
        o = n.outputs()[0]
        sp = x.sharding
        if o is None or sp is None or not sp.mesh.is_distributed or x.batch_dims:
            continue
        axes = set(n.kwargs.get("reduce_axes", ()))
        if not axes or not axes <= set(sp.partial_sum_axes) or any(set(d.axes) & axes for d in sp.dim_specs):
            continue
        rd = readers.get(id(o), [])
        if len(rd) != 1 or rd[0] not in tail_nodes:
            continue
        numel = 1
        for d in compute_local(x):
            numel *= int(d)
        if numel > max_elems:
            continue
        groups.setdefault((tuple(sorted(axes)), x.dtype, id(sp.mesh)), []).append(si)
    taken = {si for g in groups.values() if len(g) >= 2 for si in g}
    if not taken:
        return steps
    head = [st for si, st in enumerate(steps[:tail_start]) if si not in taken]
    buckets = [("all_reduce_bucket", tuple(steps[si][1][0] for si in g)) for g in groups.values() if len(g) >= 2]
    return head + buckets + steps[tail_start:]


def _fuse_dp_grad_updates(rec: _Recorded) -> None:
    """``matmul -> all_reduce(sum over replica axes) -> in-place AdamW`` on bf16 parameters: the
    all-reduce moves into the optimizer kernel (see fusion.run_fused 'gemm_to_arena' / 'adamw_reduce')."""
    from ..types import DType

    nodes = rec.nodes
    readers: dict[int, list[int]] = {}
    for ni, n in enumerate(nodes):
        for a in n.input_impls():
            readers.setdefault(id(a), []).append(ni)
    adam_step = {idxs[0]: si for si, (kind, idxs) in enumerate(rec.steps)
                 if kind == "op" and nodes[idxs[0]].op.name == "adam_wstep" and nodes[idxs[0]].kwargs.get("inplace")}
    out_ids = {id(i) for i in rec.out_impls if i is not None}
    for si, (kind, idxs) in enumerate(rec.steps):
        if kind != "gemm_all_reduce":
            continue
        ar = nodes[idxs[1]]
        g = ar.outputs()[0]
        if g is None or id(g) in out_ids or len(readers.get(id(g), [])) != 1:
            continue
        k = readers[id(g)][0]
        if k not in adam_step:
            continue
        ad = nodes[k]
        ins = ad.input_impls()
        if len(ins) < 4 or ins[1] is not g:
            continue
        p_, m_, v_ = ins[0], ins[2], ins[3]
        n_el = 1
        for d in (p_.sharding and compute_local(p_) or p_._shape):
            n_el *= int(d)
        if not (p_.dtype is DType.bfloat16 and g.dtype is DType.bfloat16 and m_.dtype is DType.float32
                and v_.dtype is DType.float32 and n_el % 8 == 0 and len(g._shape) == 2):
            continue
        mesh = g.sharding.mesh if g.sharding is not None else None
        if mesh is None:
            continue
        rec.arena_blocks[("dp_group", id(ad))] = (mesh, [x for x in mesh.axis_names if x in ar.kwargs["reduce_axes"]])
        rec.steps[si] = ("gemm_to_arena", idxs)
        rec.steps[adam_step[k]] = ("adamw_reduce", (k,))


def compute_local(impl) -> tuple:
    from ..core.sharding.spec import compute_local_shape

    mesh = impl.sharding.mesh
    return compute_local_shape(impl._shape, impl.sharding, mesh.local_ids[0])


def _mark_inplace_updates(rec: _Recorded, last_use: dict[int, int]) -> None:
    donated = {id(ph) for ph, d in zip(rec.placeholders, rec.donated) if d}
    for si, (kind, idxs) in enumerate(rec.steps):
        if kind != "op":
            continue
        n = rec.nodes[idxs[0]]
        which = getattr(n.op, "inplace_inputs", None)
        if not which:
            continue
        ins = n.input_impls()
        targets = [ins[i] for i in which if i < len(ins)]
        # in place only when every overwritten input was donated and nothing reads it later
        if targets and all(id(t) in donated and last_use.get(id(t), si) <= si for t in targets):
            n.kwargs = dict(n.kwargs, inplace=True)


def compile(fn: Callable | None = None, *, fullgraph: bool = False, max_cache_size: int = 64,
            dynamic_dims: dict[int, dict[int, str]] | None = None, cuda_graph: bool = False,
            donate_argnums: tuple[int, ...] | int = ()):
    """Decorator / wrapper: ``@compile`` or ``compile(fn, dynamic_dims={0: {0: "batch"}})``."""
    if fn is None:
        return lambda f: CompiledFunction(f, fullgraph=fullgraph, max_cache_size=max_cache_size,
                                          dynamic_dims=dynamic_dims, cuda_graph=cuda_graph, donate_argnums=donate_argnums)
    return CompiledFunction(fn, fullgraph=fullgraph, max_cache_size=max_cache_size, dynamic_dims=dynamic_dims,
                            cuda_graph=cuda_graph, donate_argnums=donate_argnums)
