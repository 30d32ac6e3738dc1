"""Control flow (reference: nabla/ops/control_flow.py:21-507): ``where`` (differentiable),
``cond`` and ``while_loop`` (data-dependent; the reference gives them no derivative, here reverse mode
works through them both eagerly and when recorded by ``compile``), ``scan`` (Python-unrolled,
differentiable through its body).

Outside ``compile`` the predicate of ``cond`` / ``while_loop`` is read on the host and the chosen
code runs right away. While ``compile`` traces, both become ONE recorded node (``CondOp`` /
``WhileOp``) that keeps the branch / body functions: every replay reads the predicate of that
call's data and runs the matching branch (or as many iterations as that call's data asks for), so
a compiled function stays data dependent (reference: ops.cond / ops.while_loop lowered into the
graph, control_flow.py:302-307, 444-446). These nodes read a device value on the host, so a step
that contains one is replayed without CUDA-graph capture; under ``compile(cuda_graph=True)``
``cond`` instead evaluates both branches and selects with ``where``, which stays on the device."""
from __future__ import annotations

import weakref
from typing import Any, Callable

import torch

from .. import config
from ..core.common import pytree
from ..core.graph.tracing import OpNode
from ..core.tensor.api import Tensor, realize_all
from ..core.tensor.impl import TensorImpl
from .base import Operation, _align_batch_dims, ensure_tensor


class WhereOp(Operation):
    def kernel(self, c, a, b):
        return torch.where(c.bool(), a, b)

    def partial_passthrough_axes(self, input_specs, kwargs=None):
        # linear in (a, b) jointly: carry an axis only if both branches carry it
        if len(input_specs) < 3:
            return set()
        return set(input_specs[1].partial_sum_axes) & set(input_specs[2].partial_sum_axes) - set(input_specs[0].partial_sum_axes)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        from .creation import zeros_like

        c, a, b = primals
        z = zeros_like(cot)
        return (None, where(c, cot, z), where(c, z, cot))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        from .creation import zeros_like

        c, a, b = primals
        ta = tangents[1] if tangents[1] is not None else zeros_like(a)
        tb = tangents[2] if tangents[2] is not None else zeros_like(b)
        return where(c, ta, tb)


_where = WhereOp()


def where(condition, x, y) -> Tensor:
    """Elementwise select with three-way numpy broadcasting."""
    if not isinstance(x, Tensor) and not isinstance(y, Tensor):
        x = ensure_tensor(x)
    x = ensure_tensor(x, y if isinstance(y, Tensor) else None)
    y = ensure_tensor(y, x)
    condition = ensure_tensor(condition, None)
    if x.dtype is not y.dtype:
        from .unary import cast

        if x.dtype.is_float() and not y.dtype.is_float():
            y = cast(y, x.dtype)
        elif y.dtype.is_float() and not x.dtype.is_float():
            x = cast(x, y.dtype)
    if condition._impl.batch_dims or x._impl.batch_dims or y._impl.batch_dims:
        condition, x, y = _align_batch_dims([condition, x, y])
    return _where(condition, x, y)


def _closure_tensors(*fns: Callable) -> list[Tensor]:
    """Tensors a function closes over (one level, through containers): they become inputs of the
    recorded node so that the replay realises them first and keeps them alive until it has run."""
    found: list[Tensor] = []
    seen: set[int] = set()
    for fn in fns:
        cells = getattr(fn, "__closure__", None) or ()
        for c in cells:
            try:
                v = c.cell_contents
            except ValueError:
                continue
            for leaf in pytree.tree_leaves(v) if isinstance(v, (Tensor, dict, list, tuple)) else ():
                if isinstance(leaf, Tensor) and id(leaf._impl) not in seen:
                    seen.add(id(leaf._impl))
                    found.append(leaf)
    return found


def _fresh(impl: TensorImpl) -> Tensor:
    """A new realized Tensor over the buffers an impl holds right now."""
    return Tensor(impl=TensorImpl(list(impl._buffers), shape=impl._shape, dtype=impl.dtype, device=impl.device,
                                  sharding=impl.sharding, batch_dims=impl.batch_dims))


def _host_bool(x) -> bool:
    if isinstance(x, Tensor):
        return bool(x.item())
    if isinstance(x, TensorImpl):
        return bool(x._buffers[0].reshape(-1)[0].item())
    return bool(x)


class _HostControlOp(Operation):
    """Base of the recorded control-flow nodes. ``host_sync`` tells ``compile`` that the node reads
    a device value on the host (no CUDA-graph capture of a schedule that contains it)."""

    host_sync = True
    partial_policy = "none"

    def build(self, inputs: list[Tensor], templates: list[Tensor], kwargs: dict) -> list[Tensor]:
        _, td = pytree.tree_flatten(tuple(inputs))
        node = OpNode(self, [t._impl for t in inputs], td, kwargs, kwargs)
        outs = []
        for i, t in enumerate(templates):
            im = t._impl
            impl = TensorImpl(None, shape=im._shape, dtype=im.dtype, device=im.device, sharding=im.sharding,
                              batch_dims=im.batch_dims, is_traced=any(t._impl.is_traced for t in inputs))
            impl.output_refs = node
            impl.output_index = i
            node.out_refs.append(weakref.ref(impl))
            outs.append(Tensor(impl=impl))
        _, node.out_treedef = pytree.tree_flatten(list(outs))
        return outs

    def run(self, kw: dict, inputs: list[Tensor]) -> Any:
        """The Python side of the node on concrete tensors (one per node input): what ``execute``
        evaluates, and what the backward node differentiates."""
        raise NotImplementedError

    def closure_objects(self, kw: dict) -> list[Tensor]:
        """The tensors the kept functions close over, in the order they were appended to the inputs."""
        return []

    def first_closure_input(self, kw: dict) -> int:
        raise NotImplementedError

    def vjp_rule(self, primals, cot, outputs, kwargs):
        """Reverse mode through a recorded ``cond`` / ``while_loop``: one more host node. At replay it
        runs the taken branch (or the loop) again on that call's data with autograd recording on,
        pulls the cotangents back through what actually ran, and hands out the gradients of the
        operands and of the tensors the functions close over."""
        prim = list(primals)
        cots = list(cot) if isinstance(cot, (list, tuple)) else [cot]
        given = [(k, c) for k, c in enumerate(cots) if isinstance(c, Tensor)]     # outputs nobody used have none
        diff = [i for i, p in enumerate(prim) if isinstance(p, Tensor) and p.dtype.is_float()
                and not (type(self) is CondOp and i == 0)]
        if not diff or not given:
            return tuple(None for _ in prim)
        kw = {"fwd": self, "fwd_kwargs": kwargs, "n_fwd": len(prim), "diff": tuple(diff),
              "cot_positions": tuple(k for k, _ in given)}
        grads = iter(_host_vjp_op.build([*prim, *[c for _, c in given]], [prim[i] for i in diff], kw))
        return tuple(next(grads) if i in diff else None for i in range(len(prim)))

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        raise NotImplementedError(f"forward mode through a '{self.name}' recorded by compile is not available: "
                                  "use reverse mode (grad / vjp / jacrev), or differentiate outside compile")

    @staticmethod
    def _result_buffers(tree: Any, n_expected: int, what: str) -> list[list[torch.Tensor]]:
        leaves = [l for l in pytree.tree_leaves(tree) if isinstance(l, Tensor)]
        if len(leaves) != n_expected:
            raise ValueError(f"{what}: produced {len(leaves)} tensors, the recorded structure has {n_expected}")
        realize_all(*leaves)
        return [list(l._impl._buffers) for l in leaves]


class CondOp(_HostControlOp):
    """inputs: [pred, *operand tensors, *closed-over tensors]; kwargs keep the two functions and the
    operand tree. Replays read ``pred`` and run the matching branch eagerly."""

    def run(self, kw, inputs):
        it = iter(inputs[1:1 + kw["n_operands"]])
        leaves = [next(it) if is_t else v for is_t, v in kw["operand_leaves"]]
        operands = pytree.tree_unflatten(kw["operand_treedef"], leaves)
        return (kw["true_fn"] if _host_bool(inputs[0]) else kw["false_fn"])(*operands)

    def closure_objects(self, kw):
        return _closure_tensors(kw["true_fn"], kw["false_fn"])

    def first_closure_input(self, kw):
        return 1 + kw["n_operands"]

    def execute(self, node):
        with config.tracing(False):
            out = self.run(node.kwargs, [_fresh(i) for i in node.input_impls()])
            return self._result_buffers(out, len(node.out_refs), "cond branch")


class WhileOp(_HostControlOp):
    """inputs: [*loop-state tensors, *closed-over tensors]. Replays run ``cond_fn`` / ``body_fn``
    eagerly until the condition computed from that call's data turns false."""

    def run(self, kw, inputs, keep_graph: bool = False):
        it = iter(inputs[:kw["n_state"]])
        state = tuple(pytree.tree_unflatten(kw["state_treedef"], [next(it) if is_t else v for is_t, v in kw["state_leaves"]]))
        return _while_eager(kw["cond_fn"], kw["body_fn"], state, kw.get("max_iters"), realize=not keep_graph)

    def closure_objects(self, kw):
        return _closure_tensors(kw["cond_fn"], kw["body_fn"])

    def first_closure_input(self, kw):
        return kw["n_state"]

    def execute(self, node):
        with config.tracing(False):
            state = self.run(node.kwargs, [_fresh(i) for i in node.input_impls()])
            return self._result_buffers(state, len(node.out_refs), "while_loop body")


class HostVjpOp(_HostControlOp):
    """Backward of a recorded ``cond`` / ``while_loop``. inputs: [*inputs of the forward node,
    *cotangents of its outputs]; outputs: one gradient per differentiable forward input."""

    _name = "host_control_vjp"

    def execute(self, node):
        from ..core.autograd.backward import backward_on_trace
        from ..core.graph.tracing import Trace
        from .creation import zeros_like

        kw = node.kwargs
        fwd, fkw, n = kw["fwd"], kw["fwd_kwargs"], kw["n_fwd"]
        ins = node.input_impls()
        inputs = [_fresh(i) for i in ins[:n]]
        given = dict(zip(kw["cot_positions"], (_fresh(i) for i in ins[n:])))
        # the kept functions read the tensors they close over from the objects they captured, not
        # from the node inputs: those objects stand in at their positions
        first = fwd.first_closure_input(fkw)
        captured = {id(t._impl): t for t in fwd.closure_objects(fkw)}
        for j in range(first, n):
            obj = captured.get(id(ins[j]))
            if obj is not None:
                inputs[j] = obj
        wrt = [inputs[i] for i in kw["diff"]]
        before = [t._impl.is_traced for t in wrt]
        for t in wrt:
            t._impl.is_traced = True
        try:
            with config.tracing(False):
                out = fwd.run(fkw, inputs, keep_graph=True) if isinstance(fwd, WhileOp) else fwd.run(fkw, inputs)
                leaves = [l for l in pytree.tree_leaves(out) if isinstance(l, Tensor)]
                tr = Trace(tuple(wrt), leaves)
                tr.compute()
                gmap = backward_on_trace(tr, [given[k] if k in given else zeros_like(l) for k, l in enumerate(leaves)])
                grads = [gmap[t] if t in gmap else zeros_like(t) for t in wrt]
                realize_all(*grads)
        finally:
            for t, b in zip(wrt, before):
                t._impl.is_traced = b
        return [list(g._impl._buffers) for g in grads]


_cond_op, _while_op, _host_vjp_op = CondOp(), WhileOp(), HostVjpOp()
WhileLoopOp = WhileOp           # the reference's name (nabla/ops/control_flow.py:314)


class ScanOp:
    """`scan` under the reference's op name (nabla/ops/control_flow.py:453). There is no node of its
    own: the loop is unrolled while tracing, so each step's ops are recorded (and differentiated)
    like any others."""

    name = "scan"

    def __call__(self, f, init, xs, length=None, reverse: bool = False):
        return scan(f, init, xs, length=length, reverse=reverse)


def _same_structure(a_leaves: list, b_leaves: list, what: str) -> None:
    if len(a_leaves) != len(b_leaves):
        raise ValueError(f"{what}: the two sides return different numbers of values")
    for x, y in zip(a_leaves, b_leaves):
        if isinstance(x, Tensor) != isinstance(y, Tensor):
            raise ValueError(f"{what}: a value is a tensor on one side only")
        if isinstance(x, Tensor) and (tuple(x._impl._shape) != tuple(y._impl._shape) or x.dtype is not y.dtype):
            raise ValueError(f"{what}: shapes / dtypes differ: {tuple(x.shape)} {x.dtype} vs {tuple(y.shape)} {y.dtype}")


def cond(pred, true_fn: Callable, false_fn: Callable, *operands: Any):
    """Run ``true_fn(*operands)`` or ``false_fn(*operands)`` depending on the scalar ``pred``; both
    branches must produce the same structure of shapes and dtypes.

    Eagerly the predicate is read on the host (one device->host sync) and only the taken branch
    runs. Inside ``compile`` the choice is made again on every call (module docstring)."""
    if isinstance(pred, Tensor) and pred._impl.batch_dims > 0:
        # under vmap with a predicate per example: both branches run, `where` picks per example
        t_leaves, out_td = pytree.tree_flatten(true_fn(*operands))
        f_leaves, _ = pytree.tree_flatten(false_fn(*operands))
        _same_structure(t_leaves, f_leaves, "cond")
        return pytree.tree_unflatten(out_td, [where(pred, a, b) if isinstance(a, Tensor) else a
                                              for a, b in zip(t_leaves, f_leaves)])
    if not (isinstance(pred, Tensor) and config.get_flag("TRACING")):
        return true_fn(*operands) if _host_bool(pred) else false_fn(*operands)
    # both branches are traced lazily to learn (and check) the output structure
    t_out = true_fn(*operands)
    f_out = false_fn(*operands)
    t_leaves, out_td = pytree.tree_flatten(t_out)
    f_leaves, _ = pytree.tree_flatten(f_out)
    _same_structure(t_leaves, f_leaves, "cond")
    if config.is_capturable_trace():
        # stays on the device: both branches are part of the graph, `where` selects per call
        sel = [where(pred, a, b) if isinstance(a, Tensor) else a for a, b in zip(t_leaves, f_leaves)]
        return pytree.tree_unflatten(out_td, sel)
    op_leaves, op_td = pytree.tree_flatten(tuple(operands))
    op_tensors = [l for l in op_leaves if isinstance(l, Tensor)]
    extra = [t for t in _closure_tensors(true_fn, false_fn) if all(t._impl is not o._impl for o in op_tensors)]
    templates = [l for l in t_leaves if isinstance(l, Tensor)]
    kwargs = {"true_fn": true_fn, "false_fn": false_fn, "operand_treedef": op_td, "n_operands": len(op_tensors),
              "operand_leaves": [(isinstance(l, Tensor), None if isinstance(l, Tensor) else l) for l in op_leaves]}
    outs = iter(_cond_op.build([pred, *op_tensors, *extra], templates, kwargs))
    return pytree.tree_unflatten(out_td, [next(outs) if isinstance(l, Tensor) else l for l in t_leaves])


def _n_positional(fn: Callable) -> int | None:
    """Number of positional parameters ``fn`` accepts (None: any number, or unknown)."""
    import inspect

    try:
        params = inspect.signature(fn).parameters.values()
    except (TypeError, ValueError):
        return None
    n = 0
    for p in params:
        if p.kind is p.VAR_POSITIONAL:
            return None
        if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD):
            n += 1
    return n


def _apply_state(fn: Callable, state: tuple):
    """Call a loop function on the loop state the way the reference does (nabla/ops/control_flow.py:
    419-436): ONE argument holding the whole state, i.e. ``fn((i, acc))`` for a tuple state. A function
    written with one parameter per element of a tuple state (``lambda i, acc: ...``) is called
    unpacked instead; for a single-tensor state the two are the same."""
    if len(state) == 1:
        return fn(state[0])
    n = _n_positional(fn)
    if n is not None and n == len(state):
        return fn(*state)
    return fn(state)


def _while_eager(cond_fn: Callable, body_fn: Callable, state: tuple, max_iters: int | None = None,
                 realize: bool = True) -> tuple:
    n = 0
    while True:
        go = _apply_state(cond_fn, state)
        if isinstance(go, Tensor) and go._impl.batch_dims > 0:
            # under vmap with a condition per example: iterate while any example wants to, and let
            # only those examples take the new state
            go.realize()
            if not any(bool(b.any().item()) for b in go._impl._buffers):
                break
            new = _apply_state(body_fn, state)
            new = tuple(new) if isinstance(new, (tuple, list)) else (new,)
            old_leaves, td = pytree.tree_flatten(state)
            new_leaves, _ = pytree.tree_flatten(new)
            state = tuple(pytree.tree_unflatten(td, [where(go, a, b) if isinstance(a, Tensor) else a
                                                     for a, b in zip(new_leaves, old_leaves)]))
        else:
            if not _host_bool(go):
                break
            new = _apply_state(body_fn, state)
            state = tuple(new) if isinstance(new, (tuple, list)) else (new,)
        if realize:
            realize_all(*pytree.tensor_leaves(state))
        n += 1
        if max_iters is not None and n >= max_iters:
            break
    return state


def while_loop(cond_fn: Callable, body_fn: Callable, init_val: Any):
    """``while cond_fn(state): state = body_fn(state)`` (reference: nabla/ops/control_flow.py:560-577).
    ``init_val`` may be a single value or a tuple / list of pytrees, handed to both functions as one
    argument; the loop state is realized every iteration so the lazy graph does not grow with the trip
    count. Inside ``compile`` the whole loop is one recorded node whose trip count follows each
    call's data (module docstring)."""
    is_tuple = isinstance(init_val, (tuple, list))
    state = tuple(init_val) if is_tuple else (init_val,)
    st_leaves, st_td = pytree.tree_flatten(state)
    st_tensors = [l for l in st_leaves if isinstance(l, Tensor)]
    if config.get_flag("TRACING") and st_tensors:
        # one lazy application of the body checks that the state keeps its structure
        probe = _apply_state(body_fn, state)
        probe = tuple(probe) if isinstance(probe, (tuple, list)) else (probe,)
        _same_structure(st_leaves, pytree.tree_flatten(probe)[0], "while_loop")
        extra = [t for t in _closure_tensors(cond_fn, body_fn) if all(t._impl is not o._impl for o in st_tensors)]
        kwargs = {"cond_fn": cond_fn, "body_fn": body_fn, "state_treedef": st_td, "n_state": len(st_tensors),
                  "state_leaves": [(isinstance(l, Tensor), None if isinstance(l, Tensor) else l) for l in st_leaves]}
        outs = iter(_while_op.build([*st_tensors, *extra], st_tensors, kwargs))
        state = tuple(pytree.tree_unflatten(st_td, [next(outs) if isinstance(l, Tensor) else l for l in st_leaves]))
    else:
        state = _while_eager(cond_fn, body_fn, state)
    return (type(init_val)(state) if isinstance(init_val, list) else state) if is_tuple else state[0]


def scan(f: Callable, init: Any, xs: Any, length: int | None = None, reverse: bool = False):
    """``carry, y_t = f(carry, x_t)`` over the leading axis of ``xs`` (unrolled in Python, so it
    is differentiable). Returns ``(final_carry, stacked ys)``. ``reverse=True`` walks the axis from
    its end; ``ys[t]`` still belongs to ``xs[t]`` (the reference accepts the flag but does not
    implement it, nabla/ops/control_flow.py:598)."""
    from .view import stack

    leaves = pytree.tensor_leaves(xs)
    n = length if length is not None else (int(leaves[0].shape[0]) if leaves else 0)
    carry = init
    ys = []
    for t in (range(n - 1, -1, -1) if reverse else range(n)):
        x_t = pytree.tree_map(lambda a: a[t] if isinstance(a, Tensor) else a, xs)
        carry, y = f(carry, x_t)
        ys.append(y)
    if reverse:
        ys.reverse()
    if not ys or ys[0] is None:
        return carry, None
    flat0, td = pytree.tree_flatten(ys[0])
    cols = [[pytree.tree_leaves(y)[i] for y in ys] for i in range(len(flat0))]
    stacked = [stack(c, axis=0) for c in cols]
    return carry, pytree.tree_unflatten(td, stacked)
