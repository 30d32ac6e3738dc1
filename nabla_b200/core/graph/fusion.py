"""Plan construction with peephole fusion.

``build_plan`` turns a topologically ordered node list into steps. Patterns recognised on
CUDA bf16 tensors:

* ``matmul -> add(bias row) [-> relu | gelu]`` where the intermediates have no other
  consumer: one tcgen05 GEMM launch with the bias/activation epilogue
  (replaces the composition of nabla/nn/functional/layers.py:30-35).

* ``matmul | linear (no bias) -> all_reduce(sum) | reduce_scatter`` on a mesh that runs one
  process per GPU: one launch of the fused GEMM + collective kernel (tiles are reduced over
  NVLink while later tiles are still being multiplied).
* ``linear (+bias) -> add(residual)``: the residual is added in the GEMM epilogue.
* ``matmul -> dact_mul`` (backward of linear + relu/gelu): the activation derivative is applied in
  the GEMM epilogue.
* compiled replays with donated optimizer state: ``matmul -> all_reduce(dp) -> adam_wstep`` becomes a
  GEMM that writes its (unreduced) weight gradient into a symmetric arena plus one kernel that sums
  the ranks' gradients while reading them and applies AdamW in place (``gemm_to_arena`` /
  ``adamw_reduce`` steps, set up by ``transforms/compile.py``).
* ``all_gather(rows) -> linear | matmul [-> dact_mul]``: one launch that pulls the peers' rows while the tensor
  cores already work on the rows that are there; the gathered tensor is still produced.

Every other node is a plain 'op' step. Fusion never changes which tensors exist: fused-away
intermediates that are still referenced are simply not fusable.
"""
from __future__ import annotations

import os

import torch

from ..tensor.impl import TensorImpl
from .tracing import OpNode


_FUSE_RESIDUAL = os.environ.get("NABLA_B200_FUSE_RESIDUAL", "0") == "1"


def enabled() -> bool:
    return os.environ.get("NABLA_B200_NO_PLAN", "0") != "1"


def _single_consumer_map(nodes: list[OpNode], targets) -> dict[int, list[int]]:
    cons: dict[int, list[int]] = {}
    for ni, n in enumerate(nodes):
        for a in n.arg_leaves:
            if isinstance(a, TensorImpl):
                cons.setdefault(id(a), []).append(ni)
    return cons


def build_plan(nodes: list[OpNode], targets: list[TensorImpl]):
    from .engine import Plan

    cons = _single_consumer_map(nodes, targets)
    target_ids = {id(t) for t in targets}
    pos = {id(n): i for i, n in enumerate(nodes)}
    used = [False] * len(nodes)
    steps = []
    producer: dict[int, int] = {}
    for ni, nd in enumerate(nodes):
        for o_ in nd.outputs():
            if o_ is not None:
                producer[id(o_)] = ni

    def sole_output(n: OpNode):
        outs = n.outputs()
        return outs[0] if len(outs) == 1 else None

    def fusable_intermediate(impl: TensorImpl) -> bool:
        # only this plan consumes it, exactly once; not requested by the caller; not traced
        return (impl is not None and id(impl) not in target_ids and not impl.is_traced
                and len(cons.get(id(impl), [])) == 1 and impl.sharding is None and impl.batch_dims == 0)

    for i, n in enumerate(nodes):
        if used[i]:
            continue
        chain = None
        if n.op.name == "matmul" and _is_cuda_bf16_2d(n):
            o = sole_output(n)
            if fusable_intermediate(o):
                j = cons[id(o)][0]
                m = nodes[j]
                if not used[j] and m.op.name == "add" and _is_bias_add(m, o):
                    chain = [i, j]
                    o2 = sole_output(m)
                    if fusable_intermediate(o2):
                        k = cons[id(o2)][0]
                        a = nodes[k]
                        if not used[k] and a.op.name in ("relu", "gelu") and not (
                                a.op.name == "gelu" and a.kwargs.get("approximate", "none") not in ("none", "tanh")):
                            chain = [i, j, k]
        kind = "linear_epilogue"
        if chain is None and n.op.name == "matmul" and _is_local_gemm(n):
            dk = _dact_consumer(n, nodes, cons, target_ids, used)
            if dk is not None:
                chain = [i, dk]
                kind = "gemm_dact"
        if chain is None and _FUSE_RESIDUAL and n.op.name == "linear" and n.kwargs.get("activation") is None \
                and _is_local_linear(n):
            # y = x @ w + b followed by "+ residual" of the same shape: the residual is added in the epilogue
            o = sole_output(n)
            if (o is not None and id(o) not in target_ids and len(cons.get(id(o), [])) == 1 and o.batch_dims == 0
                    and not (o.sharding is not None and o.sharding.partial_sum_axes)):
                k = cons[id(o)][0]
                a_ = nodes[k]
                if not used[k] and a_.op.name == "add" and _same_layout_addend(a_, o):
                    chain = [i, k]
                    kind = "gemm_residual"
        if chain is None and n.op.name in ("matmul", "linear") and _is_partial_gemm(n):
            o = sole_output(n)
            # a traced product may stay an unrealized promise: no backward rule reads its value
            if o is not None and id(o) not in target_ids and len(cons.get(id(o), [])) == 1 and o.batch_dims == 0:
                j = cons[id(o)][0]
                m = nodes[j]
                if not used[j] and m.op.name == "all_reduce" and _is_sum_over_partials(m, o):
                    chain = [i, j]
                    kind = "gemm_all_reduce"
                elif not used[j] and m.op.name == "reduce_scatter" and _is_scatter_of_partials(m, o):
                    chain = [i, j]
                    kind = "gemm_reduce_scatter"
                    # + bias row and + residual fold into the pass that sums the partial row blocks
                    cur = sole_output(m)
                    for want in ("bias", "residual"):
                        if cur is None or id(cur) in target_ids or len(cons.get(id(cur), [])) != 1 or cur.batch_dims:
                            break
                        k = cons[id(cur)][0]
                        a = nodes[k]
                        if used[k] or a.op.name != "add" or _rs_addend(a, cur) != want:
                            if want == "bias":
                                continue          # no bias: the next add may still be the residual
                            break
                        chain.append(k)
                        cur = sole_output(a)
        if chain is None and n.op.name == "all_gather" and _is_row_gather(n):
            o = sole_output(n)
            users = cons.get(id(o), []) if o is not None else []
            if o is not None and users and o.batch_dims == 0:
                j = min(users)
                m = nodes[j]
                if not used[j] and m.op.name in ("matmul", "linear") and _is_gathered_gemm(m, o):
                    # the GEMM may move up to right after its other inputs exist, but not past
                    # another user of the gathered tensor
                    ready = i
                    for x in m.input_impls():
                        if x is not o and id(x) in producer:
                            ready = max(ready, producer[id(x)])
                    idxs = [i, j]
                    dk = _dact_consumer(m, nodes, cons, target_ids, used)
                    if dk is not None:
                        z = nodes[dk].input_impls()[1]
                        zr = producer.get(id(z), -1)
                        if max(ready, zr) < j:
                            ready = max(ready, zr)
                            idxs.append(dk)
                    if ready < j and all(u > ready for u in users):
                        for c_ in idxs:
                            used[c_] = True
                        steps.append((ready + 0.5, ("all_gather_gemm", tuple(idxs))))
                        continue
        if chain is not None:
            # schedule at the position of the LAST node of the chain
            last = chain[-1]
            for c in chain:
                used[c] = True
            steps.append((last, (kind, tuple(chain))))
        else:
            used[i] = True
            steps.append((i, ("op", (i,))))
    steps.sort(key=lambda s: s[0])
    return Plan([s for _, s in steps], len(nodes))


def _is_cuda_bf16_2d(n: OpNode) -> bool:
    ins = n.input_impls()
    if len(ins) != 2:
        return False
    a, b = ins
    if a.sharding is not None or b.sharding is not None or a.batch_dims or b.batch_dims:
        return False
    from ...types import DType

    return (a.device.label == "gpu" and a.dtype is DType.bfloat16 and b.dtype is DType.bfloat16
            and len(b._shape) == 2 and len(a._shape) >= 2)


def _is_local_gemm(n: OpNode) -> bool:
    """bf16 GPU ``x @ w`` (w 2-D) whose product needs no collective."""
    ins = n.input_impls()
    if len(ins) != 2:
        return False
    a, b = ins
    outs = n.outputs()
    o = outs[0] if len(outs) == 1 else None
    if o is None or (o.sharding is not None and o.sharding.partial_sum_axes):
        return False
    from ...types import DType

    return (a.device.label == "gpu" and a.dtype is DType.bfloat16 and b.dtype is DType.bfloat16
            and len(b._shape) == 2 and len(a._shape) >= 2 and a.batch_dims == 0 and b.batch_dims == 0)


def _is_local_linear(n: OpNode) -> bool:
    ins = n.input_impls()
    if len(ins) not in (2, 3):
        return False
    a, b = ins[0], ins[1]
    from ...types import DType

    return (a.device.label == "gpu" and a.dtype is DType.bfloat16 and b.dtype is DType.bfloat16
            and len(b._shape) == 2 and len(a._shape) >= 2 and a.batch_dims == 0 and b.batch_dims == 0)


def _same_layout_addend(add: OpNode, x: TensorImpl) -> bool:
    ins = add.input_impls()
    if len(ins) != 2:
        return False
    other = ins[1] if ins[0] is x else ins[0] if ins[1] is x else None
    if other is None or other is x or other.batch_dims or other.dtype is not x.dtype or tuple(other._shape) != tuple(x._shape):
        return False
    sa = [tuple(d.axes) for d in other.sharding.dim_specs] if other.sharding is not None else None
    sb = [tuple(d.axes) for d in x.sharding.dim_specs] if x.sharding is not None else None
    if sa != sb:
        return False
    return not (other.sharding is not None and other.sharding.partial_sum_axes)


def _dact_consumer(mm: OpNode, nodes, cons, target_ids, used) -> int | None:
    """Index of the ``dact_mul`` node that is the only reader of ``mm``'s product, if any."""
    outs = mm.outputs()
    o = outs[0] if len(outs) == 1 else None
    if o is None or id(o) in target_ids or o.batch_dims or len(cons.get(id(o), [])) != 1:
        return None
    if mm.kwargs.get("activation") is not None or len(mm.input_impls()) != 2:
        return None
    k = cons[id(o)][0]
    d = nodes[k]
    if used[k] or d.op.name != "dact_mul" or d.kwargs.get("activation") not in ("relu", "gelu", "gelu_tanh"):
        return None
    ins = d.input_impls()
    if len(ins) != 2 or ins[0] is not o or ins[1] is o or tuple(ins[1]._shape) != tuple(o._shape):
        return None
    return k


def _is_partial_gemm(n: OpNode) -> bool:
    """bf16 ``x @ w`` on a one-process-per-GPU mesh whose product is a pending partial sum."""
    ins = n.input_impls()
    if len(ins) != 2 or n.kwargs.get("activation") is not None:
        return False
    a, b = ins
    outs = n.outputs()
    o = outs[0] if len(outs) == 1 else None
    if o is None or o.sharding is None or not o.sharding.partial_sum_axes or not o.sharding.mesh.is_distributed:
        return False
    from ...types import DType

    if not (a.device.label == "gpu" and a.dtype is DType.bfloat16 and b.dtype is DType.bfloat16
            and len(b._shape) == 2 and len(a._shape) >= 2 and a.batch_dims == 0 and b.batch_dims == 0):
        return False
    from ...parallel import symm

    return symm.is_ready()


def _is_sum_over_partials(m: OpNode, mm_out: TensorImpl) -> bool:
    axes = set(m.kwargs.get("reduce_axes", ()))
    if m.kwargs.get("reduce_op", "sum") != "sum" or not axes:
        return False
    sp = mm_out.sharding
    if _group_size(sp.mesh, axes) <= 1:
        return False           # a group of one rank: the all-reduce is the identity, keep the plain GEMM
    # a plain sum of the partial products: no dim of the operand is split over the reduced axes
    return axes <= set(sp.partial_sum_axes) and not any(set(d.axes) & axes for d in sp.dim_specs)


def _group_size(mesh, axes) -> int:
    n = 1
    for a in axes:
        n *= mesh.get_axis_size(a)
    return n


def _is_scatter_of_partials(m: OpNode, mm_out: TensorImpl) -> bool:
    axes = set(m.kwargs.get("scatter_axes", ()))
    dim = m.kwargs.get("dim")
    sp = mm_out.sharding
    if not axes or dim is None or dim >= len(mm_out._shape) - 1 or _group_size(sp.mesh, axes) <= 1:
        return False
    return axes <= set(sp.partial_sum_axes) and not any(set(d.axes) & axes for d in sp.dim_specs)


def _rs_addend(add: OpNode, x: TensorImpl) -> str | None:
    """What ``add`` adds to the reduce-scatter result ``x``: 'bias' (one row, no split dims),
    'residual' (same shape and layout) or None."""
    ins = add.input_impls()
    if len(ins) != 2:
        return None
    other = ins[1] if ins[0] is x else ins[0] if ins[1] is x else None
    if other is None or other.batch_dims or other.dtype is not x.dtype:
        return None
    split = [tuple(d.axes) for d in other.sharding.dim_specs] if other.sharding is not None else []
    if len(other._shape) >= 1 and other._shape[-1] == x._shape[-1] and all(d == 1 for d in other._shape[:-1]) \
            and not any(split):
        return "bias"
    if tuple(other._shape) == tuple(x._shape) and other.sharding is not None and x.sharding is not None and \
            split == [tuple(d.axes) for d in x.sharding.dim_specs] and not other.sharding.partial_sum_axes:
        return "residual"
    return None


def _is_row_gather(n: OpNode) -> bool:
    ins = n.input_impls()
    if len(ins) != 1:
        return False
    x = ins[0]
    dim = n.kwargs.get("dim")
    if x.sharding is None or not x.sharding.mesh.is_distributed or dim is None or dim >= len(x._shape) - 1:
        return False
    if not x.sharding.dim_specs[dim].axes or x.sharding.partial_sum_axes or x.batch_dims:
        return False
    if _group_size(x.sharding.mesh, x.sharding.dim_specs[dim].axes) <= 1:
        return False
    from ...types import DType

    if not (x.device.label == "gpu" and x.dtype is DType.bfloat16):
        return False
    from ...parallel import symm

    return symm.is_ready()


def _is_gathered_gemm(m: OpNode, gathered: TensorImpl) -> bool:
    ins = m.input_impls()
    if len(ins) < 2 or ins[0] is not gathered or any(x is gathered for x in ins[1:]):
        return False
    w = ins[1]
    from ...types import DType

    if not (w.dtype is DType.bfloat16 and len(w._shape) == 2 and w.batch_dims == 0):
        return False
    act = m.kwargs.get("activation")
    return act in (None, "relu", "gelu", "gelu_tanh")


def _is_bias_add(m: OpNode, mm_out: TensorImpl) -> bool:
    ins = m.input_impls()
    if len(ins) != 2:
        return False
    other = ins[1] if ins[0] is mm_out else ins[0] if ins[1] is mm_out else None
    if other is None or other.sharding is not None or other.batch_dims:
        return False
    n = mm_out._shape[-1]
    shp = other._shape
    return len(shp) >= 1 and shp[-1] == n and all(d == 1 for d in shp[:-1]) and other.dtype is mm_out.dtype


def run_fused(kind: str, group: list[OpNode], keep_graph: bool = False, arena_blocks: dict | None = None) -> None:
    """``arena_blocks`` (compiled replays only): {id(impl): (arena, offset)} of gathered tensors
    that live in a symmetric arena; the replay frees them after their last use."""
    from .engine import store_outputs

    if kind == "linear_epilogue":
        from ...native.gemm import gemm_bf16

        mm, add = group[0], group[1]
        act = group[2] if len(group) > 2 else None
        a, b = [x._buffers[0] for x in mm.input_impls()]
        mm_out = mm.outputs()[0]
        bias_impl = [x for x in add.input_impls() if x is not mm_out][0]
        bias = bias_impl._buffers[0]
        epi = "bias" if act is None else act.op.name
        tanh = act is not None and act.op.name == "gelu" and act.kwargs.get("approximate", "none") == "tanh"
        a2 = a.reshape(-1, a.shape[-1])
        out = gemm_bf16(a2, b, bias=bias, epilogue=epi, gelu_tanh=tanh).reshape(*a.shape[:-1], b.shape[-1])
        last = group[-1]
        if keep_graph:
            o = last.outputs()[0]
            if o is not None:
                o._buffers = [out]
        else:
            store_outputs(last, [[out]])
        return
    if kind == "gemm_residual":
        from ...native.gemm import gemm_bf16

        lin, add = group
        ins = lin.input_impls()
        a, b = ins[0]._buffers[0], ins[1]._buffers[0]
        bias = ins[2]._buffers[0] if len(ins) > 2 else None
        lin_out = lin.outputs()[0]
        res = [x for x in add.input_impls() if x is not lin_out][0]._buffers[0]
        if a.is_cuda and a.numel() and b.numel():
            n_out = b.shape[-1]
            out = gemm_bf16(a.reshape(-1, a.shape[-1]), b, bias=bias, aux="add",
                            aux_in=res.reshape(-1, n_out)).reshape(*a.shape[:-1], n_out)
            _store(add, [[out]], keep_graph)
        else:
            _plain(lin, keep_graph)
            _plain(add, keep_graph)
        return
    if kind == "gemm_dact":
        from ...native.gemm import gemm_bf16

        mm, da = group
        a, b = [x._buffers[0] for x in mm.input_impls()]
        z = da.input_impls()[1]._buffers[0]
        act = da.kwargs["activation"]
        if a.is_cuda and a.numel() and b.numel():
            n_out = b.shape[-1]
            out = gemm_bf16(a.reshape(-1, a.shape[-1]), b, aux="drelu" if act == "relu" else "dgelu",
                            aux_in=z.reshape(-1, n_out), gelu_tanh=act == "gelu_tanh").reshape(*a.shape[:-1], n_out)
            _store(da, [[out]], keep_graph)
        else:
            _plain(mm, keep_graph)
            _plain(da, keep_graph)
        return
    if kind == "all_reduce_bucket":
        # many small partial sums over the same device group: one flat all-reduce
        from ...parallel import backend

        first = group[0]
        mesh = first.input_impls()[0].sharding.mesh
        axes = [x for x in mesh.axis_names if x in first.kwargs["reduce_axes"]]
        xs = [n_.input_impls()[0]._buffers[0] for n_ in group]
        flat = torch.cat([x.reshape(-1) for x in xs])
        red = backend.all_reduce(flat, mesh, axes, "sum")
        off = 0
        for n_, x in zip(group, xs):
            k = x.numel()
            _store(n_, [[red[off: off + k].view(x.shape)]], keep_graph)
            off += k
        backend.stats["bucketed_all_reduce"] = backend.stats.get("bucketed_all_reduce", 0) + len(group)
        return
    if kind == "gemm_to_arena":
        # weight gradient of a data-parallel replica group: keep it unreduced, in the arena; the
        # matching adamw_reduce step sums it over the group while it reads it
        from ...native.gemm import gemm_bf16
        from ...parallel import symm

        mm, ar = group
        a, b = [x._buffers[0] for x in mm.input_impls()]
        ar_out = ar.outputs()[0]
        mesh = ar.input_impls()[0].sharding.mesh
        axes = [x for x in mesh.axis_names if x in ar.kwargs["reduce_axes"]]
        arena = symm.arena(mesh, axes) if arena_blocks is not None else None
        m_rows = a.numel() // max(a.shape[-1], 1)
        nbytes = m_rows * b.shape[-1] * 2
        off = arena.alloc(nbytes) if (arena is not None and ar_out is not None and a.dim() == 2
                                      and os.environ.get("NABLA_B200_FUSE_DP_ADAMW", "0") == "1") else None
        if off is None:
            return run_fused("gemm_all_reduce", group, keep_graph, arena_blocks)
        out = arena.buf[off: off + nbytes].view(torch.bfloat16).view(m_rows, b.shape[-1])
        gemm_bf16(a, b, out=out)
        arena_blocks[id(ar_out)] = (arena, off)
        _store(ar, [[out]], keep_graph)
        return
    if kind == "adamw_reduce":
        from ...parallel import backend, symm

        (ad,) = group
        ins = ad.input_impls()
        blk = arena_blocks.get(id(ins[1])) if arena_blocks is not None else None
        if blk is None:
            return _plain(ad, keep_graph)
        kw = ad.kwargs
        p_, m_, v_ = ins[0]._buffers[0], ins[2]._buffers[0], ins[3]._buffers[0]
        hyper = ins[4]._buffers[0].contiguous() if (len(ins) > 4 and kw.get("bias_correction", True)) else None
        mesh, axes = arena_blocks[("dp_group", id(ad))]
        symm.adamw_reduce(p_, m_, v_, blk[1], mesh, axes, lr=kw["lr"], b1=kw["beta1"], b2=kw["beta2"], eps=kw["eps"],
                          wd=kw["weight_decay"], step=kw.get("step_value") if kw.get("bias_correction", True) else None,
                          hyper=hyper)
        backend.stats["fused_dp_adamw"] = backend.stats.get("fused_dp_adamw", 0) + 1
        _store(ad, [[p_], [m_], [v_]], keep_graph)
        return
    if kind == "gemm_all_reduce":
        from ...parallel import backend, symm

        mm, ar = group
        a, b = [x._buffers[0] for x in mm.input_impls()]
        mesh = mm.outputs()[0].sharding.mesh if mm.outputs()[0] is not None else ar.input_impls()[0].sharding.mesh
        axes = [x for x in mesh.axis_names if x in ar.kwargs["reduce_axes"]]
        split = 1
        if a.is_cuda and a.dim() == 2 and a.dtype == torch.bfloat16:
            from ...native.gemm import gemm_bf16, split_k_factor

            split = split_k_factor(a.shape[0], b.shape[-1], a.shape[1])
        if split > 1:
            # few output tiles and a very long K (weight gradients of a tensor-parallel shard): the
            # fused kernel's fixed 128 x 256 tiles would leave most SMs idle, so the product runs
            # as K slices on all SMs and the small result is all-reduced on its own
            out = backend.all_reduce(gemm_bf16(a, b), mesh, axes, "sum")
            backend.stats["split_k_gemm_all_reduce"] = backend.stats.get("split_k_gemm_all_reduce", 0) + 1
        elif symm.gemm_all_reduce_supported(a, b):
            out = symm.gemm_all_reduce(a, b, mesh, axes).clone().reshape(*a.shape[:-1], b.shape[-1])
            backend.stats["fused_gemm_all_reduce"] = backend.stats.get("fused_gemm_all_reduce", 0) + 1
        else:
            y = mm.op.kernel(a, b)
            out = backend.all_reduce(y, mesh, axes, "sum")
        if keep_graph:
            o = ar.outputs()[0]
            if o is not None:
                o._buffers = [out]
        else:
            store_outputs(ar, [[out]])
        return
    if kind == "gemm_reduce_scatter":
        from ...parallel import backend, symm

        mm, rs = group[0], group[1]
        a, b = [x._buffers[0] for x in mm.input_impls()]
        bias = resid = None
        cur = rs.outputs()[0]
        for add in group[2:]:
            other = [x for x in add.input_impls() if x is not cur][0]
            if _rs_addend(add, cur) == "bias":
                bias = other._buffers[0]
            else:
                resid = other._buffers[0]
            cur = add.outputs()[0]
        mesh = rs.input_impls()[0].sharding.mesh
        axes = [x for x in mesh.axis_names if x in rs.kwargs["scatter_axes"]]
        dim = rs.kwargs["dim"]
        world = 1
        for x in axes:
            world *= mesh.get_axis_size(x)
        lead = tuple(a.shape[:-1])
        inner = 1
        for d in lead[dim + 1:]:
            inner *= d
        m_total = 1
        for d in lead:
            m_total *= d
        cs = (lead[dim] // world) * inner if lead[dim] % world == 0 else 0
        if (symm.gemm_all_reduce_supported(a, b) and symm.chunked_supported(m_total, cs, world)
                and os.environ.get("NABLA_B200_FUSE_RS", "1") != "0"):
            y = symm.gemm_reduce_scatter(a, b, mesh, axes, cs, bias=bias, residual=resid)
            out = y.reshape(*lead[:dim], lead[dim] // world, *lead[dim + 1:], b.shape[-1])
            backend.stats["fused_gemm_reduce_scatter"] = backend.stats.get("fused_gemm_reduce_scatter", 0) + 1
            _store(group[-1], [[out]], keep_graph)
        else:
            for n_ in group:
                _plain(n_, keep_graph)
        return
    if kind == "all_gather_gemm":
        from ...parallel import backend, symm

        ag, mm = group[0], group[1]
        da = group[2] if len(group) > 2 else None
        x_impl = ag.input_impls()[0]
        x = x_impl._buffers[0]
        dim = ag.kwargs["dim"]
        mesh = x_impl.sharding.mesh
        axes = list(x_impl.sharding.dim_specs[dim].axes)
        world = 1
        for a_ in axes:
            world *= mesh.get_axis_size(a_)
        ins = mm.input_impls()
        w = ins[1]._buffers[0]
        bias = ins[2]._buffers[0] if len(ins) > 2 else None
        act = mm.kwargs.get("activation")
        lead = tuple(x.shape[:-1])
        cs = 1
        for d in lead[dim:]:
            cs *= d
        m_total = world * x.numel() // max(x.shape[-1], 1)
        k, n = x.shape[-1], w.shape[-1]
        even = all(s == x.shape[dim] for s in
                   [_local_extent(x_impl, dim, r) for r in mesh.group_of(mesh.rank, axes)])
        if (even and symm.chunked_supported(m_total, cs, world) and n % 8 == 0 and k % 8 == 0 and w.dim() == 2
                and m_total // world * k * 2 + 4096 <= symm.DEFAULT_BYTES - 65536
                and os.environ.get("NABLA_B200_FUSE_AG", "1") != "0"):
            epi = "none" if act is None else ("relu" if act == "relu" else "gelu")
            off = None
            ag_out = ag.outputs()[0]
            if arena_blocks is not None and ag_out is not None and os.environ.get("NABLA_B200_AG_PUSH", "1") != "0":
                ar = symm.arena(mesh, axes)
                if ar is not None:
                    off = ar.alloc(m_total * k * 2)
                    if off is not None:
                        arena_blocks[id(ag_out)] = (ar, off)
            dact = None
            if da is not None:
                dact = (da.input_impls()[1]._buffers[0], da.kwargs["activation"])
            res = symm.all_gather_gemm(x, w, mesh, axes, cs, bias=bias, epilogue=epi, gelu_tanh=act == "gelu_tanh",
                                       store_preact=act is not None, arena_off=off, dact=dact)
            full_shape = (*lead[:dim], lead[dim] * world, *lead[dim + 1:])
            _store(ag, [[res[0].reshape(*full_shape, k)]], keep_graph)
            outs = [[res[1].reshape(*full_shape, n)]]
            if act is not None:
                outs.append([res[2].reshape(*full_shape, n)])
            _store(da if da is not None else mm, outs, keep_graph)
            backend.stats["fused_all_gather_gemm"] = backend.stats.get("fused_all_gather_gemm", 0) + 1
        else:
            for n_ in group:
                _plain(n_, keep_graph)
        return
    raise ValueError(f"unknown fused step {kind}")


def _local_extent(impl: TensorImpl, dim: int, device_id: int) -> int:
    from ..sharding.spec import compute_local_shape

    return compute_local_shape(impl._shape, impl.sharding, device_id)[dim]


def _store(node: OpNode, outs, keep_graph: bool) -> None:
    from .engine import store_outputs

    if keep_graph:
        for i, ref in enumerate(node.out_refs):
            o = ref()
            if o is not None:
                o._buffers = outs[i]
    else:
        store_outputs(node, outs)


def _plain(node: OpNode, keep_graph: bool) -> None:
    _store(node, node.op.execute(node), keep_graph)
