"""Plan construction with peephole fusion.

``build_plan`` turns a topologically ordered node list into steps. Patterns recognised on
CUDA bf16 tensors:

* ``matmul -> add(bias row) [-> relu | gelu]`` where the intermediates have no other
  consumer: one tcgen05 GEMM launch with the bias/activation epilogue
  (replaces the composition of nabla/nn/functional/layers.py:30-35).

Every other node is a plain 'op' step. Fusion never changes which tensors exist: fused-away
intermediates that are still referenced are simply not fusable.
"""
from __future__ import annotations

import os

import torch

from ..tensor.impl import TensorImpl
from .tracing import OpNode


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
        if chain is not None and all(c == chain[0] + d for d, c in enumerate(chain)) is False:
            # the fused step runs at the position of its last node; all inputs of the later
            # nodes must already be available there, which holds because they precede it
            pass
        if chain is not None:
            # schedule at the position of the LAST node of the chain
            last = chain[-1]
            for c in chain:
                used[c] = True
            steps.append((last, ("linear_epilogue", tuple(chain))))
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


def run_fused(kind: str, group: list[OpNode], keep_graph: bool = False) -> None:
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
    raise ValueError(f"unknown fused step {kind}")
