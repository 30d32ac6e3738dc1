"""jaxpr-like text rendering of a ``Trace`` (reference: nabla/core/graph/tracing.py:417-680).

    fn(%a1: f32[4,8], %a2: f32[8]) {
      %v1: f32[4,8] = mul(%a1, %a2)
      spmd @mesh {
        %v2: f32[4,8](<dp, *>)(local=[2,8]) = shard(%v1, ...)
      }
      return %v2
    }
"""
from __future__ import annotations

from ..tensor.impl import TensorImpl

COMM_OPS = {"shard", "all_gather", "all_reduce", "reduce_scatter", "all_to_all", "ppermute", "gather_all_axes",
            "distributed_broadcast", "axis_index", "pmean", "reshard", "transfer_to"}


def _fmt_val(v) -> str:
    if isinstance(v, (tuple, list)) and len(v) > 8:
        return "(" + ", ".join(_fmt_val(x) for x in v[:8]) + ", ...)"
    if isinstance(v, float):
        return f"{v:g}"
    if hasattr(v, "axis_names") and hasattr(v, "name"):
        return f"@{v.name}"
    return repr(v)


class GraphPrinter:
    def __init__(self, trace):
        self.trace = trace
        self.names: dict[int, str] = {}
        self._n_const = 0
        self._n_val = 0

    def _name(self, impl: TensorImpl, kind: str = "v") -> str:
        k = id(impl)
        if k not in self.names:
            if kind == "a":
                self.names[k] = f"%a{len([n for n in self.names.values() if n.startswith('%a')]) + 1}"
            elif kind == "c":
                self._n_const += 1
                self.names[k] = f"%c{self._n_const}"
            else:
                self._n_val += 1
                self.names[k] = f"%v{self._n_val}"
        return self.names[k]

    def to_string(self) -> str:
        tr = self.trace
        lines = []
        args = ", ".join(f"{self._name(i, 'a')}: {i.format_metadata()}" for i in tr.input_impls)
        lines.append(f"fn({args}) {{")
        in_spmd = None
        for node in tr.nodes:
            outs = [o for o in node.outputs() if o is not None]
            ins = []
            for a in node.arg_leaves:
                if isinstance(a, TensorImpl):
                    if id(a) not in self.names:
                        self._name(a, "c" if a.output_refs is None else "v")
                    ins.append(self.names[id(a)])
            mesh = None
            for o in outs:
                if o.sharding is not None:
                    mesh = o.sharding.mesh
            if mesh is not None and in_spmd != mesh.name:
                if in_spmd is not None:
                    lines.append("  }")
                lines.append(f"  spmd @{mesh.name} {{")
                in_spmd = mesh.name
            elif mesh is None and in_spmd is not None:
                lines.append("  }")
                in_spmd = None
            indent = "    " if in_spmd else "  "
            lhs = ", ".join(f"{self._name(o)}: {o.format_metadata()}" for o in outs) or "_"
            kw = ", ".join(f"{k}={_fmt_val(v)}" for k, v in node.op_kwargs.items() if v is not None)
            call = f"{node.op.name}({', '.join(ins)}{', ' + kw if kw and ins else kw})"
            if node.op.name in COMM_OPS:
                call = f"\033[1m{call}\033[0m" if False else call
            lines.append(f"{indent}{lhs} = {call}")
        if in_spmd is not None:
            lines.append("  }")
        rets = ", ".join(self.names.get(id(o), self._name(o, "c")) for o in tr.output_impls)
        lines.append(f"  return {rets}")
        lines.append("}")
        return "\n".join(lines)
