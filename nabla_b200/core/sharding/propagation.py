"""Factor-based sharding propagation (reference: nabla/core/sharding/propagation.py:42-324).

Every op describes its dimensions with einsum-like *factors*
(``"... m k, ... k n -> ... m n"``). Shardings flow from input dims to factors and from
factors to output dims; a factor that appears in inputs but in no output is *contracting*,
and a sharded contracting factor leaves the output with a pending sum over those mesh axes
(``partial_sum_axes``). Conflicts are resolved first-input-wins, and an axis is claimed by
the first output dimension that asks for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

from .spec import DeviceMesh, DimSpec, ShardingSpec

Mapping = dict[int, list[str]]


@dataclass
class OpShardingRule:
    input_mappings: list[Mapping]
    output_mappings: list[Mapping]
    factor_sizes: dict[str, int] = field(default_factory=dict)

    def get_all_factors(self) -> set[str]:
        out: set[str] = set()
        for m in self.input_mappings + self.output_mappings:
            for fs in m.values():
                out.update(fs)
        return out

    def get_factor_tensors(self, factor_name: str) -> list[tuple[str, int, int]]:
        """Where a factor appears: ``("input" | "output", operand index, dim index)`` triples."""
        out = []
        for kind, maps in (("input", self.input_mappings), ("output", self.output_mappings)):
            for t, m in enumerate(maps):
                out += [(kind, t, d) for d, fs in m.items() if factor_name in fs]
        return out

    def get_contracting_factors(self) -> set[str]:
        ins: set[str] = set()
        outs: set[str] = set()
        for m in self.input_mappings:
            for fs in m.values():
                ins.update(fs)
        for m in self.output_mappings:
            for fs in m.values():
                outs.update(fs)
        return ins - outs

    def to_einsum_notation(self) -> str:
        def side(ms):
            return ", ".join(" ".join("(" + " ".join(fs) + ")" if len(fs) != 1 else fs[0]
                                      for _, fs in sorted(m.items())) for m in ms)
        return f"{side(self.input_mappings)} -> {side(self.output_mappings)}"


class OpShardingRuleTemplate:
    """A rule written with ``...`` for leading batch dims, instantiated against shapes."""

    def __init__(self, inputs: list, outputs: list):
        # each operand: list of tokens; token = str | tuple[str,...] | Ellipsis. The reference's form,
        # one ``{dim: [factor names]}`` dict per operand (nabla/core/sharding/propagation.py:107-111),
        # is accepted too and turned into tokens in dim order.
        self.inputs = [self._tokens(m) for m in inputs]
        self.outputs = [self._tokens(m) for m in outputs]

    @staticmethod
    def _tokens(m) -> list:
        if not isinstance(m, dict):
            return list(m)
        out: list = []
        for d in range(max(m) + 1 if m else 0):
            fs = [str(f) for f in m.get(d, [f"_free{d}"])]
            out.append(fs[0] if len(fs) == 1 else tuple(fs))
        return out

    @staticmethod
    def _mapping(tokens: list) -> dict:
        return {d: (list(t) if isinstance(t, tuple) else [t]) for d, t in enumerate(tokens) if t is not Ellipsis}

    @property
    def input_mappings(self) -> list[dict]:
        """The operands' ``{dim: [factors]}`` dicts (dims counted without any ``...``)."""
        return [self._mapping(t) for t in self.inputs]

    @property
    def output_mappings(self) -> list[dict]:
        return [self._mapping(t) for t in self.outputs]

    def to_einsum_notation(self) -> str:
        def one(tokens):
            return " ".join("..." if t is Ellipsis else ("(" + " ".join(t) + ")" if isinstance(t, tuple) else t)
                            for t in tokens)
        return ", ".join(one(t) for t in self.inputs) + " -> " + ", ".join(one(t) for t in self.outputs)

    @staticmethod
    def parse(equation: str, input_shapes: Sequence[Sequence[int]] | None = None) -> "OpShardingRuleTemplate":
        """Template from einsum-like notation. With ``input_shapes`` every ``...`` is expanded at
        once to the batch factors those shapes imply, as the reference's two-argument form does
        (nabla/core/sharding/propagation.py:161-200)."""
        tpl = OpShardingRuleTemplate._parse(equation)
        if input_shapes is None:
            return tpl
        rule = tpl.instantiate(input_shapes)
        return OpShardingRuleTemplate(rule.input_mappings, rule.output_mappings)

    @staticmethod
    def _parse(notation: str) -> "OpShardingRuleTemplate":
        def toks(s: str) -> list:
            out: list = []
            i, s = 0, s.strip()
            parts = s.replace("(", " ( ").replace(")", " ) ").split()
            group = None
            for p in parts:
                if p == "(":
                    group = []
                elif p == ")":
                    out.append(tuple(group))
                    group = None
                elif group is not None:
                    group.append(p)
                elif p == "...":
                    out.append(Ellipsis)
                else:
                    out.append(p)
            return out
        lhs, rhs = notation.split("->")
        return OpShardingRuleTemplate([toks(x) for x in lhs.split(",")], [toks(x) for x in rhs.split(",")])

    def instantiate(self, input_shapes: Sequence[Sequence[int]],
                    output_shapes: Sequence[Sequence[int]] | None = None) -> OpShardingRule:
        sizes: dict[str, int] = {}

        max_batch = 0
        batch_extent: dict[int, int] = {}        # right-aligned batch position -> largest extent over the operands
        for i, toks in enumerate(self.inputs):
            if Ellipsis in toks and i < len(input_shapes):
                nb_ = len(input_shapes[i]) - sum(1 for t in toks if t is not Ellipsis)
                max_batch = max(max_batch, nb_)
                at = toks.index(Ellipsis)
                for b in range(max(nb_, 0)):
                    pos = nb_ - 1 - b
                    batch_extent[pos] = max(batch_extent.get(pos, 1), int(input_shapes[i][at + b]))

        def expand(tokens: list, shape: Sequence[int] | None, operand: int = 0) -> Mapping:
            n_named = sum(1 for t in tokens if t is not Ellipsis)
            if shape is not None:
                n_batch = max(0, len(shape) - n_named) if Ellipsis in tokens else 0
            else:
                # unknown (output) shape: it carries the broadcast of all operands' batch dims
                n_batch = max_batch if Ellipsis in tokens else 0
            mapping: Mapping = {}
            d = 0
            for t in tokens:
                if t is Ellipsis:
                    # batch factors are right-aligned across operands (numpy broadcasting); a size-1
                    # dim that broadcasts against a larger one gets a factor of its own, so the
                    # other operand's sharding of that position is never pushed onto it
                    for b in range(n_batch):
                        pos = n_batch - 1 - b
                        if shape is not None and int(shape[d]) == 1 and batch_extent.get(pos, 1) != 1:
                            mapping[d] = [f"_bcast{operand}_{pos}"]
                        else:
                            mapping[d] = [f"_b{pos}"]
                        d += 1
                else:
                    fs = list(t) if isinstance(t, tuple) else [t]
                    mapping[d] = fs
                    if shape is not None and d < len(shape) and len(fs) == 1:
                        sizes.setdefault(fs[0], int(shape[d]))
                    d += 1
            return mapping

        ins = [expand(t, input_shapes[i] if i < len(input_shapes) else None, i) for i, t in enumerate(self.inputs)]
        outs = [expand(t, output_shapes[i] if output_shapes and i < len(output_shapes) else None)
                for i, t in enumerate(self.outputs)]
        return OpShardingRule(ins, outs, sizes)


def elementwise_rule(input_shapes: Sequence[Sequence[int]], output_rank: int) -> OpShardingRule:
    """Right-aligned broadcasting rule: dim j (from the right) of every operand shares factor
    ``d<j>`` unless the operand's extent there is 1 while the output's is not."""
    out_map: Mapping = {i: [f"d{output_rank - 1 - i}"] for i in range(output_rank)}
    out_extent = [1] * output_rank
    for s in input_shapes:
        for j in range(len(s)):
            k = output_rank - len(s) + j
            if k >= 0:
                out_extent[k] = max(out_extent[k], int(s[j]))
    ins = []
    for s in input_shapes:
        m: Mapping = {}
        for j in range(len(s)):
            k = output_rank - len(s) + j
            if k < 0:
                continue
            if int(s[j]) == 1 and out_extent[k] != 1:
                m[j] = [f"bcast{len(ins)}_{j}"]   # size-1 dim: its own factor (never sharded)
            else:
                m[j] = [f"d{output_rank - 1 - k}"]
        ins.append(m)
    return OpShardingRule(ins, [out_map])


def _assign_factor_axes(rule: OpShardingRule, input_specs: Sequence[ShardingSpec | None]) -> dict[str, list[str]]:
    """Mesh axes of every factor, read off the operands' layouts: the first operand dim that shards
    a factor decides for it (a dim made of several factors gives its axes to the major one), and a
    mesh axis goes to ONE factor only. Without the second rule ``x @ x.T`` with the rows of ``x``
    split over an axis would ask for both output dims on that axis: the output can honour one, so
    the other operand has to give the axis up (it is gathered) rather than keep a layout the
    output does not describe."""
    factor_axes: dict[str, list[str]] = {}
    taken: set[str] = set()
    for t_idx, spec in enumerate(input_specs):
        if spec is None or t_idx >= len(rule.input_mappings):
            continue
        for dim_idx, factors in rule.input_mappings[t_idx].items():
            if dim_idx >= len(spec.dim_specs) or not factors:
                continue
            axes = spec.dim_specs[dim_idx].axes
            f = factors[0]
            if not axes or f in factor_axes:
                continue
            free = [a for a in axes if a not in taken]
            if free:
                factor_axes[f] = free
                taken.update(free)
    return factor_axes


def infer_from_rule(rule: OpShardingRule, input_specs: Sequence[ShardingSpec | None], mesh: DeviceMesh,
                    output_index: int = 0) -> tuple[ShardingSpec, set[str]]:
    """Output sharding and the set of mesh axes that became partial by contraction."""
    factor_axes = _assign_factor_axes(rule, input_specs)
    out_map = rule.output_mappings[output_index] if rule.output_mappings else {}
    # contraction is judged per output: a sharded input factor that this output does not carry
    # was summed away on the way to it (e.g. the row factors for LayerNorm's dgamma)
    own = {f for fs in out_map.values() for f in fs}
    in_factors = {f for m in rule.input_mappings for fs in m.values() for f in fs}
    contracting = in_factors - own
    rank = max(out_map.keys(), default=-1) + 1
    used: set[str] = set()
    dims: list[DimSpec] = []
    for d in range(rank):
        axes: list[str] = []
        for f in out_map.get(d, []):
            for a in factor_axes.get(f, []):
                if a not in used:
                    axes.append(a)
                    used.add(a)
        dims.append(DimSpec(axes))
    partial: set[str] = set()
    for f in contracting:
        for a in factor_axes.get(f, []):
            if a not in used:
                partial.add(a)
    return ShardingSpec(mesh, dims, partial_sum_axes=set(partial)), partial


def required_input_specs(rule: OpShardingRule, input_specs: Sequence[ShardingSpec | None], mesh: DeviceMesh,
                         input_ranks: Sequence[int]) -> list[ShardingSpec]:
    """Input layouts consistent with the factor assignment chosen by ``infer_from_rule``:
    every input dim takes the axes of its factor (first-wins), so operands that disagree are
    resharded to agree before the per-shard kernel runs."""
    factor_axes = _assign_factor_axes(rule, input_specs)
    out = []
    for t_idx, rank in enumerate(input_ranks):
        spec = input_specs[t_idx] if t_idx < len(input_specs) else None
        mapping = rule.input_mappings[t_idx] if t_idx < len(rule.input_mappings) else {}
        used: set[str] = set()
        dims = []
        for d in range(rank):
            fs = mapping.get(d, [])
            axes = []
            if fs and not fs[0].startswith("bcast"):
                for a in factor_axes.get(fs[0], []):
                    if a not in used:
                        axes.append(a)
                        used.add(a)
            dims.append(DimSpec(axes))
        partial = set(spec.partial_sum_axes) if spec is not None else set()
        partial -= used
        out.append(ShardingSpec(mesh, dims, partial_sum_axes=partial))
    return out


class PropagationStrategy:
    """How `propagate_sharding` settles a factor that several operands shard differently.
    BASIC: the proposal with the smallest priority number wins, ties go to the one that splits the
    factor over more devices, then to the first operand."""

    BASIC = "basic"


def propagate_sharding(rule: OpShardingRule, input_specs, output_specs, strategy=PropagationStrategy.BASIC,
                       **_kw) -> bool:
    """One bidirectional step over an op: every operand dim proposes its mesh axes for the factor it
    maps to, one proposal per factor is chosen, and every OPEN dim of every operand (inputs and
    outputs alike) takes the chosen axes of its factors. Closed dims (``is_open=False``) keep what
    they have, and an axis is never used twice inside one tensor. Returns whether anything changed;
    a solver calls this over all ops until nothing does. (The reference kept only a forward stub
    under this name, nabla/core/sharding/propagation.py:314.)"""
    operands = [(m, sp) for m, sp in zip(rule.input_mappings, input_specs) if sp is not None]
    operands += [(m, sp) for m, sp in zip(rule.output_mappings, output_specs) if sp is not None]
    if not operands:
        return False
    mesh = operands[0][1].mesh
    best: dict[str, tuple] = {}
    order = 0
    for mapping, spec in operands:
        for dim, factors in mapping.items():
            if dim >= len(spec.dim_specs) or not factors:
                continue
            ds = spec.dim_specs[dim]
            if not ds.axes:
                continue
            shards = 1
            for a in ds.axes:
                shards *= mesh.get_axis_size(a)
            # closed dims are facts, open ones are suggestions: facts first, then priority, then width
            key = (0 if not ds.is_open else 1, ds.priority, -shards, order)
            order += 1
            f = factors[0]                      # a dim made of several factors gives its axes to the major one
            if f not in best or key < best[f][0]:
                best[f] = (key, list(ds.axes), ds.priority)
    changed = False
    for mapping, spec in operands:
        used = {a for d, ds in enumerate(spec.dim_specs) if not ds.is_open or d not in mapping for a in ds.axes}
        used |= set(spec.replicated_axes) | set(spec.partial_sum_axes)
        for dim in sorted(mapping):
            if dim >= len(spec.dim_specs):
                continue
            ds = spec.dim_specs[dim]
            if not ds.is_open:
                continue
            want: list[str] = []
            prio = ds.priority
            for f in mapping[dim]:
                if f in best:
                    for a in best[f][1]:
                        if a not in used and a not in want:
                            want.append(a)
                    prio = min(prio, best[f][2]) if ds.axes else best[f][2]
            size = rule.factor_sizes.get(mapping[dim][0]) if mapping[dim] else None
            shards = 1
            for a in want:
                shards *= mesh.get_axis_size(a)
            if size is not None and shards > 1 and int(size) % shards:
                want = []                       # would not divide the dim: leave it alone
            if want and want != ds.axes and len(want) >= len(ds.axes):
                spec.dim_specs[dim] = DimSpec(want, is_open=True, priority=prio)
                changed = True
            used |= set(spec.dim_specs[dim].axes)
    return changed
