"""Sharding data model: ``DeviceMesh``, ``DimSpec``, ``ShardingSpec``, ``PartitionSpec``.

Reference: nabla/core/sharding/spec.py:17-616. Semantics kept: named mesh axes in row-major
device order, sub-axis syntax ``"x:(pre)size"``, per-dimension axis lists, explicit
``replicated_axes`` and deferred ``partial_sum_axes``, ceil-div chunking with short or empty
trailing shards.

Execution modes of a mesh (this is where the design departs from the reference):

* **distributed** - ``torch.distributed`` is initialised with exactly one rank per mesh
  position (one process per GPU). Each process holds only its own shard; collectives run
  over NCCL / peer-memory kernels on the sub-groups of the mesh axes.
* **simulated** - anything else (the reference's "simulation mode",
  nabla/core/sharding/spec.py:128-142): the single process holds every shard on one device
  and collectives are list computations. All CPU tests run this way.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Any, Iterable, Sequence

import torch

from ...types import CPU, Accelerator, Device

_SUB = re.compile(r"^(\w+):\((\d+)\)(\d+)$")


def parse_sub_axis(axis_name: str) -> tuple[str, int, int] | None:
    """``'x:(2)4'`` -> ``('x', 2, 4)``: the size-4 factor of ``x`` that sits after a size-2
    major factor. ``None`` for a plain axis name."""
    if ":" not in axis_name:
        return None
    m = _SUB.match(axis_name)
    if not m:
        raise ValueError(f"Invalid sub-axis format: {axis_name}")
    return m.group(1), int(m.group(2)), int(m.group(3))


def check_sub_axes_maximality(axes: Iterable[str]) -> list[str]:
    """Warnings for sub-axes of one parent that sit next to each other and could be written as one
    (``'x:(1)2'`` and ``'x:(2)2'`` are ``'x:(1)4'``). Reference: nabla/core/sharding/spec.py:53-79."""
    by_parent: dict[str, list[tuple[int, int, str]]] = {}
    for ax in axes:
        p = parse_sub_axis(ax)
        if p is not None:
            by_parent.setdefault(p[0], []).append((p[1], p[2], ax))
    out = []
    for parent, subs in by_parent.items():
        subs.sort()
        for (pre1, size1, ax1), (pre2, size2, ax2) in zip(subs, subs[1:]):
            if pre1 * size1 == pre2:
                out.append(f"Adjacent sub-axes '{ax1}' and '{ax2}' could be merged into '{parent}:({pre1}){size1 * size2}'")
    return out


def validate_sub_axes_non_overlapping(axes: Iterable[str]) -> None:
    seen: dict[str, list[tuple[int, int, str]]] = {}
    for ax in axes:
        p = parse_sub_axis(ax)
        if p is None:
            continue
        parent, pre, size = p
        lo, hi = pre, pre * size
        for lo2, hi2, other in seen.get(parent, []):
            if not (hi <= lo2 or lo >= hi2):
                raise ValueError(f"Sub-axes overlap: '{ax}' and '{other}'")
        seen.setdefault(parent, []).append((lo, hi, ax))


class DeviceMesh:
    """A named N-dimensional grid of devices."""

    def __init__(self, name: str, shape: Sequence[int], axis_names: Sequence[str], devices: Sequence[int] | None = None,
                 device_refs: Sequence[Device] | None = None, bandwidth: float = 1.0):
        self.name = name
        self.shape = tuple(int(s) for s in shape)
        self.axis_names = tuple(axis_names)
        if len(self.shape) != len(self.axis_names):
            raise ValueError("shape and axis_names must have the same length")
        if len(set(self.axis_names)) != len(self.axis_names):
            raise ValueError("axis names must be unique")
        n = math.prod(self.shape)
        self.devices = list(devices) if devices is not None else list(range(n))
        if len(self.devices) != n:
            raise ValueError(f"mesh of shape {self.shape} needs {n} devices, got {len(self.devices)}")
        self.bandwidth = float(bandwidth)
        self.strides = tuple(math.prod(self.shape[i + 1:]) for i in range(len(self.shape)))
        self.phys_strides = list(self.strides)                                   # the reference's name
        self.axis_lookup = {a: i for i, a in enumerate(self.axis_names)}
        self._groups: dict[tuple[str, ...], Any] = {}
        # ---- execution mode
        self.rank: int | None = None
        dist = torch.distributed
        if device_refs is None and dist.is_available() and dist.is_initialized() and dist.get_world_size() == n and n > 1:
            self.rank = dist.get_rank()
            if torch.cuda.is_available() and dist.get_backend() != "gloo":
                me: Device = Accelerator(torch.cuda.current_device())
            else:
                me = CPU()
            self.device_refs = [me] * n
        elif device_refs is not None:
            self.device_refs = list(device_refs)
        else:
            from ..common.context import get_default_device

            self.device_refs = [get_default_device()] * n

    # ---- modes
    @property
    def is_distributed(self) -> bool:
        """True when every mesh position is a separate process/GPU."""
        return self.rank is not None

    @property
    def local_ids(self) -> list[int]:
        """Mesh positions whose shards this process holds."""
        return [self.rank] if self.rank is not None else list(range(len(self.devices)))

    @property
    def num_local(self) -> int:
        return 1 if self.rank is not None else len(self.devices)

    @property
    def size(self) -> int:
        return len(self.devices)

    # ---- geometry
    def _axis_geometry(self, axis_name: str) -> tuple[int, int]:
        """(size, stride) of an axis or sub-axis in flat device-index space."""
        p = parse_sub_axis(axis_name)
        if p is None:
            i = self.axis_names.index(axis_name)
            return self.shape[i], self.strides[i]
        parent, pre, size = p
        i = self.axis_names.index(parent)
        total = self.shape[i]
        if total % (pre * size) != 0:
            raise ValueError(f"sub-axis {axis_name} does not divide axis of size {total}")
        post = total // (pre * size)
        return size, self.strides[i] * post

    def get_axis_size(self, axis_name: str) -> int:
        return self._axis_geometry(axis_name)[0]

    def get_coordinate(self, device_id: int, axis_name: str) -> int:
        size, stride = self._axis_geometry(axis_name)
        return (device_id // stride) % size

    def get_axis_indices(self, device_id) -> dict[str, int] | list[int]:
        """Coordinates of a device along every mesh axis, ``{axis name: coordinate}`` (reference:
        nabla/core/sharding/spec.py:256-258). Given an axis NAME instead, the coordinates that exist on
        that axis."""
        if isinstance(device_id, str):
            return list(range(self.get_axis_size(device_id)))
        return {name: self.get_coordinate(int(device_id), name) for name in self.axis_names}

    def has_axis(self, axis_name: str) -> bool:
        p = parse_sub_axis(axis_name)
        return (p[0] if p else axis_name) in self.axis_names

    def group_of(self, device_id: int, axes: Iterable[str]) -> list[int]:
        """Device ids that differ from ``device_id`` only in the coordinates of ``axes``,
        ordered by those coordinates (first axis most significant)."""
        axes = list(axes)
        geo = [self._axis_geometry(a) for a in axes]
        base = device_id
        for (size, stride) in geo:
            base -= ((device_id // stride) % size) * stride
        ids = [base]
        for (size, stride) in geo:
            ids = [i + c * stride for i in ids for c in range(size)]
        return ids

    def groups(self, axes: Iterable[str]) -> list[list[int]]:
        """Partition of all devices into groups along ``axes``."""
        axes = list(axes)
        seen: set[int] = set()
        out = []
        for d in range(len(self.devices)):
            if d in seen:
                continue
            g = self.group_of(d, axes)
            seen.update(g)
            out.append(g)
        return out

    def get_devices_on_axis_slice(self, axis_name: str, coordinate: int) -> list[int]:
        """Device ids whose coordinate along ``axis_name`` is ``coordinate``."""
        return [d for d in range(len(self.devices)) if self.get_coordinate(d, axis_name) == coordinate]

    def get_signal_buffers(self, buffer_size: int = 65536, use_cache: bool = False) -> list:
        """Flag memory that the collectives of this mesh synchronise through, one entry per locally
        held device (reference: nabla/core/sharding/spec.py:152, MAX signal buffers). Here the flags
        are the first 64 KB of the symmetric workspace of the whole-mesh group
        (`parallel/symm.py`); a simulated mesh, or a process without a GPU, has none."""
        if not self.is_distributed:
            return []
        try:
            from ...parallel import symm

            if not symm.is_ready():
                return []
            ws = symm.workspace(self, tuple(self.axis_names))
            return [ws.buf[: min(int(buffer_size), ws.flag_bytes)]]
        except Exception:
            return []

    def process_group(self, axes: Iterable[str]):
        """torch.distributed group of this rank along ``axes`` (distributed mode only)."""
        key = tuple(sorted(axes, key=lambda a: self.axis_names.index(parse_sub_axis(a)[0] if parse_sub_axis(a) else a)))
        if key not in self._groups:
            dist = torch.distributed
            mine = None
            for g in self.groups(key):   # every rank must create every group, in the same order
                pg = dist.new_group(ranks=g)
                if self.rank in g:
                    mine = (pg, g)
            self._groups[key] = mine
        return self._groups[key]

    def __repr__(self) -> str:
        ax = ", ".join(f"{n}={s}" for n, s in zip(self.axis_names, self.shape))
        return f"DeviceMesh('{self.name}', {ax})"

    def __eq__(self, o: Any) -> bool:
        return (isinstance(o, DeviceMesh) and o.name == self.name and o.shape == self.shape
                and o.axis_names == self.axis_names and o.devices == self.devices)

    def __hash__(self) -> int:
        return hash((self.name, self.shape, self.axis_names, tuple(self.devices)))


@dataclass
class DimSpec:
    """Mesh axes a tensor dimension is split over (major to minor)."""

    axes: list[str] = field(default_factory=list)
    is_open: bool = False
    priority: int = 0

    def __post_init__(self):
        self.axes = list(self.axes)

    @staticmethod
    def from_raw(raw: Any) -> "DimSpec":
        if isinstance(raw, DimSpec):
            return raw
        if raw is None:
            return DimSpec([])
        if isinstance(raw, str):
            return DimSpec([raw])
        if isinstance(raw, (tuple, list)):
            return DimSpec([str(a) for a in raw])
        raise TypeError(f"cannot build DimSpec from {raw!r}")

    def is_replicated(self) -> bool:
        return not self.axes

    def get_total_shards(self, mesh: DeviceMesh) -> int:
        return math.prod(mesh.get_axis_size(a) for a in self.axes) if self.axes else 1

    def clone(self) -> "DimSpec":
        return DimSpec(list(self.axes), self.is_open, self.priority)

    def __repr__(self) -> str:
        if not self.axes:
            return "{?}" if self.is_open else "{}"
        body = ", ".join(f"'{a}'" for a in self.axes)
        return "{" + body + (", ?" if self.is_open else "") + "}" + (f"p{self.priority}" if self.priority else "")

    __str__ = __repr__


@dataclass
class ShardingSpec:
    """Layout of a tensor on a mesh plus its pending cross-device reductions."""

    mesh: DeviceMesh
    dim_specs: list[DimSpec] = field(default_factory=list)
    replicated_axes: set[str] = field(default_factory=set)
    partial_sum_axes: set[str] = field(default_factory=set)

    def __post_init__(self) -> None:
        self.dim_specs = [DimSpec.from_raw(d) for d in self.dim_specs]
        self.replicated_axes = set(self.replicated_axes)
        self.partial_sum_axes = set(self.partial_sum_axes)
        used: set[str] = set()
        for i, d in enumerate(self.dim_specs):
            for a in d.axes:
                if not self.mesh.has_axis(a):
                    raise ValueError(f"Axis '{a}' is not an axis of mesh {self.mesh!r}")
                if a in self.replicated_axes:
                    raise ValueError(f"Axis '{a}' is explicitly replicated but assigned to dimension {i}.")
                if a in used:
                    raise ValueError(f"Axis '{a}' used multiple times in sharding.")
                used.add(a)
        for a in self.partial_sum_axes:
            if a in used:
                raise ValueError(f"Axis '{a}' is both a dimension axis and a partial sum axis.")
            if a in self.replicated_axes:
                raise ValueError(f"Axis '{a}' is both explicitly replicated and a partial sum axis.")
            used.add(a)
        validate_sub_axes_non_overlapping(used)

    # ---- queries
    def ordered_axes(self, axes_set: Iterable[str]) -> list[str]:
        """Axes in mesh order; sub-axes after their parent position, by ``pre`` size."""
        def key(a):
            p = parse_sub_axis(a)
            parent = p[0] if p else a
            idx = self.mesh.axis_names.index(parent) if parent in self.mesh.axis_names else 10 ** 6
            return (idx, 0 if p is None else 1, p[1] if p else 0)
        return sorted(axes_set, key=key)

    def all_partial_axes(self) -> set[str]:
        return set(self.partial_sum_axes)

    def used_axes(self) -> set[str]:
        u = set()
        for d in self.dim_specs:
            u.update(d.axes)
        return u

    def effect_signature(self) -> tuple:
        """Hashable identity including deferred-reduction metadata (for caches)."""
        return ((self.mesh.name, self.mesh.shape, self.mesh.axis_names),
                tuple((tuple(d.axes), bool(d.is_open), int(d.priority)) for d in self.dim_specs),
                tuple(self.ordered_axes(self.replicated_axes)), tuple(self.ordered_axes(self.partial_sum_axes)))

    def get_implicitly_replicated_axes(self) -> set[str]:
        used = self.used_axes() | self.replicated_axes | self.partial_sum_axes
        parents = {parse_sub_axis(a)[0] if parse_sub_axis(a) else a for a in used}
        return {a for a in self.mesh.axis_names if a not in parents}

    def is_fully_replicated(self) -> bool:
        return all(not d.axes for d in self.dim_specs) and not self.partial_sum_axes

    @property
    def total_shards(self) -> int:
        return math.prod(d.get_total_shards(self.mesh) for d in self.dim_specs)

    def get_max_priority(self) -> int:
        """Largest (least urgent) propagation priority among the dimensions."""
        return max((d.priority for d in self.dim_specs), default=0)

    def get_min_priority(self) -> int:
        """Smallest (most urgent) propagation priority among the dimensions."""
        return min((d.priority for d in self.dim_specs), default=0)

    def clone(self, **changes) -> "ShardingSpec":
        return ShardingSpec(changes.get("mesh", self.mesh),
                            changes.get("dim_specs", [d.clone() for d in self.dim_specs]),
                            set(changes.get("replicated_axes", self.replicated_axes)),
                            set(changes.get("partial_sum_axes", self.partial_sum_axes)))

    def without_partial(self) -> "ShardingSpec":
        return self.clone(partial_sum_axes=set())

    def __repr__(self) -> str:
        dims = ", ".join(str(d) for d in self.dim_specs)
        rep = ""
        if self.replicated_axes:
            rep = ", replicated={" + ", ".join(f"'{a}'" for a in self.ordered_axes(self.replicated_axes)) + "}"
        par = ""
        if self.partial_sum_axes:
            par = ", partial={" + ", ".join(f"'{a}'" for a in self.ordered_axes(self.partial_sum_axes)) + "}"
        return f"sharding<@{self.mesh.name}, [{dims}]{rep}{par}>"

    def __eq__(self, o: Any) -> bool:
        return isinstance(o, ShardingSpec) and self.effect_signature() == o.effect_signature()

    def __hash__(self) -> int:
        return hash(self.effect_signature())


def shard_index(spec: ShardingSpec, dim: int, device_id: int) -> tuple[int, int]:
    """(index of this device's chunk, number of chunks) along tensor dimension ``dim``."""
    idx, total = 0, 1
    for a in spec.dim_specs[dim].axes:
        size = spec.mesh.get_axis_size(a)
        idx = idx * size + spec.mesh.get_coordinate(device_id, a)
        total *= size
    return idx, total


def shard_salt(spec: "ShardingSpec | None", device_id: int) -> int:
    """Linear index of this device's shard over the SHARDED dimensions only: copies of a replicated
    (or partially replicated) tensor get the same value on every device that holds the same piece,
    so random ops draw identical numbers for identical pieces and replicas do not diverge."""
    if spec is None:
        return 0
    idx = 0
    for d in range(len(spec.dim_specs)):
        i, total = shard_index(spec, d, device_id)
        idx = idx * total + i
    return idx


def local_slice(global_len: int, idx: int, total: int) -> tuple[int, int]:
    """Ceil-div chunk ``idx`` of ``total``: (start, length); trailing chunks may be short/empty."""
    chunk = math.ceil(global_len / total) if total else global_len
    start = min(idx * chunk, global_len)
    return start, max(0, min(start + chunk, global_len) - start)


def compute_local_shape(global_shape: Sequence[int], sharding: ShardingSpec, device_id: int) -> tuple[int, ...]:
    if len(global_shape) != len(sharding.dim_specs):
        raise ValueError(f"Rank mismatch: global_shape has rank {len(global_shape)}, "
                         f"but sharding spec has {len(sharding.dim_specs)} dim specs.")
    out = []
    for i, g in enumerate(global_shape):
        if not sharding.dim_specs[i].axes:
            out.append(int(g))
        else:
            idx, total = shard_index(sharding, i, device_id)
            out.append(local_slice(int(g), idx, total)[1])
    return tuple(out)


def compute_local_slices(global_shape: Sequence[int], sharding: ShardingSpec, device_id: int) -> tuple[slice, ...]:
    sl = []
    for i, g in enumerate(global_shape):
        if not sharding.dim_specs[i].axes:
            sl.append(slice(0, int(g)))
        else:
            idx, total = shard_index(sharding, i, device_id)
            st, ln = local_slice(int(g), idx, total)
            sl.append(slice(st, st + ln))
    return tuple(sl)


def compute_global_shape(local_shape: Sequence[int], sharding: ShardingSpec | None,
                         shard_shapes: Sequence[Sequence[int]] | None = None) -> tuple[int, ...]:
    """Global shape from local shape(s). With all shard shapes given the sharded dims are
    summed (exact for uneven shards); otherwise local * number of chunks."""
    if sharding is None or not len(local_shape):
        return tuple(int(d) for d in local_shape)
    res = []
    for i, d in enumerate(local_shape):
        ds = sharding.dim_specs[i] if i < len(sharding.dim_specs) else None
        if ds is None or not ds.axes:
            res.append(int(d))
        elif shard_shapes is not None and len(shard_shapes) == sharding.mesh.size:
            total = ds.get_total_shards(sharding.mesh)
            rep = max(1, len(shard_shapes) // total)
            res.append(sum(int(s[i]) for s in shard_shapes) // rep)
        else:
            res.append(int(d) * ds.get_total_shards(sharding.mesh))
    return tuple(res)


def get_num_shards(sharding: ShardingSpec) -> int:
    return len(sharding.mesh.devices)


def needs_reshard(from_spec: ShardingSpec | None, to_spec: ShardingSpec | None) -> bool:
    if (from_spec is None) != (to_spec is None):
        return True
    if from_spec is None:
        return False
    if len(from_spec.dim_specs) != len(to_spec.dim_specs):
        return True
    return (any(f.axes != t.axes for f, t in zip(from_spec.dim_specs, to_spec.dim_specs))
            or from_spec.partial_sum_axes != to_spec.partial_sum_axes)


class PartitionSpec(tuple):
    """JAX-style partition spec: ``P('dp', None)``."""

    def __new__(cls, *args):
        return super().__new__(cls, args)

    def __repr__(self):
        return "P(" + ", ".join(repr(a) for a in self) + ")"


P = PartitionSpec
