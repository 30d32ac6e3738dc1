"""User-visible value types: ``DType``, ``Dim``/``Shape`` and ``Device``.

The reference re-exports these from the MAX runtime (``max.dtype.DType``, ``max.graph.Shape``
/ ``Dim`` / ``StaticDim`` / ``SymbolicDim``, ``max.driver.CPU`` / ``Accelerator``;
nabla/__init__.py:21-22, nabla/core/tensor/api.py:639-647). Here they are small standalone
classes over torch so that notebooks print the same things (``[Dim(2), Dim(3)]``,
``DType.float32``, ``Device(type=cpu,id=0)``) and ``int(d)`` works.
"""
from __future__ import annotations

import enum
from typing import Iterable

import numpy as np
import torch


class DType(enum.Enum):
    bool = "bool"
    int8 = "si8"
    int16 = "si16"
    int32 = "si32"
    int64 = "si64"
    uint8 = "ui8"
    uint16 = "ui16"
    uint32 = "ui32"
    uint64 = "ui64"
    float16 = "f16"
    bfloat16 = "bf16"
    float32 = "f32"
    float64 = "f64"
    complex64 = "c64"
    complex128 = "c128"

    def __repr__(self) -> str:
        return f"DType.{self.name}"

    __str__ = __repr__

    # ---- conversions
    def to_torch(self) -> torch.dtype:
        return _TO_TORCH[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DType":
        return _FROM_TORCH[dt]

    def to_numpy(self) -> np.dtype:
        if self is DType.bfloat16:
            raise TypeError("numpy has no bfloat16; cast to float32 first")
        return np.dtype(_TO_NUMPY[self])

    @staticmethod
    def from_numpy(dt) -> "DType":
        return _FROM_NUMPY[np.dtype(dt).name]

    # ---- queries
    def is_float(self) -> bool:
        return self in (DType.float16, DType.bfloat16, DType.float32, DType.float64)

    def is_integral(self) -> bool:
        return self.name.startswith(("int", "uint"))

    def is_signed(self) -> bool:
        return self.is_float() or self.name.startswith("int")

    @property
    def size_in_bytes(self) -> int:
        return torch.empty((), dtype=self.to_torch()).element_size()

    @property
    def short(self) -> str:
        """Short name used in tensor headers: f32, bf16, i64, bool."""
        v = self.value
        if v.startswith("si"):
            return "i" + v[2:]
        if v.startswith("ui"):
            return "u" + v[2:]
        return v


_TO_TORCH = {
    DType.bool: torch.bool, DType.int8: torch.int8, DType.int16: torch.int16, DType.int32: torch.int32,
    DType.int64: torch.int64, DType.uint8: torch.uint8, DType.uint16: torch.uint16, DType.uint32: torch.uint32,
    DType.uint64: torch.uint64, DType.float16: torch.float16, DType.bfloat16: torch.bfloat16,
    DType.float32: torch.float32, DType.float64: torch.float64, DType.complex64: torch.complex64,
    DType.complex128: torch.complex128,
}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}
_TO_NUMPY = {
    DType.bool: "bool", DType.int8: "int8", DType.int16: "int16", DType.int32: "int32", DType.int64: "int64",
    DType.uint8: "uint8", DType.uint16: "uint16", DType.uint32: "uint32", DType.uint64: "uint64",
    DType.float16: "float16", DType.float32: "float32", DType.float64: "float64", DType.complex64: "complex64",
    DType.complex128: "complex128",
}
_FROM_NUMPY = {v: k for k, v in _TO_NUMPY.items()}


def as_dtype(x) -> DType:
    """Normalise a DType / torch dtype / numpy dtype / string to ``DType``."""
    if isinstance(x, DType):
        return x
    if isinstance(x, torch.dtype):
        return DType.from_torch(x)
    if isinstance(x, str):
        if x in DType.__members__:
            return DType[x]
        for d in DType:
            if d.value == x or d.short == x:
                return d
    if x is float:
        return DType.float32
    if x is int:
        return DType.int64
    if x is bool:
        return DType.bool
    return DType.from_numpy(x)


# ---------------------------------------------------------------- dims and shapes
class Dim:
    """A dimension: static (an int) or symbolic (a name). ``int(d)`` works on static dims."""

    __slots__ = ()

    def __new__(cls, value=None):
        if cls is Dim:
            if isinstance(value, Dim):
                return value
            if isinstance(value, str):
                return SymbolicDim(value)
            return StaticDim(int(value))
        return object.__new__(cls)


class StaticDim(Dim):
    __slots__ = ("dim",)

    def __init__(self, value):
        self.dim = int(value.dim if isinstance(value, StaticDim) else value)

    def __int__(self):
        return self.dim

    __index__ = __int__

    def __repr__(self):
        return f"Dim({self.dim})"

    def __hash__(self):
        return hash(self.dim)

    def __eq__(self, o):
        return self.dim == (o.dim if isinstance(o, StaticDim) else o)

    def _b(self, o, f):
        if isinstance(o, StaticDim):
            o = o.dim
        if isinstance(o, (int, float)):
            return f(self.dim, o)
        return NotImplemented

    def __add__(self, o): return self._b(o, lambda a, b: a + b)
    def __radd__(self, o): return self._b(o, lambda a, b: b + a)
    def __sub__(self, o): return self._b(o, lambda a, b: a - b)
    def __rsub__(self, o): return self._b(o, lambda a, b: b - a)
    def __mul__(self, o): return self._b(o, lambda a, b: a * b)
    def __rmul__(self, o): return self._b(o, lambda a, b: b * a)
    def __floordiv__(self, o): return self._b(o, lambda a, b: a // b)
    def __rfloordiv__(self, o): return self._b(o, lambda a, b: b // a)
    def __truediv__(self, o): return self._b(o, lambda a, b: a / b)
    def __rtruediv__(self, o): return self._b(o, lambda a, b: b / a)
    def __mod__(self, o): return self._b(o, lambda a, b: a % b)
    def __lt__(self, o): return self._b(o, lambda a, b: a < b)
    def __le__(self, o): return self._b(o, lambda a, b: a <= b)
    def __gt__(self, o): return self._b(o, lambda a, b: a > b)
    def __ge__(self, o): return self._b(o, lambda a, b: a >= b)
    def __neg__(self): return -self.dim
    def __float__(self): return float(self.dim)
    def __bool__(self): return self.dim != 0


class SymbolicDim(Dim):
    __slots__ = ("name",)

    def __init__(self, name):
        self.name = str(name.name if isinstance(name, SymbolicDim) else name)

    def __int__(self):
        raise TypeError(f"symbolic dimension '{self.name}' has no static value")

    def __repr__(self):
        return f"Dim('{self.name}')"

    def __hash__(self):
        return hash(self.name)

    def __eq__(self, o):
        return isinstance(o, SymbolicDim) and o.name == self.name


class Shape(list):
    """A list of ``Dim``. Prints as ``[Dim(2), Dim(3)]``; compares equal to int tuples/lists."""

    def __init__(self, dims: Iterable = ()):
        super().__init__(Dim(d) for d in dims)

    @property
    def rank(self) -> int:
        return len(self)

    @property
    def static_dims(self) -> list[int]:
        return [int(d) for d in self]

    def __eq__(self, other):
        try:
            return len(self) == len(other) and all(a == b for a, b in zip(self, other))
        except TypeError:
            return False

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash(tuple(self))

    def __getitem__(self, i):
        r = super().__getitem__(i)
        return Shape(r) if isinstance(i, slice) else r

    def __add__(self, other):
        return Shape(list(self) + list(other))

    def __radd__(self, other):
        return Shape(list(other) + list(self))


# ---------------------------------------------------------------- devices
class Device:
    """A compute device. ``label`` is ``cpu`` or ``gpu``."""

    __slots__ = ("label", "id")

    def __init__(self, label: str = "cpu", id: int = 0):
        self.label = label
        self.id = int(id)

    @property
    def is_host(self) -> bool:
        return self.label == "cpu"

    @property
    def api(self) -> str:
        return "cpu" if self.is_host else "cuda"

    def to_torch(self) -> torch.device:
        return torch.device("cpu") if self.is_host else torch.device("cuda", self.id)

    @staticmethod
    def from_torch(d) -> "Device":
        d = torch.device(d)
        if d.type == "cuda":
            return Accelerator(d.index or 0)
        return CPU()

    def __repr__(self):
        return f"Device(type={self.label},id={self.id})"

    def __eq__(self, o):
        return isinstance(o, Device) and o.label == self.label and o.id == self.id

    def __hash__(self):
        return hash((self.label, self.id))


class CPU(Device):
    __slots__ = ()

    def __init__(self, id: int = 0):
        super().__init__("cpu", id)


class Accelerator(Device):
    __slots__ = ()

    def __init__(self, id: int = 0):
        super().__init__("gpu", id)


def accelerator_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def as_device(d) -> Device:
    if d is None:
        from .core.common.context import get_default_device

        return get_default_device()
    if isinstance(d, Device):
        return d
    if isinstance(d, str) and d in ("gpu", "accelerator"):
        return Accelerator(0)
    if isinstance(d, int) and not isinstance(d, bool):
        # a device id taken from a mesh (`mesh.devices[i]`): that GPU when this process has it, else
        # the host, where a mesh larger than the machine is simulated
        return Accelerator(d) if torch.cuda.is_available() and d < torch.cuda.device_count() else CPU()
    return Device.from_torch(d)
