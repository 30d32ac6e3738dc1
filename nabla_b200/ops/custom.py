"""Custom-kernel registry (reference: nabla/ops/utils.py:765-824, tests/mojo/op.py:15-32).

``call_custom_kernel(name, path, values, out_types)`` runs a user kernel inside an op's
``kernel()``. Kernels come from (a) ``register_kernel(name, fn)`` - a Python callable on torch
tensors (handy on CPU), or (b) a ``.cu`` file / directory / ``.so`` exporting the C ABI of
``csrc/include/nabla_custom_kernel.h``; sources are compiled once with nvcc for sm_100a and
cached next to the source.
"""
from __future__ import annotations

import ctypes
import hashlib
import subprocess
from pathlib import Path
from typing import Any, Callable, Sequence

import torch

_PY_KERNELS: dict[str, Callable] = {}
_LIBS: dict[str, ctypes.CDLL] = {}
launch_count = 0

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float64: 3, torch.int32: 4, torch.int64: 5,
       torch.uint8: 6, torch.bool: 7}


class NbTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("numel", ctypes.c_int64), ("rank", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("shape", ctypes.c_int64 * 8)]


def register_kernel(name: str, fn: Callable | None = None):
    """Register a Python implementation ``fn(*inputs) -> tensor | tuple`` (decorator-friendly)."""
    if fn is None:
        return lambda f: register_kernel(name, f)
    _PY_KERNELS[name] = fn
    return fn


def registered_kernels() -> list[str]:
    return sorted(_PY_KERNELS)


def _include_dir() -> Path:
    return Path(__file__).resolve().parent.parent / "csrc" / "include"


def _build(src_files: list[Path]) -> Path:
    h = hashlib.sha256()
    for f in src_files:
        h.update(f.read_bytes())
    out_dir = src_files[0].parent / "_nabla_build"
    out_dir.mkdir(exist_ok=True)
    out = out_dir / f"custom_{h.hexdigest()[:16]}.so"
    if not out.exists():
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
               "-Xcompiler", "-fPIC", "-I", str(_include_dir()), "-o", str(out), *map(str, src_files)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for custom kernels {src_files}:\n{res.stderr}")
    return out


def load_kernel_library(path) -> ctypes.CDLL:
    paths = path if isinstance(path, (list, tuple)) else [path]
    key = "|".join(str(Path(p).resolve()) for p in paths)
    lib = _LIBS.get(key)
    if lib is not None:
        return lib
    srcs: list[Path] = []
    so: Path | None = None
    for p in paths:
        p = Path(p).resolve()
        if p.is_dir():
            srcs += sorted(p.glob("*.cu"))
            if not srcs:
                sos = sorted(p.glob("*.so"))
                so = sos[0] if sos else None
        elif p.suffix == ".cu":
            srcs.append(p)
        elif p.suffix == ".so":
            so = p
        else:
            raise ValueError(f"unsupported custom kernel path: {p}")
    if srcs:
        so = _build(srcs)
    if so is None:
        raise FileNotFoundError(f"no .cu or .so kernels under {paths}")
    lib = ctypes.CDLL(str(so))
    _LIBS[key] = lib
    return lib


def _describe(t: torch.Tensor) -> NbTensor:
    nt = NbTensor()
    nt.data = t.data_ptr()
    nt.numel = t.numel()
    nt.rank = t.dim()
    nt.dtype = _DT[t.dtype]
    for i, d in enumerate(t.shape[:8]):
        nt.shape[i] = d
    return nt


def _out_spec(o) -> tuple[tuple[int, ...], torch.dtype]:
    if callable(o) and isinstance(getattr(o, "__self__", None), torch.Tensor):
        o = o.__self__              # `x.type` of an input, the reference's way to say "like x"
    if isinstance(o, torch.Tensor):
        return tuple(o.shape), o.dtype
    shape, dt = o
    from ..types import DType

    if isinstance(dt, DType):
        dt = dt.to_torch()
    return tuple(int(d) for d in shape), dt


def call_custom_kernel(func_name: str, kernel_path: Any, values, out_types, device=None, **kwargs):
    global launch_count
    single_in = isinstance(values, torch.Tensor)
    ins = [values] if single_in else list(values)
    single_out = not isinstance(out_types, list)
    outs_spec = [_out_spec(o) for o in ([out_types] if single_out else out_types)]
    dev = ins[0].device if ins else torch.device("cpu")
    if dev.type == "meta":
        res = [torch.empty(s, dtype=d, device="meta") for s, d in outs_spec]
        return res[0] if single_out else res
    py = _PY_KERNELS.get(func_name)
    if py is not None and kernel_path is None:
        r = py(*ins, **kwargs)
        res = [r] if isinstance(r, torch.Tensor) else list(r)
        return res[0] if single_out else res
    if kernel_path is None:
        raise KeyError(f"custom kernel '{func_name}' is not registered and no kernel_path was given")
    if dev.type != "cuda" and py is not None:
        r = py(*ins, **kwargs)
        res = [r] if isinstance(r, torch.Tensor) else list(r)
        return res[0] if single_out else res
    lib = load_kernel_library(kernel_path)
    try:
        fn = getattr(lib, func_name)
    except AttributeError as e:
        raise KeyError(f"kernel '{func_name}' not found in {kernel_path}") from e
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(NbTensor), ctypes.c_int, ctypes.POINTER(NbTensor), ctypes.c_int, ctypes.c_void_p]
    ins_c = [t.contiguous() for t in ins]
    outs = [torch.empty(s, dtype=d, device=dev) for s, d in outs_spec]
    a_in = (NbTensor * len(ins_c))(*[_describe(t) for t in ins_c])
    a_out = (NbTensor * len(outs))(*[_describe(t) for t in outs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream) if dev.type == "cuda" else ctypes.c_void_p(0)
    rc = fn(a_in, len(ins_c), a_out, len(outs), stream)
    if rc != 0:
        raise RuntimeError(f"custom kernel '{func_name}' returned {rc}")
    launch_count += 1
    return outs[0] if single_out else outs
