"""Build the native libraries of nabla_b200 for sm_100a with nvcc.

Each `.cu` / `.cpp` translation unit listed in ``TARGETS`` becomes one shared library in
``nabla_b200/lib``. The libraries export plain C symbols and are loaded with ctypes
(`nabla_b200.native`), so there is no dependency on the torch C++ headers and a full rebuild
takes seconds. nvcc cross-compiles without a GPU present.

``build_all(debug=True)`` (``python -m nabla_b200.csrc.build --debug``) compiles the same sources
with ``-DNB_DEBUG_CHECKS`` into ``nabla_b200/lib/debug``: every data- or geometry-derived global,
peer and TMA coordinate is checked before use (``nb_debug.cuh``); ``NABLA_B200_DEBUG_KERNELS=1``
makes ``nabla_b200.native`` load that build.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB = CSRC.parent / "lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]

# library name -> (sources, extra flags)
TARGETS: dict[str, tuple[list[str], list[str]]] = {
    "libnb_gemm.so": (["gemm_tcgen05.cu"], []),
    "libnb_kernels.so": (["fused_kernels.cu", "elementwise_kernels.cu"], []),
    "libnb_attention.so": (["attention_tcgen05.cu"], []),
    "libnb_comm.so": (["peer_collectives.cu"], []),
    "libnb_runtime.so": (["plan_runtime.cpp"], []),
    "libnb_noalloc.so": (["no_alloc_entry.cu"], []),
}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def build_all(force: bool = False, verbose: bool = False, debug: bool = False) -> list[Path]:
    """Compile every target whose sources changed. Returns the list of built libraries.
    ``debug=True`` builds the bounds-checked variant into ``lib/debug``."""
    lib_dir = LIB / "debug" if debug else LIB
    lib_dir.mkdir(parents=True, exist_ok=True)
    built = []
    for name, (srcs, extra) in TARGETS.items():
        paths = [CSRC / s for s in srcs]
        if not all(p.exists() for p in paths):
            continue
        out = lib_dir / name
        stamp = lib_dir / (name + ".sha")
        is_cuda = any(p.suffix == ".cu" for p in paths)
        flags = (NVCC_FLAGS if is_cuda else ["-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC"]) + extra
        if debug:
            flags = flags + ["-DNB_DEBUG_CHECKS"]
        dig = _digest(paths, flags)
        if not force and out.exists() and stamp.exists() and stamp.read_text() == dig:
            built.append(out)
            continue
        cmd = [_nvcc(), *flags, "-o", str(out), *map(str, paths)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
        stamp.write_text(dig)
        built.append(out)
    return built


if __name__ == "__main__":
    libs = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv, debug="--debug" in sys.argv)
    for lib in libs:
        print(lib)
