"""ctypes bindings to the hand-written sm_100a libraries in ``nabla_b200/lib``.

The libraries export plain C symbols (see ``nabla_b200/csrc``). Tensors stay torch tensors;
the wrappers pass raw device pointers and the current CUDA stream. On a machine with a GPU a
missing library is an error (no silent fallback): ``require()`` raises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

# NABLA_B200_DEBUG_KERNELS=1 loads the build with device-side index checks (`csrc/nb_debug.cuh`,
# `python -m nabla_b200.csrc.build --debug`) from lib/debug instead of the release build.
DEBUG_KERNELS = os.environ.get("NABLA_B200_DEBUG_KERNELS", "0") == "1"
_LIB_DIR = Path(__file__).resolve().parent.parent / "lib" / ("debug" if DEBUG_KERNELS else "")
_libs: dict[str, ctypes.CDLL] = {}
_status: dict[int, torch.Tensor] = {}
_debug_rec: dict[int, torch.Tensor] = {}
# translation units of each library (each has its own nb_debug_bind_<tu> / nb_debug_enabled_<tu>)
_DEBUG_UNITS = {"libnb_gemm.so": ("gemm",), "libnb_kernels.so": ("fused", "elementwise"),
                "libnb_attention.so": ("attention",), "libnb_comm.so": ("comm",)}


class NativeLibraryMissing(RuntimeError):
    pass


def lib_path(name: str) -> Path:
    return _LIB_DIR / name


def available(name: str) -> bool:
    return lib_path(name).exists()


def load(name: str) -> ctypes.CDLL:
    """Load (once) and return the named shared library; build it first if it is absent."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    p = lib_path(name)
    if not p.exists():
        try:
            from ..csrc.build import build_all

            build_all(debug=DEBUG_KERNELS)
        except Exception as e:  # pragma: no cover - build environment problems
            raise NativeLibraryMissing(f"{name} is not built and building failed: {e}") from e
    if not p.exists():
        raise NativeLibraryMissing(f"{p} not found; run `python -m nabla_b200.csrc.build`")
    lib = ctypes.CDLL(str(p))
    _libs[name] = lib
    if DEBUG_KERNELS and name in _DEBUG_UNITS:
        for tu in _DEBUG_UNITS[name]:
            if getattr(lib, f"nb_debug_enabled_{tu}")() != 1:
                raise NativeLibraryMissing(f"{p} was not built with -DNB_DEBUG_CHECKS")
        if torch.cuda.is_available():
            _debug_bind(lib, name, torch.cuda.current_device())
    return lib


# ---------------------------------------------------------------- debug-build index checks
_DEBUG_CODES = {5: "index out of bounds", 6: "misaligned coordinate"}
_DEBUG_SITES = {
    1: "embedding gather: row id", 2: "embedding scatter-add: source row", 3: "cross-entropy: class id",
    4: "row-wise kernel: row index", 5: "flat element index", 6: "pooling: pixel index",
    7: "direct convolution: input pixel", 8: "NF4: scale block", 9: "reduction: element index",
    10: "GEMM: TMA tile coordinate", 11: "GEMM: TMA innermost coordinate alignment", 12: "GEMM epilogue: output offset",
    13: "fused GEMM + collective: peer rank", 14: "fused GEMM + collective: block offset",
    15: "attention: TMA tile coordinate", 16: "attention: row-statistics index", 17: "attention: output row",
    18: "peer collectives: rank / world size", 19: "peer collectives: element offset", 20: "peer collectives: flag slot",
}


def debug_record(device: int | None = None) -> torch.Tensor:
    """The int32[8] record that the checked kernels of ``device`` write their first failure to."""
    idx = torch.cuda.current_device() if device is None else int(device)
    rec = _debug_rec.get(idx)
    if rec is None:
        rec = torch.zeros(8, dtype=torch.int32, device=torch.device("cuda", idx))
        _debug_rec[idx] = rec
    return rec


def _debug_bind(lib: ctypes.CDLL, name: str, device: int) -> None:
    rec = debug_record(device)
    with torch.cuda.device(device):
        for tu in _DEBUG_UNITS[name]:
            fn = getattr(lib, f"nb_debug_bind_{tu}")
            fn.argtypes = [ctypes.c_void_p]
            fn.restype = ctypes.c_int
            if fn(ctypes.c_void_p(rec.data_ptr())) != 0:
                raise RuntimeError(f"could not bind the debug record of {name}:{tu}")


def debug_bind(device: int | None = None) -> None:
    """Point every loaded debug library at the record of ``device`` (the libraries bind the device
    that is current when they are loaded; a process that drives more devices calls this per device)."""
    if not DEBUG_KERNELS:
        return
    idx = torch.cuda.current_device() if device is None else int(device)
    for name, lib in _libs.items():
        if name in _DEBUG_UNITS:
            _debug_bind(lib, name, idx)


def debug_selftest(name: str, value: int, limit: int, addr: int = 0, align: int = 16) -> None:
    """Run the one-thread self-test kernel of every translation unit of library ``name``: it
    evaluates ``0 <= value < limit`` and ``addr % align == 0`` through the same macros as the real
    kernels and touches nothing but the record."""
    lib = load(name)
    for tu in _DEBUG_UNITS[name]:
        fn = getattr(lib, f"nb_debug_selftest_{tu}")
        fn.argtypes = [ctypes.c_longlong] * 4 + [ctypes.c_void_p]
        fn.restype = ctypes.c_int
        if fn(int(value), int(limit), int(addr), int(align), stream_ptr()) != 0:
            raise RuntimeError(f"self-test launch of {name}:{tu} failed")


def debug_report(device: int | None = None, clear: bool = True) -> dict | None:
    """What the checked kernels recorded on ``device`` since the last report: ``None`` when every
    check passed (or the release build is loaded), else ``{"code", "what", "site", "where", "value",
    "limit", "count"}`` for the first failed check and the number of failed checks. Synchronises."""
    if not DEBUG_KERNELS:
        return None
    idx = torch.cuda.current_device() if device is None else int(device)
    rec = _debug_rec.get(idx)
    if rec is None:
        return None
    r = rec.cpu().tolist()
    if r[0] == 0:
        return None
    if clear:
        rec.zero_()
    u = lambda lo, hi: ((hi & 0xFFFFFFFF) << 32 | (lo & 0xFFFFFFFF))
    s64 = lambda v: v - (1 << 64) if v >= (1 << 63) else v
    return {"code": r[0], "what": _DEBUG_CODES.get(r[0], "unknown"), "site": r[1],
            "where": _DEBUG_SITES.get(r[1], "unknown"), "value": s64(u(r[2], r[3])), "limit": s64(u(r[4], r[5])),
            "count": r[6]}


class KernelDebugCheckFailed(RuntimeError):
    """A device-side index check of the debug build failed (the access was skipped)."""


def debug_check(device: int | None = None) -> None:
    """Raise ``KernelDebugCheckFailed`` if a checked kernel recorded a failure."""
    rep = debug_report(device)
    if rep is not None:
        raise KernelDebugCheckFailed(f"{rep['where']}: {rep['what']} (value {rep['value']}, limit {rep['limit']}, "
                                     f"{rep['count']} failed checks)")


def use_native(t: torch.Tensor) -> bool:
    """True when ``t`` lives on a CUDA device and native kernels are not disabled."""
    return t.is_cuda and os.environ.get("NABLA_B200_DISABLE_NATIVE", "0") != "1"


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 status word that kernels with bounded waits write on failure."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _status.get(idx)
    if s is None:
        s = torch.zeros(4, dtype=torch.int32, device=device)
        _status[idx] = s
    return s


class KernelStatusError(RuntimeError):
    """A device-side bounded wait ran out (the kernel returned an error status)."""


_STATUS_NAMES = {1: "TMA producer wait timed out", 2: "MMA issuer wait timed out",
                 3: "epilogue wait timed out", 4: "peer flag wait timed out"}


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a bounded-wait failure."""
    devs = list(_status) if device is None else [device.index or 0]
    for idx in devs:
        s = _status.get(idx)
        if s is None:
            continue
        code = int(s[0].item())
        if code != 0:
            s.zero_()
            raise KernelStatusError(f"cuda:{idx}: kernel status {code}: {_STATUS_NAMES.get(code, 'unknown')}")


from .gemm import gemm_bf16, gemm_supported  # noqa: E402,F401


def total_launches() -> int:
    """Number of launches of this package's own kernels issued so far by this process
    (GEMM, attention, fused kernels, peer-memory collectives and fused GEMM+collective)."""
    import sys

    n = 0
    for name in ("nabla_b200.native.gemm", "nabla_b200.native.kernels", "nabla_b200.native.attention",
                 "nabla_b200.parallel.symm"):
        m = sys.modules.get(name)
        if m is not None:
            n += getattr(m, "launch_count", 0)
    return n


# ---------------------------------------------------------------- status watchdog (C++ thread)
def _rt():
    lib = load("libnb_runtime.so")
    lib.nb_rt_watch_start.restype = ctypes.c_int
    lib.nb_rt_watch_start.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
    lib.nb_rt_watch_stop.argtypes = [ctypes.c_int]
    lib.nb_rt_watch_last.restype = ctypes.c_int
    lib.nb_rt_watch_last.argtypes = [ctypes.c_int]
    lib.nb_rt_watch_polls.restype = ctypes.c_longlong
    lib.nb_rt_watch_polls.argtypes = [ctypes.c_int]
    lib.nb_rt_watch_stalled_ms.restype = ctypes.c_double
    lib.nb_rt_watch_stalled_ms.argtypes = [ctypes.c_int]
    lib.nb_rt_watch_clear.argtypes = [ctypes.c_int]
    return lib


def watchdog_start(device: torch.device | None = None, interval_ms: int = 50, word: torch.Tensor | None = None) -> None:
    """Start the C++ watchdog thread of ``device``: it copies the device's status word (or
    ``word``, an int32 CUDA tensor) to pinned host memory on its own stream every ``interval_ms``
    without holding the GIL, so that a failed bounded wait is noticed while Python is busy or
    blocked, and without a device synchronisation in the training loop."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    w = word if word is not None else status_word(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if _rt().nb_rt_watch_start(idx, ctypes.c_void_p(w.data_ptr()), int(interval_ms)) != 0:
        raise RuntimeError("could not start the status watchdog")
    _watched[idx] = w


def watchdog_stop(device: torch.device | None = None) -> None:
    idx = (device.index if device is not None and device.index is not None else torch.cuda.current_device())
    _rt().nb_rt_watch_stop(idx)
    _watched.pop(idx, None)


def watchdog_poll(device: torch.device | None = None) -> dict:
    """What the watchdog has seen so far, without touching the device: ``code`` (first non-zero
    status, 0 if none), ``polls`` (completed copies) and ``stalled_ms`` (age of a copy that has not
    come back yet: a device that stopped answering shows up here)."""
    idx = (device.index if device is not None and device.index is not None else torch.cuda.current_device())
    lib = _rt()
    return {"code": int(lib.nb_rt_watch_last(idx)), "polls": int(lib.nb_rt_watch_polls(idx)),
            "stalled_ms": float(lib.nb_rt_watch_stalled_ms(idx))}


def watchdog_check(device: torch.device | None = None) -> None:
    """Raise ``KernelStatusError`` if the watchdog has recorded a failed bounded wait."""
    idx = (device.index if device is not None and device.index is not None else torch.cuda.current_device())
    code = int(_rt().nb_rt_watch_last(idx))
    if code > 0:
        raise KernelStatusError(f"cuda:{idx}: kernel status {code}: {_STATUS_NAMES.get(code, 'unknown')} (seen by the watchdog)")


_watched: dict = {}
