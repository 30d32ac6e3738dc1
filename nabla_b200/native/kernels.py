"""Python wrappers of the memory-bound fused kernels (``csrc/fused_kernels.cu``).

Inputs and outputs are torch CUDA tensors (bf16 or fp32, contiguous); scratch buffers come
from torch's caching allocator. ``launch_count`` counts kernel launches issued from here.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import load, ptr, stream_ptr

_lib = None
launch_count = 0
c_int, c_ll, c_f, c_vp, c_ull = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_ulonglong


def _L():
    global _lib
    if _lib is None:
        lib = load("libnb_kernels.so")
        sig = {
            "nb_layernorm_fwd": [c_vp] * 6 + [c_int, c_int, c_f, c_int, c_vp],
            "nb_layernorm_bwd_nblocks": [c_int, c_int, c_int],
            "nb_layernorm_bwd": [c_vp] * 9 + [c_int, c_int, c_int, c_vp],
            "nb_colsum_nparts": [c_int],
            "nb_colsum": [c_vp] * 3 + [c_int] * 4 + [c_vp],
            "nb_softmax": [c_vp, c_vp, c_int, c_int, c_int, c_int, c_vp],
            "nb_lse_pick_fwd": [c_vp] * 4 + [c_int, c_int, c_int, c_vp],
            "nb_lse_pick_bwd": [c_vp] * 6 + [c_int, c_int, c_int, c_vp],
            "nb_adamw": [c_vp] * 7 + [c_ll] + [c_f] * 8 + [c_vp, c_int, c_int, c_vp],
            "nb_sgd": [c_vp] * 5 + [c_ll] + [c_f] * 4 + [c_int, c_int, c_vp],
            "nb_embedding_gather": [c_vp] * 3 + [c_int] * 4 + [c_vp],
            "nb_embedding_scatter_add": [c_vp] * 5 + [c_int] * 4 + [c_vp],
            "nb_embedding_scatter_sorted": [c_vp] * 5 + [c_int] * 4 + [c_vp],
            "nb_cast": [c_vp, c_vp, c_ll, c_int, c_int, c_vp],
            "nb_activation": [c_vp] * 3 + [c_ll, c_int, c_int, c_int, c_vp],
            "nb_rng": [c_vp, c_ll, c_ull, c_ull, c_int, c_f, c_f, c_int, c_vp],
            "nb_dropout": [c_vp] * 3 + [c_ll, c_f, c_ull, c_ull, c_int, c_vp],
            "nb_rng_dev": [c_vp, c_ll, c_vp, c_ull, c_int, c_f, c_f, c_int, c_vp],
            "nb_dropout_dev": [c_vp] * 3 + [c_ll, c_f, c_vp, c_ull, c_int, c_vp],
            "nb_nf4_dequant": [c_vp] * 3 + [c_ll, c_int, c_int, c_vp],
            "nb_nf4_dequant_codes": [c_vp] * 4 + [c_ll, c_int, c_int, c_vp],
            "nb_pool2d_fwd": [c_vp, c_vp] + [c_int] * 14 + [c_vp],
            "nb_pool2d_bwd": [c_vp] * 3 + [c_int] * 14 + [c_vp],
            "nb_pool2d_select": [c_vp] * 3 + [c_int] * 13 + [c_vp],
            "nb_conv2d_direct": [c_vp] * 4 + [c_int] * 14 + [c_vp],
            "nb_conv2d_wgrad_direct": [c_vp] * 3 + [c_int] * 14 + [c_vp],
            "nb_sum_slices": [c_vp, c_vp, c_ll, c_int, c_int, c_vp],
            "nb_binary": [c_vp, c_vp, c_vp, c_ll, c_int, c_int, c_ll, c_int, c_int, c_vp],
            "nb_unary": [c_vp, c_vp, c_ll, c_int, c_int, c_vp],
            "nb_reduce": [c_vp, c_vp, c_vp, c_ll, c_ll, c_ll, c_int, c_int, c_vp],
            "nb_reduce_splits": [c_ll, c_ll, c_ll],
            "nb_cumsum": [c_vp, c_vp, c_ll, c_ll, c_ll, c_int, c_int, c_int, c_vp],
        }
        for name, args in sig.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        lib.nb_layernorm_bwd_two_kernels.argtypes = [c_int]
        lib.nb_layernorm_bwd_two_kernels.restype = None
        # NABLA_B200_LN_BWD=two_kernels: dx and dgamma / dbeta in separate passes (the layout for rows
        # wider than 8 vectors per lane), instead of the one-pass kernel
        lib.nb_layernorm_bwd_two_kernels(1 if os.environ.get("NABLA_B200_LN_BWD", "fused") == "two_kernels" else 0)
        _lib = lib
    return _lib


def has(name: str) -> bool:
    """True when the native library is present (every kernel family ships in one library)."""
    try:
        _L()
        return True
    except Exception:
        return False


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise TypeError(f"native kernels take bf16 or fp32, got {t.dtype}")


def _ok(rc: int, what: str) -> None:
    global launch_count
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
    launch_count += 1


def supports_rows(x: torch.Tensor, d_limit: int = 4096) -> bool:
    v = 8 if x.dtype == torch.bfloat16 else 4
    return x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] % v == 0 and x.shape[-1] <= d_limit * (v // 4)


# ---------------------------------------------------------------- layer norm
def layernorm_fwd(x: torch.Tensor, gamma, beta, eps: float):
    D = x.shape[-1]
    x2 = x.contiguous().view(-1, D)
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    g = gamma.contiguous().to(x.dtype) if gamma is not None else None
    b = beta.contiguous().to(x.dtype) if beta is not None else None
    _ok(_L().nb_layernorm_fwd(ptr(x2), ptr(g), ptr(b), ptr(y), ptr(mean), ptr(rstd), rows, D, float(eps), _dt(x),
                              stream_ptr()), "layernorm_fwd")
    return y.view(x.shape), mean, rstd


def layernorm_bwd(dy: torch.Tensor, x: torch.Tensor, gamma, mean: torch.Tensor, rstd: torch.Tensor):
    global launch_count
    D = x.shape[-1]
    x2 = x.contiguous().view(-1, D)
    dy2 = dy.contiguous().view(-1, D)
    rows = x2.shape[0]
    dx = torch.empty_like(x2)
    dgamma = torch.empty(D, dtype=x.dtype, device=x.device)
    dbeta = torch.empty(D, dtype=x.dtype, device=x.device)
    nb = _L().nb_layernorm_bwd_nblocks(rows, D, _dt(x))
    partial = torch.empty((nb, 2, D), dtype=torch.float32, device=x.device)
    g = gamma.contiguous().to(x.dtype) if gamma is not None else None
    _ok(_L().nb_layernorm_bwd(ptr(dy2), ptr(x2), ptr(g), ptr(mean), ptr(rstd), ptr(dx), ptr(dgamma), ptr(dbeta),
                              ptr(partial), rows, D, _dt(x), stream_ptr()), "layernorm_bwd")
    launch_count += 2
    return dx.view(x.shape), dgamma, dbeta


def colsum(x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Sum over all leading dims: (..., N) -> (N,)."""
    global launch_count
    N = x.shape[-1]
    x2 = x.contiguous().view(-1, N)
    rows = x2.shape[0]
    out = torch.empty(N, dtype=out_dtype or x.dtype, device=x.device)
    np_ = _L().nb_colsum_nparts(rows)
    partial = torch.empty((np_, N), dtype=torch.float32, device=x.device)
    _ok(_L().nb_colsum(ptr(x2), ptr(out), ptr(partial), rows, N, _dt(x), _dt(out), stream_ptr()), "colsum")
    launch_count += 1
    return out


# ---------------------------------------------------------------- softmax / cross entropy
def softmax(x: torch.Tensor, log: bool = False) -> torch.Tensor:
    D = x.shape[-1]
    x2 = x.contiguous().view(-1, D)
    y = torch.empty_like(x2)
    _ok(_L().nb_softmax(ptr(x2), ptr(y), x2.shape[0], D, int(log), _dt(x), stream_ptr()), "softmax")
    return y.view(x.shape)


def lse_pick_fwd(logits: torch.Tensor, targets: torch.Tensor):
    """Per row: (logsumexp(logits), logits[target] or 0 when the target is outside [0, D))."""
    D = logits.shape[-1]
    l2 = logits.contiguous().view(-1, D)
    t = targets.contiguous().view(-1).to(torch.int64)
    rows = l2.shape[0]
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    picked = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _ok(_L().nb_lse_pick_fwd(ptr(l2), ptr(t), ptr(lse), ptr(picked), rows, D, _dt(logits), stream_ptr()), "lse_pick_fwd")
    return lse.view(targets.shape), picked.view(targets.shape)


def lse_pick_bwd(logits: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, g_lse, g_pick) -> torch.Tensor:
    D = logits.shape[-1]
    l2 = logits.contiguous().view(-1, D)
    t = targets.contiguous().view(-1).to(torch.int64)
    d = torch.empty_like(l2)
    gl = g_lse.reshape(-1).float().contiguous() if g_lse is not None else None
    gp = g_pick.reshape(-1).float().contiguous() if g_pick is not None else None
    _ok(_L().nb_lse_pick_bwd(ptr(l2), ptr(t), ptr(lse.reshape(-1).float().contiguous()), ptr(gl), ptr(gp), ptr(d),
                             l2.shape[0], D, _dt(logits), stream_ptr()), "lse_pick_bwd")
    return d.view(logits.shape)


# ---------------------------------------------------------------- optimizers
def adamw(p, g, m, v, *, lr, b1, b2, eps, wd, step: int | None = None, hyper: torch.Tensor | None = None,
          grad_scale: float = 1.0, inplace: bool = False):
    """Returns (p', m', v'). ``hyper`` = device tensor [lr, 1-b1^t, 1-b2^t, grad_scale] overrides
    the scalar arguments (lets a captured CUDA graph advance the step)."""
    p = p.contiguous()
    g = g.contiguous()
    po = p if inplace else torch.empty_like(p)
    mo = m if inplace else torch.empty_like(m)
    vo = v if inplace else torch.empty_like(v)
    bc1 = 1.0 - b1 ** step if step is not None else 1.0
    bc2 = 1.0 - b2 ** step if step is not None else 1.0
    _ok(_L().nb_adamw(ptr(p), ptr(g), ptr(m), ptr(v), ptr(po), ptr(mo), ptr(vo), p.numel(), float(lr), float(b1),
                      float(b2), float(eps), float(wd), float(bc1), float(bc2), float(grad_scale), ptr(hyper), _dt(p),
                      _dt(g), stream_ptr()), "adamw")
    return po, mo, vo


def sgd(p, g, buf, *, lr, momentum=0.0, wd=0.0, grad_scale=1.0):
    p = p.contiguous()
    g = g.contiguous()
    po = torch.empty_like(p)
    bo = torch.empty_like(buf) if buf is not None else None
    _ok(_L().nb_sgd(ptr(p), ptr(g), ptr(buf), ptr(po), ptr(bo), p.numel(), float(lr), float(momentum), float(wd),
                    float(grad_scale), _dt(p), _dt(g), stream_ptr()), "sgd")
    return po, bo


# ---------------------------------------------------------------- embedding
def embedding_gather(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    table = table.contiguous()
    flat = ids.contiguous().view(-1).to(torch.int64)
    D = table.shape[1]
    out = torch.empty((flat.numel(), D), dtype=table.dtype, device=table.device)
    _ok(_L().nb_embedding_gather(ptr(table), ptr(flat), ptr(out), flat.numel(), D, table.shape[0], _dt(table),
                                 stream_ptr()), "embedding_gather")
    return out.view(*ids.shape, D)


def embedding_scatter_add(base: torch.Tensor, ids: torch.Tensor, upd: torch.Tensor) -> torch.Tensor:
    """base + scatter_add(ids, upd) with fp32 accumulation (embedding backward)."""
    global launch_count
    base = base.contiguous()
    V, D = base.shape
    flat = ids.contiguous().view(-1).to(torch.int64)
    u = upd.contiguous().view(-1, D).to(base.dtype)
    from .. import config

    if config.is_deterministic():
        # no atomics: stable sort of the ids, then one block per run of equal ids adds the run's rows
        # in their original order
        sorted_ids, perm = torch.sort(flat, stable=True)
        out = base.clone()
        _ok(_L().nb_embedding_scatter_sorted(ptr(sorted_ids), ptr(perm), ptr(u), ptr(base), ptr(out), flat.numel(), D, V,
                                             _dt(base), stream_ptr()), "embedding_scatter_sorted")
        launch_count += 1
        return out
    acc = torch.zeros((V, D), dtype=torch.float32, device=base.device)
    out = torch.empty_like(base)
    _ok(_L().nb_embedding_scatter_add(ptr(acc), ptr(flat), ptr(u), ptr(base), ptr(out), flat.numel(), D, V, _dt(base),
                                      stream_ptr()), "embedding_scatter_add")
    launch_count += 1
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _ok(_L().nb_cast(ptr(x), ptr(out), x.numel(), _dt(x), _dt(out), stream_ptr()), "cast")
    return out


ACT = {"relu": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3}


def activation(z: torch.Tensor, mode: str) -> torch.Tensor:
    z = z.contiguous()
    out = torch.empty_like(z)
    _ok(_L().nb_activation(ptr(z), None, ptr(out), z.numel(), ACT[mode], 0, _dt(z), stream_ptr()), "activation")
    return out


def activation_bwd(z: torch.Tensor, dy: torch.Tensor, mode: str) -> torch.Tensor:
    z = z.contiguous()
    dy = dy.contiguous().to(z.dtype)
    out = torch.empty_like(z)
    _ok(_L().nb_activation(ptr(z), ptr(dy), ptr(out), z.numel(), ACT[mode], 1, _dt(z), stream_ptr()), "activation_bwd")
    return out


# ---------------------------------------------------------------- RNG
_rng_states: dict = {}      # device -> (int64[2] tensor [seed, draws so far], host epoch it was written for)


def rng_state(device) -> torch.Tensor:
    """This device's random-stream position ``[seed, draws so far]`` in device memory. The kernels
    read it when they run and a one-thread kernel advances it after each draw, so a CUDA-graph replay
    continues the stream instead of repeating it. Re-written from the host after every ``seed()``
    call (never during stream capture: run one uncaptured step first, which ``compile`` does)."""
    from ..core.graph.engine import GRAPH

    device = torch.device(device)
    epoch = (GRAPH.seed, getattr(GRAPH, "seed_epoch", 0))
    ent = _rng_states.get(device)
    if ent is None or ent[1] != epoch:
        if torch.cuda.is_current_stream_capturing():
            if ent is None:
                raise RuntimeError("random op inside CUDA-graph capture before the device stream state exists")
            return ent[0]
        t = ent[0] if ent is not None else torch.zeros(2, dtype=torch.int64, device=device)
        t.copy_(torch.tensor([GRAPH.seed & (2 ** 63 - 1), GRAPH.rng_counter], dtype=torch.int64))
        ent = (t, epoch)
        _rng_states[device] = ent
    return ent[0]


def rng_dev(shape, dtype: torch.dtype, device, salt: int, mode: str, a: float, b: float) -> torch.Tensor:
    """Uniform / gaussian tensor from this device's stream (``rng_state``), Philox in one kernel."""
    out = torch.empty(shape, dtype=dtype, device=device)
    st = rng_state(out.device)
    _ok(_L().nb_rng_dev(ptr(out), out.numel(), ptr(st), salt & (2 ** 64 - 1), 0 if mode == "uniform" else 1,
                        float(a), float(b), _dt(out), stream_ptr()), "rng")
    return out


def dropout_dev(x: torch.Tensor, p: float, salt: int):
    """Dropout whose mask comes from this device's stream (``rng_state``): ``(y, keep mask uint8)``."""
    x = x.contiguous()
    y = torch.empty_like(x)
    mask = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    st = rng_state(x.device)
    _ok(_L().nb_dropout_dev(ptr(x), ptr(y), ptr(mask), x.numel(), float(p), ptr(st), salt & (2 ** 64 - 1), _dt(x),
                            stream_ptr()), "dropout")
    return y, mask


def rng(shape, dtype: torch.dtype, device, seed: int, offset: int, mode: str, a: float, b: float) -> torch.Tensor:
    out = torch.empty(shape, dtype=dtype, device=device)
    _ok(_L().nb_rng(ptr(out), out.numel(), seed & (2 ** 64 - 1), offset & (2 ** 64 - 1), 0 if mode == "uniform" else 1,
                    float(a), float(b), _dt(out), stream_ptr()), "rng")
    return out


def dropout(x: torch.Tensor, p: float, seed: int, offset: int):
    x = x.contiguous()
    y = torch.empty_like(x)
    mask = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    _ok(_L().nb_dropout(ptr(x), ptr(y), ptr(mask), x.numel(), float(p), seed & (2 ** 64 - 1), offset & (2 ** 64 - 1),
                        _dt(x), stream_ptr()), "dropout")
    return y, mask


def nf4_dequant(packed: torch.Tensor, absmax: torch.Tensor, n: int, block: int, dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty(n, dtype=dtype, device=packed.device)
    _ok(_L().nb_nf4_dequant(ptr(packed.contiguous()), ptr(absmax.contiguous().float()), ptr(out), n, block, _dt(out),
                            stream_ptr()), "nf4_dequant")
    return out


# ---------------------------------------------------------------- pooling / conv (NHWC)
def pool2d_fwd(x, kh, kw, sh, sw, ph, pw, mode: str):
    x = x.contiguous()
    N, H, W, C = x.shape
    OH = (H + 2 * ph - kh) // sh + 1
    OW = (W + 2 * pw - kw) // sw + 1
    y = torch.empty((N, OH, OW, C), dtype=x.dtype, device=x.device)
    _ok(_L().nb_pool2d_fwd(ptr(x), ptr(y), N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw, 0 if mode == "avg" else 1,
                           _dt(x), stream_ptr()), "pool2d_fwd")
    return y


def pool2d_bwd(x, dy, kh, kw, sh, sw, ph, pw, mode: str):
    x = x.contiguous()
    dy = dy.contiguous()
    N, H, W, C = x.shape
    _, OH, OW, _ = dy.shape
    dx = torch.empty_like(x)
    _ok(_L().nb_pool2d_bwd(ptr(x), ptr(dy), ptr(dx), N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw,
                           0 if mode == "avg" else 1, _dt(x), stream_ptr()), "pool2d_bwd")
    return dx


def pool2d_select(x, t, kh, kw, sh, sw, ph, pw):
    """``out[window] = t[arg-max of x over the window]`` (NHWC; the tangent of max pooling)."""
    x = x.contiguous()
    t = t.contiguous().to(x.dtype)
    N, H, W, C = x.shape
    OH = (H + 2 * ph - kh) // sh + 1
    OW = (W + 2 * pw - kw) // sw + 1
    y = torch.empty((N, OH, OW, C), dtype=x.dtype, device=x.device)
    _ok(_L().nb_pool2d_select(ptr(x), ptr(t), ptr(y), N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw, _dt(x), stream_ptr()),
        "pool2d_select")
    return y


def conv2d_direct(x, w, bias, stride, padding):
    """NHWC x RSCF direct convolution; padding = (top, bottom, left, right)."""
    x = x.contiguous()
    w = w.contiguous().to(x.dtype)
    N, H, W, C = x.shape
    R, S, _, F = w.shape
    pt, pb, pl, pr = padding
    OH = (H + pt + pb - R) // stride[0] + 1
    OW = (W + pl + pr - S) // stride[1] + 1
    y = torch.empty((N, OH, OW, F), dtype=x.dtype, device=x.device)
    b = bias.contiguous().to(x.dtype).view(-1) if bias is not None else None
    _ok(_L().nb_conv2d_direct(ptr(x), ptr(w), ptr(b), ptr(y), N, H, W, C, R, S, F, OH, OW, stride[0], stride[1], pt, pl,
                              _dt(x), stream_ptr()), "conv2d_direct")
    return y


def conv2d_wgrad_direct(x, dy, w_shape, stride, padding):
    """Filter gradient of the NHWC x RSCF convolution: ``dw[r,s,c,f] = sum x[...] * dy[...]`` over
    the batch and all output pixels (deterministic, no atomics)."""
    x = x.contiguous()
    dy = dy.contiguous().to(x.dtype)
    N, H, W, C = x.shape
    R, S, _, F = w_shape
    OH, OW = dy.shape[1], dy.shape[2]
    dw = torch.empty((R, S, C, F), dtype=x.dtype, device=x.device)
    _ok(_L().nb_conv2d_wgrad_direct(ptr(x), ptr(dy), ptr(dw), N, H, W, C, R, S, F, OH, OW, stride[0], stride[1],
                                    padding[0], padding[2], _dt(x), stream_ptr()), "conv2d_wgrad_direct")
    return dw


def nf4_dequant_codes(codes: torch.Tensor, absmax: torch.Tensor, codebook: torch.Tensor, n: int, block: int,
                      dtype: torch.dtype) -> torch.Tensor:
    """``out[i] = codebook[codes[i]] * absmax[i // block]`` for one-code-per-byte NF4 weights, in one
    kernel; ``dtype`` fp32 or bf16."""
    out = torch.empty(n, dtype=dtype, device=codes.device)
    _ok(_L().nb_nf4_dequant_codes(ptr(codes.contiguous()), ptr(absmax.contiguous().float()),
                                  ptr(codebook.contiguous().float()), ptr(out), n, block, _dt(out), stream_ptr()),
        "nf4_dequant_codes")
    return out


def sum_slices(part: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Sum a contiguous fp32 tensor over its leading dim (the partial products of a split-K GEMM)."""
    s_ = part.shape[0]
    out = torch.empty(part.shape[1:], dtype=out_dtype, device=part.device)
    _ok(_L().nb_sum_slices(ptr(part), ptr(out), out.numel(), s_, _dt(out), stream_ptr()), "sum_slices")
    return out


# ---------------------------------------------------------------- pointwise / reduction families
BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "maximum": 4, "minimum": 5, "pow": 6}
UNARY_OPS = {"neg": 0, "abs": 1, "exp": 2, "log": 3, "sqrt": 4, "rsqrt": 5, "tanh": 6, "sigmoid": 7, "sin": 8, "cos": 9,
             "erf": 10, "log1p": 11, "floor": 12, "trunc": 13, "round": 14, "square": 15, "reciprocal": 16}
REDUCE_OPS = {"sum": 0, "max": 1, "min": 2, "mean": 3, "argmax": 4, "argmin": 5}
_FLOATS = (torch.float32, torch.bfloat16)


def elementwise_enabled() -> bool:
    import os

    return os.environ.get("NABLA_B200_ELEMENTWISE", "native") == "native"


def binary(a: torch.Tensor, b: torch.Tensor, op: str):
    """``a (op) b`` in one kernel when both are fp32 / bf16 CUDA tensors of one dtype and ``b`` (or
    ``a``) has the other's shape, is a single element, or is a vector over the trailing dims (bias
    style). Returns None for anything else (mixed dtypes, general broadcasting, integers): the caller
    then uses the framework's generic path."""
    if not (a.is_cuda and b.is_cuda and a.dtype == b.dtype and a.dtype in _FLOATS and elementwise_enabled()):
        return None
    swap = 0
    if a.numel() < b.numel():
        a, b, swap = b, a, 1
    if a.numel() == 0 or tuple(torch.broadcast_shapes(a.shape, b.shape)) != tuple(a.shape):
        return None
    v = 16 // a.element_size()
    if b.numel() == 1:
        mode, inner = 1, 1
    elif tuple(b.shape) == tuple(a.shape):
        mode, inner = 0, 1
    else:
        bs = tuple(b.shape)
        while bs and bs[0] == 1:
            bs = bs[1:]
        if not bs or tuple(a.shape[len(a.shape) - len(bs):]) != bs:
            return None
        mode, inner = 2, b.numel()
        if inner % v:
            return None
    a_c, b_c = a.contiguous(), b.contiguous()
    if (a_c.data_ptr() | b_c.data_ptr()) & 15:
        return None
    out = torch.empty_like(a_c)
    _ok(_L().nb_binary(ptr(a_c), ptr(b_c), ptr(out), a_c.numel(), BINARY_OPS[op], mode, inner, swap, _dt(a_c), stream_ptr()),
        "binary")
    return out


def unary(x: torch.Tensor, op: str):
    """``f(x)`` in one kernel for fp32 / bf16 CUDA tensors; None otherwise."""
    if not (x.is_cuda and x.dtype in _FLOATS and x.numel() and elementwise_enabled()):
        return None
    xc = x.contiguous()
    if xc.data_ptr() & 15:
        return None
    out = torch.empty_like(xc)
    _ok(_L().nb_unary(ptr(xc), ptr(out), xc.numel(), UNARY_OPS[op], _dt(xc), stream_ptr()), "unary")
    return out


def _outer_r_inner(x: torch.Tensor, axis: int):
    outer = 1
    for d in x.shape[:axis]:
        outer *= int(d)
    inner = 1
    for d in x.shape[axis + 1:]:
        inner *= int(d)
    return outer, int(x.shape[axis]), inner


def reduce(x: torch.Tensor, axis: int, op: str, keepdims: bool = False):
    """sum / max / min / mean / argmax / argmin over one axis in one kernel (fp32 / bf16 CUDA, non-empty
    axis); None otherwise."""
    if not (x.is_cuda and x.dtype in _FLOATS and x.numel() and elementwise_enabled()):
        return None
    axis = axis % x.dim() if x.dim() else 0
    if x.dim() == 0:
        return None
    xc = x.contiguous()
    outer, r, inner = _outer_r_inner(xc, axis)
    if inner > 1 and op == "sum" and outer == 1 and r > 4096 and supports_rows(xc.reshape(r, inner)):
        # column sums of a tall 2-D matrix (bias-gradient shape) have their own slab kernel
        out = colsum(xc.reshape(r, inner), out_dtype=x.dtype)
        return out.reshape([1] + list(xc.shape[axis + 1:]) if keepdims else list(xc.shape[axis + 1:]))
    shape = list(xc.shape)
    if keepdims:
        shape[axis] = 1
    else:
        shape.pop(axis)
    out = torch.empty(shape, dtype=torch.int64 if op.startswith("arg") else x.dtype, device=x.device)
    splits = _L().nb_reduce_splits(outer, r, inner)
    scratch = torch.empty(outer * splits * inner * 3, dtype=torch.float32, device=x.device) if splits > 1 else None
    _ok(_L().nb_reduce(ptr(xc), ptr(out), ptr(scratch), outer, r, inner, REDUCE_OPS[op], _dt(xc), stream_ptr()), "reduce")
    return out


def cumsum(x: torch.Tensor, axis: int, exclusive: bool = False, reverse: bool = False):
    if not (x.is_cuda and x.dtype in _FLOATS and x.numel() and x.dim() and elementwise_enabled()):
        return None
    xc = x.contiguous()
    outer, r, inner = _outer_r_inner(xc, axis % x.dim())
    if outer * inner < 4096 and r > 2048:
        return None                      # a few long scans: the sequential-per-column kernel is the wrong tool
    out = torch.empty_like(xc)
    _ok(_L().nb_cumsum(ptr(xc), ptr(out), outer, r, inner, int(exclusive), int(reverse), _dt(xc), stream_ptr()), "cumsum")
    return out
