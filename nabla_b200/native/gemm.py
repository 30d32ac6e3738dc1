"""Python wrapper of the tcgen05 bf16 GEMM (``csrc/gemm_tcgen05.cu``)."""
from __future__ import annotations

import ctypes
import os

import torch

EPI = {"none": 0, "bias": 1, "relu": 2, "gelu": 3}
AUX = {"none": 0, "store_preact": 1, "drelu": 2, "dgelu": 3, "add": 4}

_fn = None
launch_count = 0


def _get():
    global _fn
    if _fn is None:
        from . import load

        lib = load("libnb_gemm.so")
        fn = lib.nb_gemm_bf16
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 4 + [ctypes.c_longlong] * 8 + [ctypes.c_int] * 8 + [
            ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        lib.nb_gemm_set_pair_mode.argtypes = [ctypes.c_int]
        lib.nb_gemm_set_pair_mode.restype = ctypes.c_int
        lib.nb_gemm_pair_alloc_probe.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.nb_gemm_pair_alloc_probe.restype = ctypes.c_int
        _fn = fn
        # CTA pairs are the default for wide tiles (NABLA_B200_GEMM_PAIR=0: lone CTAs only). The first
        # call runs the allocator probe, so it must not happen inside a stream capture; `compile`
        # replays a step once uncaptured before it captures.
        if os.environ.get("NABLA_B200_GEMM_PAIR", "1") != "0" and torch.cuda.is_available() \
                and not torch.cuda.is_current_stream_capturing():
            set_pair_mode(True)
    return _fn


def pair_alloc_probe() -> tuple[int, int]:
    """Tensor-memory base addresses that the two CTAs of one cluster get when each asks the pair
    allocator (``tcgen05.alloc.cta_group::2``) for 256 columns. Equal: the two requests are one
    allocation made together, which is what the CTA-pair GEMM assumes."""
    from . import load, stream_ptr

    lib = load("libnb_gemm.so")
    _get()
    out = torch.full((2,), 0xFFFFFFFF, dtype=torch.int64, device="cuda").to(torch.int32)
    rc = lib.nb_gemm_pair_alloc_probe(ctypes.c_void_p(out.data_ptr()), stream_ptr())
    if rc != 0:
        raise RuntimeError(f"nb_gemm_pair_alloc_probe failed with code {rc}")
    torch.cuda.synchronize()
    a, b = (int(v) & 0xFFFFFFFF for v in out.tolist())
    return a, b


_pair_checked = False


def set_pair_mode(on: bool) -> bool:
    """Run wide-tile GEMMs on CTA pairs (``cta_group::2``: 256 x 256 tiles, each CTA staging half of
    B). Switched on only after the allocator probe has shown that a pair's two allocation requests
    are one joint allocation; otherwise the lone-CTA kernel stays. The fused GEMM + collective kernels
    follow unless ``NABLA_B200_GEMM_PAIR_FUSED=0``. Returns whether pairs are on."""
    global _pair_checked
    from . import load

    lib = load("libnb_gemm.so")
    _get()
    if on and not _pair_checked:
        a, b = pair_alloc_probe()
        if a != b:
            lib.nb_gemm_set_pair_mode(0)
            return False
        _pair_checked = True
    fused = os.environ.get("NABLA_B200_GEMM_PAIR_FUSED", "1") != "0"
    lib.nb_gemm_set_pair_mode((3 if fused else 1) if on else 0)
    return bool(on)


def _prep(t: torch.Tensor):
    """Return (tensor, kind, ld, batch_stride) where kind is 'row' (last dim contiguous) or
    'col' (second-to-last dim contiguous). Copies to contiguous row-major when neither holds
    or alignment (multiples of 8 elements, 16-byte base) is not met."""
    assert t.dim() == 3
    b, r, c = t.shape
    sb, sr, sc = t.stride()

    def ok(ld, sbatch):
        return ld % 8 == 0 and (b == 1 or sbatch % 8 == 0) and t.data_ptr() % 16 == 0 and ld > 0

    if sc == 1 and ok(sr, sb) and sr >= c:
        return t, "row", sr, sb
    if sr == 1 and ok(sc, sb) and sc >= r:
        return t, "col", sc, sb
    if c % 8 != 0:
        # pad the contiguous dim to a multiple of 8 so that rows stay 16-byte aligned
        cp = (c + 7) // 8 * 8
        buf = torch.zeros((b, r, cp), dtype=t.dtype, device=t.device)
        buf[:, :, :c] = t
        return buf[:, :, :c], "row", cp, r * cp
    t2 = t.contiguous()
    return t2, "row", c, r * c


def gemm_supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16


_SMS = 0


def split_k_factor(M: int, N: int, K: int) -> int:
    """How many K slices a weight-gradient-shaped GEMM (few output tiles, long K) is cut into: 1 (no
    split), 2, 4 or 8. A small cost model of the kernel picks it: whole waves of tiles over the SMs,
    the tile width the launcher would choose (256, or 128 / 64 when there are too few tiles, which
    run at about 0.9 / 0.4 of the wide tile's rate), plus the fp32 partial sums that a split writes
    and reads back. Measured on a B200: 512 x 2048 x 65536 runs 0.319 ms unsplit (64-wide tiles) and
    0.131 ms in 4 slices; 2048 x 1536 x 65536 0.418 -> 0.366 ms; 2048 x 2048 x 16384 is best unsplit
    (0.118 ms on 128-wide tiles)."""
    global _SMS
    if _SMS == 0:
        _SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    if K < 4096 or (M * N) % 4:
        return 1
    m_t = (M + 127) // 128
    rate = 1.4e15 / _SMS                          # FLOP/s of one SM on wide tiles (sustained)
    tile_eff = {256: 1.0, 128: 0.9, 64: 0.4}

    def est(s: int) -> float:
        bn = 256
        if N <= 64 or m_t * ((N + 255) // 256) * s < _SMS // 2:
            bn = 128
        if N <= 64 or (bn == 128 and m_t * ((N + 127) // 128) * s < _SMS // 2):
            bn = 64
        tiles = m_t * ((N + bn - 1) // bn) * s
        waves = -(-tiles // _SMS)
        t = waves * (2.0 * 128 * bn * (K / s)) / (rate * tile_eff[bn])
        if s > 1:
            t += (s * M * N * 8 + M * N * 2) / 5e12 + 4e-6
        return t

    best, best_t = 1, est(1)
    for s in (2, 4, 8):
        if K % (s * 64) or K // s < 1024:
            break
        t = est(s)
        if t < 0.93 * best_t:
            best, best_t = s, t
    return best


def _k_slices(t3: torch.Tensor, kind: str, ld: int, s: int, k_dim: int) -> torch.Tensor:
    """(1, R, C) operand -> (s, ...) strided view whose batch index walks the K slices (no copy).
    ``k_dim`` is the position of K in the (R, C) shape."""
    _, R, C = t3.shape
    if k_dim == 1:                      # A: (M, K)
        ks = C // s
        strides = (ks, ld, 1) if kind == "row" else (ks * ld, 1, ld)
        return t3.as_strided((s, R, ks), strides, t3.storage_offset())
    ks = R // s                          # B: (K, N)
    strides = (ks * ld, ld, 1) if kind == "row" else (ks, 1, ld)
    return t3.as_strided((s, ks, C), strides, t3.storage_offset())


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, bias: torch.Tensor | None = None, epilogue: str = "none",
              aux: str = "none", aux_in: torch.Tensor | None = None, out: torch.Tensor | None = None,
              out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, gelu_tanh: bool = False,
              alpha: float = 1.0, block_n: int = 0, max_ctas: int = 0, split_k: int | None = None):
    """``out = epilogue(alpha * a @ b + bias)`` for bf16 ``a`` (..., M, K) and ``b`` (..., K, N).

    ``a`` and ``b`` may be arbitrary 2-D/3-D strided views (e.g. ``.transpose(-1, -2)``); views
    whose rows or columns are contiguous are consumed in place through TMA descriptors.
    Returns ``out`` or ``(out, preact)`` when ``aux == 'store_preact'``.
    """
    global launch_count
    from . import ptr, status_word, stream_ptr

    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gemm_bf16 needs bf16 operands"
    squeeze = a.dim() == 2 and b.dim() == 2
    a3 = a if a.dim() == 3 else a.unsqueeze(0)
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    batch = max(a3.shape[0], b3.shape[0])
    if batch > 1 and (b3.shape[0] == 1 or b3.stride(0) == 0) and out is None and aux_in is None:
        # x[b] @ W with a shared W: fold the batch into M (no copy when rows are contiguous)
        if a3.is_contiguous() or (a3.stride(2) == 1 and a3.stride(0) == a3.shape[1] * a3.stride(1)):
            a2 = a3.as_strided((batch * a3.shape[1], a3.shape[2]), (a3.stride(1), 1)) if not a3.is_contiguous() \
                else a3.reshape(batch * a3.shape[1], a3.shape[2])
            r = gemm_bf16(a2, b3[0], bias=bias, epilogue=epilogue, aux=aux, out_dtype=out_dtype,
                          gelu_tanh=gelu_tanh, alpha=alpha, block_n=block_n, max_ctas=max_ctas)
            if isinstance(r, tuple):
                return tuple(x.reshape(batch, a3.shape[1], -1) for x in r)
            return r.reshape(batch, a3.shape[1], -1)
    if a3.shape[0] != batch or (batch > 1 and a3.stride(0) == 0):
        a3 = a3.expand(batch, -1, -1).contiguous()
    if b3.shape[0] != batch or (batch > 1 and b3.stride(0) == 0):
        b3 = b3.expand(batch, -1, -1).contiguous()
    M, K = a3.shape[1], a3.shape[2]
    K2, N = b3.shape[1], b3.shape[2]
    assert K == K2, f"contraction mismatch {a.shape} @ {b.shape}"
    # A: 'row' layout of (M,K) is K-major; 'col' is MN-major.
    a3, akind, lda, sa = _prep(a3)
    # B (K,N): 'row' (N contiguous) is MN-major; 'col' (K contiguous) is K-major.
    b3, bkind, ldb, sb = _prep(b3)
    # split-K: few output tiles and a long K (weight gradients): the K range is cut into slices that
    # run as a batch (each slice an fp32 partial product), and one pass adds the slices
    if (batch == 1 and bias is None and epilogue == "none" and aux == "none" and out is None and not accumulate
            and alpha == 1.0 and block_n == 0 and split_k != 1 and out_dtype in (torch.bfloat16, torch.float32)):
        s_ = split_k if split_k else split_k_factor(M, N, K)
        if s_ > 1 and K % (s_ * 64) == 0:
            from . import kernels

            part = gemm_bf16(_k_slices(a3, akind, lda, s_, 1), _k_slices(b3, bkind, ldb, s_, 0),
                             out_dtype=torch.float32, split_k=1, max_ctas=max_ctas)
            res = kernels.sum_slices(part, out_dtype)
            return res if squeeze else res.unsqueeze(0)
    a_mn = 0 if akind == "row" else 1
    b_mn = 1 if bkind == "row" else 0
    if out is None:
        out = torch.empty((batch, M, N), dtype=out_dtype, device=a.device)
        assert not accumulate
    else:
        out = out if out.dim() == 3 else out.unsqueeze(0)
        assert out.shape == (batch, M, N) and out.stride(2) == 1
    out_fp32 = 1 if out.dtype == torch.float32 else 0
    aux_out = None
    aux_t = None
    if aux == "store_preact":
        aux_out = torch.empty((batch, M, N), dtype=torch.bfloat16, device=a.device)
        aux_t = aux_out
    elif aux != "none":
        aux_t = aux_in if aux_in.dim() == 3 else aux_in.unsqueeze(0)
        assert aux_t.shape == (batch, M, N) and aux_t.dtype == torch.bfloat16
        if aux_t.stride(2) != 1:
            aux_t = aux_t.contiguous()
    if bias is not None:
        bias = bias.reshape(-1)
        assert bias.numel() == N
        if not bias.is_contiguous():
            bias = bias.contiguous()
        if epilogue == "none":
            epilogue = "bias"
    bias_fp32 = 1 if (bias is not None and bias.dtype == torch.float32) else 0
    if bias is not None and bias.dtype not in (torch.float32, torch.bfloat16):
        bias = bias.to(torch.bfloat16)
    st = status_word(a.device)
    rc = _get()(
        ptr(a3), ptr(b3), ptr(out), ptr(bias), ptr(aux_t if aux not in ("none", "store_preact") else None),
        ptr(aux_out), M, N, K, batch, lda, ldb, out.stride(1), sa, sb, out.stride(0) if batch > 1 else M * out.stride(1),
        aux_t.stride(1) if aux_t is not None else 0, aux_t.stride(0) if aux_t is not None else 0,
        a_mn, b_mn, out_fp32, bias_fp32, EPI[epilogue], AUX[aux], int(accumulate), int(gelu_tanh), float(alpha),
        block_n, max_ctas, ptr(st), stream_ptr())
    if rc != 0:
        raise RuntimeError(f"nb_gemm_bf16 failed with code {rc} for {tuple(a.shape)} @ {tuple(b.shape)}")
    launch_count += 1
    res = out[0] if squeeze else out
    if aux == "store_preact":
        return res, (aux_out[0] if squeeze else aux_out)
    return res
