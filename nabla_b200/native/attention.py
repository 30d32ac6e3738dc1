"""Python wrapper of the tcgen05 flash-attention kernels (``csrc/attention_tcgen05.cu``).

Operands are (B, H, S, D) bf16 views with D contiguous; arbitrary batch / head / row strides are
passed to the kernel (TMA descriptors), so q/k/v sliced out of a packed projection are read in
place. The output is written in (B, S, H, D) memory order and returned as a (B, H, S, D) view,
which makes the following head-merge reshape free.
"""
from __future__ import annotations

import ctypes
import os

import torch

launch_count = 0
_fwd = None
_bwd = None
_checked = False
c_int, c_ll, c_f, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _lib():
    global _fwd, _bwd, _checked
    if not _checked:
        _checked = True
        from . import available, load

        if available("libnb_attention.so"):
            lib = load("libnb_attention.so")
            f = lib.nb_attn_fwd
            f.restype = c_int
            f.argtypes = [c_vp] * 5 + [c_int] * 5 + [c_ll] * 12 + [c_f, c_int, c_vp, c_ll, c_ll, c_ll, c_vp, c_vp]
            _fwd = f
            if hasattr(lib, "nb_attn_bwd"):
                g = lib.nb_attn_bwd
                g.restype = c_int
                g.argtypes = [c_vp] * 10 + [c_int] * 5 + [c_ll] * 24 + [c_f, c_int, c_vp, c_ll, c_ll, c_ll, c_vp, c_vp]
                _bwd = g
    return _fwd


def _ok_view(t: torch.Tensor) -> bool:
    return (t.dim() == 4 and t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0)


def supported(q, k, v, mask, dropout_p) -> bool:
    """Shapes the kernels take: 4-D bf16 (B, H, S, D) with D in {64, 128}, no dropout, and a mask
    (additive float or boolean) that broadcasts to (B, H, Sq, Skv)."""
    if os.environ.get("NABLA_B200_ATTENTION", "native") != "native":
        return False
    if dropout_p or not q.is_cuda or q.dtype != torch.bfloat16:
        return False
    if q.dim() != 4 or q.shape[-1] not in (64, 128) or k.shape != v.shape or k.shape[-1] != q.shape[-1]:
        return False
    if mask is not None:
        if mask.dim() > 4 or mask.dim() < 2 or mask.shape[-1] != k.shape[2] or mask.shape[-2] not in (1, q.shape[2]):
            return False
        lead = (1,) * (4 - mask.dim()) + tuple(mask.shape[:-2])
        if lead[0] not in (1, q.shape[0]) or lead[1] not in (1, q.shape[1]):
            return False
    return _lib() is not None


def _mask_args(mask, B, H, Sq, Skv):
    """fp32 additive mask with the key dim contiguous plus its (batch, head, row) element strides
    (0 where the mask broadcasts). Boolean masks become 0 / -inf. Returns (tensor | None, sb, sh, sq)."""
    if mask is None:
        return None, 0, 0, 0
    m = mask
    if m.dtype == torch.bool:
        m = torch.zeros(m.shape, dtype=torch.float32, device=m.device).masked_fill_(~m, float("-inf"))
    m = m.to(torch.float32)
    while m.dim() < 4:
        m = m.unsqueeze(0)
    if m.stride(3) != 1:
        m = m.contiguous()
    sb = m.stride(0) if m.shape[0] > 1 else 0
    sh = m.stride(1) if m.shape[1] > 1 else 0
    sq = m.stride(2) if m.shape[2] > 1 else 0
    return m, sb, sh, sq


def bwd_available() -> bool:
    _lib()
    return _bwd is not None and os.environ.get("NABLA_B200_ATTENTION_BWD", "native") == "native"


def _prep(t: torch.Tensor) -> torch.Tensor:
    return t if _ok_view(t) else t.contiguous()


def sdpa_fwd(q, k, v, *, causal: bool, scale: float, mask=None):
    """Returns (o, lse): o is a (B, H, S, D) view over (B, S, H, D) memory, lse fp32 (B, H, S)."""
    global launch_count
    from . import ptr, status_word, stream_ptr

    if _lib() is None:
        raise RuntimeError("libnb_attention.so is not built")
    q, k, v = _prep(q), _prep(k), _prep(v)
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    if causal and Sq > Skv:
        raise ValueError("causal attention needs seq_q <= seq_kv")
    o_mem = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    o = o_mem.permute(0, 2, 1, 3)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    st = status_word(q.device)
    m, m_sb, m_sh, m_sq = _mask_args(mask, B, H, Sq, Skv)
    rc = _lib()(ptr(q), ptr(k), ptr(v), ptr(o_mem), ptr(lse), B, H, Sq, Skv, D,
              q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
              v.stride(0), v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2),
              float(scale), int(causal), c_vp(0 if m is None else m.data_ptr()), m_sb, m_sh, m_sq, ptr(st), stream_ptr())
    if rc != 0:
        raise RuntimeError(f"nb_attn_fwd failed with code {rc}")
    launch_count += 1
    return o, lse


def sdpa_bwd(do, q, k, v, o, lse, *, causal: bool, scale: float, out=None, mask=None):
    """Returns (dq, dk, dv); with ``out`` = three (B, H, S, D) views they are written in place."""
    global launch_count
    from . import ptr, status_word, stream_ptr

    _lib()
    q, k, v, do, o = _prep(q), _prep(k), _prep(v), _prep(do), _prep(o)
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    if out is None:
        dq = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
        dk = torch.empty((B, Skv, H, D), dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
        dv = torch.empty((B, Skv, H, D), dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    else:
        dq, dk, dv = out
    # fp32 scratch: delta = rowsum(dO * O) and the log2-domain row statistics, padded to whole tiles
    sq_pad = (Sq + 127) // 128 * 128
    stats = torch.empty((2, B, H, sq_pad), dtype=torch.float32, device=q.device)
    st = status_word(q.device)
    m, m_sb, m_sh, m_sq = _mask_args(mask, B, H, Sq, Skv)
    args = [ptr(do), ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse.contiguous()), ptr(dq), ptr(dk), ptr(dv), ptr(stats)]
    strides = []
    for t in (q, k, v, do, o, dq, dk, dv):
        strides += [t.stride(0), t.stride(1), t.stride(2)]
    rc = _bwd(*args, B, H, Sq, Skv, D, *strides, float(scale), int(causal), c_vp(0 if m is None else m.data_ptr()),
              m_sb, m_sh, m_sq, ptr(st), stream_ptr())
    if rc != 0:
        raise RuntimeError(f"nb_attn_bwd failed with code {rc}")
    launch_count += 3
    return dq, dk, dv
