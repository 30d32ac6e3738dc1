"""QLoRA helpers: NF4 quantisation on the host, dequantisation on the device
(reference: nabla/nn/finetune/qlora.py:18-113). The dict layout is the reference's:
``indices`` (uint8, one code per element), ``scales`` (fp32 per block), ``original_shape``,
``original_numel``, ``padded_numel``, ``block_size``."""
from __future__ import annotations

from typing import Any

import numpy as np
import torch

from ...core.tensor.api import Tensor
from ...ops.base import Operation
from ...ops.unary import cast
from ...types import DType, as_dtype
from .lora import lora_delta

NF4_CODEBOOK = np.array([-1.0000, -0.6962, -0.5251, -0.3949, -0.2844, -0.1848, -0.0911, 0.0000, 0.0796, 0.1609,
                         0.2461, 0.3379, 0.4407, 0.5626, 0.7230, 1.0000], dtype=np.float32)


def quantize_nf4(weight: Tensor, block_size: int = 64) -> dict[str, Any]:
    if len(weight.shape) != 2:
        raise ValueError("quantize_nf4 expects a 2D weight tensor")
    if block_size <= 0:
        raise ValueError("block_size must be > 0")
    w = weight.to_numpy().astype(np.float32)
    shape = tuple(int(d) for d in w.shape)
    flat = w.reshape(-1)
    n = int(flat.size)
    pad = (block_size - n % block_size) % block_size
    if pad:
        flat = np.pad(flat, (0, pad))
    blocks = flat.reshape(-1, block_size)
    scales = np.max(np.abs(blocks), axis=-1, keepdims=True)
    scales[scales == 0] = 1.0
    norm = (blocks / scales).reshape(-1)
    # nearest codebook entry via the midpoints between sorted codes
    mids = (NF4_CODEBOOK[1:] + NF4_CODEBOOK[:-1]) / 2
    idx = np.searchsorted(mids, norm, side="left").astype(np.uint8)
    exact = np.abs(norm[:, None] - NF4_CODEBOOK[None, :]).argmin(-1) if norm.size <= 1 << 16 else None
    if exact is not None:
        idx = exact.astype(np.uint8)
    dev = weight.device.to_torch()
    return {"indices": Tensor(buffers=[torch.from_numpy(idx).to(dev)]),
            "scales": Tensor(buffers=[torch.from_numpy(scales.reshape(-1).astype(np.float32)).to(dev)]),
            "original_shape": shape, "original_numel": n, "padded_numel": int(flat.size), "block_size": int(block_size)}


_CODEBOOKS: dict = {}      # device -> the 16 codes as an fp32 device tensor


def _codebook_on(device: torch.device) -> torch.Tensor:
    t = _CODEBOOKS.get(device)
    if t is None:
        t = torch.tensor(NF4_CODEBOOK, dtype=torch.float32, device=device)
        _CODEBOOKS[device] = t
    return t


class DequantizeNF4Op(Operation):
    """``codebook[indices] * scale_of_block`` -> dense weight. On a GPU this is ONE launch of
    ``nf4_dequant_codes_kernel`` (fp32 or bf16 output); elsewhere torch indexing."""

    def kernel(self, indices, scales, *, shape, numel: int, block_size: int, dtype: DType):
        td = dtype.to_torch()
        if indices.is_cuda and td in (torch.float32, torch.bfloat16) and indices.dtype == torch.uint8 and numel > 0:
            from ... import native

            if native.use_native(indices):
                from ...native import kernels

                return kernels.nf4_dequant_codes(indices.reshape(-1), scales.reshape(-1), _codebook_on(indices.device),
                                                 int(numel), int(block_size), td).reshape(shape)
        code = _codebook_on(indices.device) if indices.device.type != "meta" else torch.empty(16, device="meta")
        vals = code[indices.long()].reshape(-1, block_size) * scales.float().reshape(-1, 1)
        return vals.reshape(-1)[:numel].reshape(shape).to(td)

    def vjp_rule(self, primals, cot, outputs, kwargs):
        return (None, None)

    def jvp_rule(self, primals, tangents, outputs, kwargs):
        return None


_dequant = DequantizeNF4Op()


def dequantize_nf4(qweight: dict[str, Any], *, dtype=DType.float32) -> Tensor:
    return _dequant(qweight["indices"], qweight["scales"], shape=tuple(qweight["original_shape"]),
                    numel=int(qweight["original_numel"]), block_size=int(qweight["block_size"]), dtype=as_dtype(dtype))


def qlora_linear(x: Tensor, qweight: dict[str, Any], adapter: dict[str, Tensor], *, alpha: float = 1.0,
                 compute_dtype=DType.float32) -> Tensor:
    cd = as_dtype(compute_dtype)
    w = dequantize_nf4(qweight, dtype=cd)
    xc = cast(x, cd)
    A, B = cast(adapter["A"], cd), cast(adapter["B"], cd)
    scale = alpha / float(int(A.shape[1]))
    return (xc @ w) + ((xc @ A) @ B) * scale
