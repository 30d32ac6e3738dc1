"""Kernel micro-benchmarks: ``python -m nabla_b200.utils.microbench <kernel> [--m ...]``.

Times one native kernel with CUDA events on the launching stream (warm-up, then ``--iters``
timed launches with a write larger than L2 between them) and prints one JSON line with the
achieved TFLOP/s or GB/s. The same command line is what the ``ncu`` summaries under
``profiles/`` were captured from (a handful of launches, small enough to end by itself).

Kernels: gemm, gemm_gelu, attn_fwd, attn_bwd, layernorm_fwd, layernorm_bwd, adamw, lse_pick,
colsum.
"""
from __future__ import annotations

import argparse
import json

import torch


def _flush_l2(buf: torch.Tensor) -> None:
    buf.add_(1)


def _time(fn, iters: int, warmup: int, flush: torch.Tensor | None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            _flush_l2(flush)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--block-n", type=int, default=0, help="gemm: force the tile width (256, 128 or 64)")
    a = ap.parse_args()

    from nabla_b200 import native
    from nabla_b200.native import attention, kernels
    from nabla_b200.native.gemm import gemm_bf16

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    flush = None if a.no_flush else torch.zeros(256 * 1024 * 1024 // 4, device=dev)
    bf = torch.bfloat16
    flops = bytes_ = 0.0
    if a.kernel in ("gemm", "gemm_gelu"):
        x = torch.randn(a.m, a.k, device=dev, dtype=bf)
        w = torch.randn(a.k, a.n, device=dev, dtype=bf)
        b = torch.randn(a.n, device=dev, dtype=bf)
        if a.kernel == "gemm":
            fn = lambda: gemm_bf16(x, w, block_n=a.block_n)
        else:
            fn = lambda: gemm_bf16(x, w, bias=b, epilogue="gelu", aux="store_preact")
        flops = 2.0 * a.m * a.n * a.k
        bytes_ = 2.0 * (a.m * a.k + a.k * a.n + a.m * a.n * (2 if a.kernel == "gemm_gelu" else 1))
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        B, H, S, D = a.batch, a.heads, a.seq, a.head_dim
        qkv = torch.randn(B, S, H, 3, D, device=dev, dtype=bf)
        q, k, v = (qkv[:, :, :, i].transpose(1, 2) for i in range(3))
        sc = D ** -0.5
        o, lse = attention.sdpa_fwd(q, k, v, causal=True, scale=sc)
        do = torch.randn_like(o)
        if a.kernel == "attn_fwd":
            fn = lambda: attention.sdpa_fwd(q, k, v, causal=True, scale=sc)
            flops = 4.0 * B * H * S * S * D / 2
        else:
            fn = lambda: attention.sdpa_bwd(do, q, k, v, o, lse, causal=True, scale=sc)
            flops = 10.0 * B * H * S * S * D / 2
        bytes_ = 2.0 * 4 * B * H * S * D
    elif a.kernel in ("layernorm_fwd", "layernorm_bwd"):
        x = torch.randn(a.m, a.n, device=dev, dtype=bf)
        g = torch.randn(a.n, device=dev, dtype=bf)
        b = torch.randn(a.n, device=dev, dtype=bf)
        y, mean, rstd = kernels.layernorm_fwd(x, g, b, 1e-5)
        dy = torch.randn_like(x)
        if a.kernel == "layernorm_fwd":
            fn = lambda: kernels.layernorm_fwd(x, g, b, 1e-5)
            bytes_ = 2.0 * 2 * a.m * a.n
        else:
            fn = lambda: kernels.layernorm_bwd(dy, x, g, mean, rstd)
            bytes_ = 2.0 * 3 * a.m * a.n
    elif a.kernel == "adamw":
        n = a.m * a.n
        p = torch.randn(n, device=dev, dtype=bf)
        g = torch.randn(n, device=dev, dtype=bf)
        m = torch.zeros(n, device=dev)
        v = torch.zeros(n, device=dev)
        fn = lambda: kernels.adamw(p, g, m, v, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, step=1, inplace=True)
        bytes_ = n * (2 + 2 + 4 + 4 + 2 + 4 + 4)
    elif a.kernel == "lse_pick":
        x = torch.randn(a.m, a.n, device=dev, dtype=bf)
        t = torch.randint(0, a.n, (a.m,), device=dev)
        fn = lambda: kernels.lse_pick_fwd(x, t)
        bytes_ = 2.0 * a.m * a.n
    elif a.kernel == "colsum":
        x = torch.randn(a.m, a.n, device=dev, dtype=bf)
        fn = lambda: kernels.colsum(x)
        bytes_ = 2.0 * a.m * a.n
    else:
        raise SystemExit(f"unknown kernel {a.kernel}")
    ms = _time(fn, a.iters, a.warmup, flush)
    native.check_status()
    out = {"kernel": a.kernel, "ms": ms, "args": {k: v for k, v in vars(a).items() if k != "kernel"}}
    if flops:
        out["tflops"] = flops / ms / 1e9
    out["gbs_algorithmic"] = bytes_ / ms / 1e6
    print(json.dumps(out))


if __name__ == "__main__":
    main()
