"""Kernel micro-benchmarks: ``python -m nabla_b200.utils.microbench <kernel> [--m ...]``.

Times one native kernel with CUDA events on the launching stream (warm-up, then ``--iters``
timed launches with a write larger than L2 between them) and prints one JSON line with the
achieved TFLOP/s or GB/s. The same command line is what the ``ncu`` summaries under
``profiles/`` were captured from (a handful of launches, small enough to end by itself).

Kernels: gemm, gemm_gelu, attn_fwd, attn_bwd, layernorm_fwd, layernorm_bwd, adamw, lse_pick,
colsum.

Multi-rank modes (run under torchrun, one rank per GPU; device time, max over ranks; rank 0 prints):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m nabla_b200.utils.microbench comm_allreduce
    ... -m nabla_b200.utils.microbench comm_fused [--tokens 16384]

``comm_allreduce``: the peer-memory all-reduce against NCCL at 1 / 16 / 128 MB over all N ranks.
``comm_fused``: GEMM -> reduce-scatter, all-gather -> GEMM and GEMM -> all-reduce at the shapes the
benchmark transformer (d_model 2048, d_ff 8192) runs with tensor parallelism N and ``--tokens`` rows
per rank, each beside "library collective then GEMM", the plain GEMM and the collective alone, with
the fraction of the roofline max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s).
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


def _rank_time(fn, iters: int = 10, warmup: int = 3) -> float:
    """Mean device time of ``fn`` in ms, max over ranks (CUDA events between two barriers)."""
    import torch.distributed as dist

    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return round(float(t.item()), 4)


def comm_main(kind: str, tokens: int) -> None:
    """Multi-rank micro-benchmarks of the peer-memory collectives and the fused GEMM + collective
    kernels (module docstring)."""
    import os

    import torch.distributed as dist

    import nabla_b200 as nb
    from nabla_b200 import native
    from nabla_b200.native.gemm import gemm_bf16
    from nabla_b200.parallel import init_distributed, shutdown, symm

    rank, world = init_distributed()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    mesh = nb.DeviceMesh("m", (world,), ("x",))
    ws = symm.workspace(mesh, ("x",))
    bf = torch.bfloat16
    peaks = _peaks()
    out = {"kernel": kind, "world": world, "nvls": bool(ws.mc_ptr)}
    if kind == "comm_allreduce":
        for mb in (1, 16, 128):
            x = torch.randn(mb * 1024 * 1024 // 2, device=dev, dtype=bf)
            y = x.clone()
            out[f"native_{mb}MB_ms"] = _rank_time(lambda: symm.all_reduce(x, mesh, ("x",)))
            out[f"nccl_{mb}MB_ms"] = _rank_time(lambda: dist.all_reduce(y))
            out[f"native_{mb}MB_busbw_GBs"] = round(2 * (world - 1) / world * mb * 1.048576 / out[f"native_{mb}MB_ms"], 1)
    else:
        d_model, d_ff = 2048, 8192
        M = tokens * world                      # gathered rows of one tensor-parallel group
        link = 770e9

        def roof(flops, nvlink_bytes):
            return max(flops / (peaks["bf16_tflops"] * 1e12), nvlink_bytes / link) * 1e3

        rows = []
        # GEMM -> reduce-scatter: MLP down projection and attention output projection
        for name, K in (("rs_mlp_down", d_ff // world), ("rs_attn_out", d_model // world)):
            a = torch.randn(M, K, device=dev, dtype=bf)
            b = torch.randn(K, d_model, device=dev, dtype=bf)
            o = torch.empty(M // world, d_model, device=dev, dtype=bf)

            def lib():
                dist.reduce_scatter_tensor(o, gemm_bf16(a, b))

            r = {"path": name, "M": M, "N": d_model, "K": K,
                 "fused_ms": _rank_time(lambda: symm.gemm_reduce_scatter(a, b, mesh, ("x",), M // world)),
                 "gemm_then_nccl_ms": _rank_time(lib), "gemm_only_ms": _rank_time(lambda: gemm_bf16(a, b))}
            r["roofline_ms"] = round(roof(2.0 * M * d_model * K, M * d_model * 2 * (world - 1) / world), 4)
            rows.append(r)
        # all-gather -> GEMM: MLP up projection and the packed qkv projection
        for name, N in (("ag_mlp_up", d_ff // world), ("ag_qkv", 3 * d_model // world)):
            xs = torch.randn(tokens, d_model, device=dev, dtype=bf)
            w = torch.randn(d_model, N, device=dev, dtype=bf)
            full = torch.empty(M, d_model, device=dev, dtype=bf)
            ar = symm.arena(mesh, ("x",))
            off = ar.alloc(M * d_model * 2) if ar is not None else None

            def lib():
                dist.all_gather_into_tensor(full, xs)
                return gemm_bf16(full, w)

            r = {"path": name, "M": M, "N": N, "K": d_model,
                 "fused_ms": _rank_time(lambda: symm.all_gather_gemm(xs, w, mesh, ("x",), tokens, arena_off=off)),
                 "nccl_then_gemm_ms": _rank_time(lib), "gemm_only_ms": _rank_time(lambda: gemm_bf16(full, w)),
                 "nccl_all_gather_ms": _rank_time(lambda: dist.all_gather_into_tensor(full, xs)),
                 "switch_multicast": bool(ar is not None and ar.mc_ptr)}
            os.environ["NABLA_B200_AG_MULTIMEM"] = "1"          # one multicast store through the switch
            for c in (4, 8, 12, 16):      # copy CTAs taken from the GEMM
                r[f"fused_multicast_{c}ctas_ms"] = _rank_time(lambda: symm.all_gather_gemm(xs, w, mesh, ("x",), tokens, arena_off=off,
                                                                               comm_ctas=c))
            os.environ["NABLA_B200_AG_MULTIMEM"] = "0"          # one store per peer instead of one multicast store
            r["fused_peer_stores_ms"] = _rank_time(lambda: symm.all_gather_gemm(xs, w, mesh, ("x",), tokens, arena_off=off))
            for c in (8, 12, 16, 20):
                r[f"fused_peer_stores_{c}ctas_ms"] = _rank_time(
                    lambda: symm.all_gather_gemm(xs, w, mesh, ("x",), tokens, arena_off=off, comm_ctas=c))
            os.environ["NABLA_B200_AG_MULTIMEM"] = "auto"
            r["roofline_ms"] = round(roof(2.0 * M * N * d_model, tokens * d_model * 2 * (world - 1)), 4)
            rows.append(r)
            if off is not None:
                ar.free(off)
        # GEMM -> all-reduce: weight gradients summed over the data-parallel replicas (K = tokens of a replica)
        for name, (Mw, Nw) in (("ar_dw_mlp", (d_model, d_ff // 4)), ("ar_dw_qkv", (d_model, 3 * d_model // 4))):
            a = torch.randn(tokens * 4, Mw, device=dev, dtype=bf).t()
            b = torch.randn(tokens * 4, Nw, device=dev, dtype=bf)

            def lib():
                y = gemm_bf16(a, b)
                dist.all_reduce(y)
                return y

            r = {"path": name, "M": Mw, "N": Nw, "K": tokens * 4,
                 "fused_ms": _rank_time(lambda: symm.gemm_all_reduce(a, b, mesh, ("x",))),
                 "gemm_then_nccl_ms": _rank_time(lib), "gemm_only_ms": _rank_time(lambda: gemm_bf16(a, b))}
            r["roofline_ms"] = round(roof(2.0 * Mw * Nw * tokens * 4, 2 * Mw * Nw * 2 * (world - 1) / world), 4)
            rows.append(r)
        for r in rows:
            r["fraction_of_roofline"] = round(r["roofline_ms"] / r["fused_ms"], 3)
        out["rows"] = rows
        out["denominators"] = {"bf16_tflops_burst_measured": peaks["bf16_tflops"], "nvlink_GBs_per_direction": 770}
    native.check_status()
    if rank == 0:
        print(json.dumps(out), flush=True)
    shutdown()


def _peaks() -> dict:
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        return json.load(open(path))
    except Exception:
        return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0}          # documented fallback figures


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel")
    ap.add_argument("--tokens", type=int, default=16384, help="comm_fused: rows per rank")
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
    ap.add_argument("--split-k", type=int, default=0, help="gemm: K slices (0 = automatic, 1 = never split)")
    ap.add_argument("--ta", action="store_true", help="gemm: A given as the transpose of a (K, M) matrix (weight gradient)")
    a = ap.parse_args()
    if a.kernel in ("comm_allreduce", "comm_fused"):
        return comm_main(a.kernel, a.tokens)

    from nabla_b200 import native
    from nabla_b200.native import attention, kernels
    from nabla_b200.native.gemm import gemm_bf16

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    flush = None if a.no_flush else torch.zeros(256 * 1024 * 1024 // 4, device=dev)
    bf = torch.bfloat16
    flops = bytes_ = 0.0
    if a.kernel in ("gemm", "gemm_gelu"):
        x = torch.randn(a.k, a.m, device=dev, dtype=bf).t() if a.ta else torch.randn(a.m, a.k, device=dev, dtype=bf)
        w = torch.randn(a.k, a.n, device=dev, dtype=bf)
        b = torch.randn(a.n, device=dev, dtype=bf)
        if a.kernel == "gemm":
            fn = lambda: gemm_bf16(x, w, block_n=a.block_n, split_k=a.split_k or None)
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
