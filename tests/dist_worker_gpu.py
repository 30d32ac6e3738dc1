"""Worker run under torchrun by tests/test_gpu_multi.py (one rank per GPU, NCCL).

Checks, on every rank: the peer-memory collectives and the fused GEMM + collective kernels against
NCCL results (mode 'grouped': on the tp and dp groups of a ('dp', 'tp') mesh, (2, 4) on 8 GPUs),
the sharded transformer step against the unsharded one, and (mode 'lost_peer') that a rank which
leaves between steps is reported to the others as an error. Prints one ``RESULT {json}`` line per
rank. Timing sweeps live in ``nabla_b200.utils.microbench`` (comm_allreduce, comm_fused).
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np
import torch
import torch.distributed as dist

import nabla_b200 as nb
from nabla_b200.parallel import init_distributed


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "collectives"
    rank, world = init_distributed(timeout_s=20 if mode == "lost_peer" else 120)
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    out = {"rank": rank, "world": world, "mode": mode}
    if mode == "collectives":
        from nabla_b200 import native
        from nabla_b200.parallel import backend, symm

        mesh = nb.DeviceMesh("m", (world,), ("x",))
        out["symm_ready"] = symm.is_ready()
        ws = symm.workspace(mesh, ("x",))
        out["nvls"] = bool(ws.mc_ptr)
        errs = {}
        for dtype in (torch.bfloat16, torch.float32):
            for n in (1000, 4096, 1 << 20, (1 << 22) + 24):
                torch.manual_seed(100 + rank)
                x = torch.randn(n, device=dev, dtype=dtype)
                ref = x.clone().float()
                dist.all_reduce(ref)
                algos = ["oneshot", "twoshot"] + (["multimem"] if ws.mc_ptr else [])
                for algo in algos:
                    y = symm.all_reduce(x, mesh, ("x",), "sum", algo=algo)
                    e = ((y.float() - ref).abs().max() / (ref.abs().max() + 1e-6)).item()
                    errs[f"ar_{algo}_{str(dtype)[6:]}_{n}"] = e
            xm = torch.randn(4096, device=dev, dtype=dtype)
            rm = xm.clone()
            dist.all_reduce(rm, op=dist.ReduceOp.MAX)
            errs[f"max_{str(dtype)[6:]}"] = (symm.all_reduce(xm, mesh, ("x",), "max").float() - rm.float()).abs().max().item()
        x = torch.randn(64, 256, device=dev, dtype=torch.bfloat16)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        errs["all_gather"] = (symm.all_gather_dim0(x, mesh, ("x",)).float() - torch.cat(parts).float()).abs().max().item()
        big = torch.randn(64 * world, 256, device=dev, dtype=torch.float32)
        rs_ref = torch.empty(64, 256, device=dev)
        dist.reduce_scatter_tensor(rs_ref, big.clone())
        errs["reduce_scatter"] = (symm.reduce_scatter_dim0(big, mesh, ("x",)) - rs_ref).abs().max().item()
        a2a_ref = torch.empty_like(big)
        dist.all_to_all_single(a2a_ref, big.clone())
        errs["all_to_all"] = (symm.all_to_all_dim0(big, mesh, ("x",)) - a2a_ref).abs().max().item()
        bc = big.clone()
        dist.broadcast(bc, src=0)
        errs["broadcast"] = (symm.broadcast(big, mesh, ("x",), 0) - bc).abs().max().item()
        # point-to-point shift: a pipeline shift (no wrap-around: rank 0 receives zeros, the last rank
        # sends nothing), a ring, and a swap of two ranks that leaves the others out; repeated, so
        # that an inbox is overwritten while the flags and counters carry on
        for shape, dtype in (((64, 4096), torch.bfloat16), ((3, 5, 8), torch.float32), ((1 << 20,), torch.bfloat16)):
            for name, perm in (("pipe", [(i, i + 1) for i in range(world - 1)]),
                               ("ring", [(i, (i + 1) % world) for i in range(world)]),
                               ("swap", [(0, 1), (1, 0)])):
                for rep in range(3):
                    torch.manual_seed(1000 * rep + rank)
                    x = torch.randn(*shape, device=dev).to(dtype)
                    got = backend.permute(x, mesh, perm)
                    src = next((s_ for s_, d_ in perm if d_ == rank), None)
                    if src is None:
                        want = torch.zeros_like(x)
                    else:
                        torch.manual_seed(1000 * rep + src)
                        want = torch.randn(*shape, device=dev).to(dtype)
                    errs[f"permute_{name}_{len(shape)}_{rep}"] = (got.float() - want.float()).abs().max().item()
        out["native_permute"] = backend.stats.get("native_permute", 0)
        torch.cuda.synchronize()
        native.check_status()
        out["max_err"] = max(errs.values())
        out["errs"] = {k: v for k, v in errs.items() if v > 1e-2}
        out["timeout_probe_status"] = symm.wait_flag_timeout_probe(20.0)
        out["canary_ok"] = ws.check_canary()        # nothing wrote past the end of the workspace
    elif mode == "fused_gemm":
        from nabla_b200 import native
        from nabla_b200.native.gemm import gemm_bf16
        from nabla_b200.parallel import symm

        mesh = nb.DeviceMesh("m", (world,), ("x",))
        ws = symm.workspace(mesh, ("x",))
        out["nvls"] = bool(ws.mc_ptr)
        errs = {}
        shapes = [(256, 512, 256), (1000, 264, 328), (4096, 2048, 1024), (300, 2048, 72)]
        for (M, N, K) in shapes:
            for b_t in (False, True):
                torch.manual_seed(7 + rank)
                a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
                b = torch.randn(N, K, device=dev, dtype=torch.bfloat16).t() if b_t else \
                    torch.randn(K, N, device=dev, dtype=torch.bfloat16)
                ref = a.float() @ b.float()
                dist.all_reduce(ref)
                for rep in range(2):          # the flags and counters must be reusable
                    y = symm.gemm_all_reduce(a, b, mesh, ("x",)).clone()
                    torch.cuda.synchronize()
                    errs[f"{M}x{N}x{K}_{int(b_t)}_{rep}"] = ((y.float() - ref).abs().max() / ref.abs().max()).item()
        # reduce-scatter and all-gather variants; rows are dealt to ranks in chunks of `cs`
        for (M, N, K, cs) in [(256 * world, 512, 256, 128), (1024 * world, 264, 328, 256), (512 * world, 2048, 72, 512)]:
            torch.manual_seed(11 + rank)
            a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            b = torch.randn(K, N, device=dev, dtype=torch.bfloat16)
            ref = a.float() @ b.float()
            dist.all_reduce(ref)
            mine = ref.view(-1, world, cs, N)[:, rank].reshape(-1, N)         # this rank's row chunks
            for rep in range(3):
                y = symm.gemm_reduce_scatter(a, b, mesh, ("x",), cs)
                torch.cuda.synchronize()
                errs[f"rs_{M}x{N}x{K}_{rep}"] = ((y.float() - mine).abs().max() / ref.abs().max()).item()
            rb = torch.randn(N, device=dev, dtype=torch.bfloat16)
            rr = torch.randn(M // world, N, device=dev, dtype=torch.bfloat16)
            y = symm.gemm_reduce_scatter(a, b, mesh, ("x",), cs, bias=rb, residual=rr)
            torch.cuda.synchronize()
            errs[f"rs_bias_res_{M}x{N}x{K}"] = ((y.float() - (mine + rb.float() + rr.float())).abs().max()
                                                 / ref.abs().max()).item()
            # all-gather -> GEMM with bias + gelu epilogue and stored pre-activation
            torch.manual_seed(5)                                              # same weights on every rank
            w = torch.randn(K, N, device=dev, dtype=torch.bfloat16) * 0.05
            bias = torch.randn(N, device=dev, dtype=torch.bfloat16)
            torch.manual_seed(13 + rank)
            xs = torch.randn(M // world, K, device=dev, dtype=torch.bfloat16)
            parts = [torch.empty_like(xs) for _ in range(world)]
            dist.all_gather(parts, xs)
            full = torch.stack([p_.view(-1, cs, K) for p_ in parts], 1).reshape(M, K)
            z_ref = full.float() @ w.float() + bias.float()
            ar = symm.arena(mesh, ("x",))
            out["arena"] = ar is not None
            for rep in range(4):
                off = ar.alloc(M * K * 2) if (ar is not None and rep >= 2) else None      # reps 2, 3: push variant
                a_full, y, z = symm.all_gather_gemm(xs, w, mesh, ("x",), cs, bias=bias, epilogue="gelu", store_preact=True,
                                                    arena_off=off)
                torch.cuda.synchronize()
                if off is not None:
                    a_full = a_full.clone()
                    dist.barrier()
                    ar.free(off)
                errs[f"ag_gather_{M}x{K}_{rep}"] = (a_full.float() - full.float()).abs().max().item()
                errs[f"ag_z_{M}x{N}x{K}_{rep}"] = ((z.float() - z_ref).abs().max() / z_ref.abs().max()).item()
                errs[f"ag_y_{M}x{N}x{K}_{rep}"] = ((y.float() - torch.nn.functional.gelu(z_ref)).abs().max()
                                                    / z_ref.abs().max()).item()
        # data-parallel gradient all-reduce fused into AdamW: gradients stay unreduced in the arena
        from nabla_b200.native import kernels as NK

        if ar is not None:
            for n_el in (4096, 1 << 20, (1 << 21) + 4096):
                torch.manual_seed(3)
                p0 = torch.randn(n_el, device=dev, dtype=torch.bfloat16)
                m0 = torch.rand(n_el, device=dev) * 0.1
                v0 = torch.rand(n_el, device=dev) * 0.01
                torch.manual_seed(50 + rank)
                g = torch.randn(n_el, device=dev, dtype=torch.bfloat16)
                gsum = g.float().clone()
                dist.all_reduce(gsum)
                pr, mr, vr = NK.adamw(p0.clone(), gsum, m0.clone(), v0.clone(), lr=1e-2, b1=0.9, b2=0.999, eps=1e-8,
                                      wd=0.01, step=3)
                for rep in range(2):
                    off = ar.alloc(n_el * 2)
                    ar.buf[off: off + n_el * 2].view(torch.bfloat16).copy_(g)
                    p1, m1, v1 = p0.clone(), m0.clone(), v0.clone()
                    symm.adamw_reduce(p1, m1, v1, off, mesh, ("x",), lr=1e-2, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, step=3)
                    torch.cuda.synchronize()
                    ar.free(off)
                    errs[f"dp_adamw_p_{n_el}_{rep}"] = (p1.float() - pr.float()).abs().max().item()
                    errs[f"dp_adamw_m_{n_el}_{rep}"] = ((m1 - mr).abs().max() / mr.abs().max()).item()
                    errs[f"dp_adamw_v_{n_el}_{rep}"] = ((v1 - vr).abs().max() / vr.abs().max()).item()
        # deterministic replay: fixed reduce-job order, peer loads in rank order instead of sums in
        # the switch -> the same bits on every call and on every rank
        from nabla_b200 import config as nb_config

        det_equal, det_same_on_ranks = True, True
        with nb_config.deterministic():
            for (M, N, K) in [(1000, 264, 328), (4096, 2048, 1024)]:
                torch.manual_seed(21 + rank)
                a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
                b = torch.randn(K, N, device=dev, dtype=torch.bfloat16)
                ref = a.float() @ b.float()
                dist.all_reduce(ref)
                ys = []
                for rep in range(3):
                    ys.append(symm.gemm_all_reduce(a, b, mesh, ("x",)).clone())
                    torch.cuda.synchronize()
                errs[f"det_ar_{M}x{N}x{K}"] = ((ys[0].float() - ref).abs().max() / ref.abs().max()).item()
                det_equal &= all(torch.equal(ys[0], y) for y in ys[1:])
                hi, lo = ys[0].float().clone(), ys[0].float().clone()
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                det_same_on_ranks &= bool(torch.equal(hi, lo))
            g = torch.randn((1 << 21) + 24, device=dev, dtype=torch.bfloat16)
            r1 = symm.all_reduce(g, mesh, ("x",)).clone()
            r2 = symm.all_reduce(g, mesh, ("x",)).clone()
            torch.cuda.synchronize()
            det_equal &= bool(torch.equal(r1, r2))
            gs = g.float().clone()
            dist.all_reduce(gs)
            errs["det_allreduce"] = ((r1.float() - gs).abs().max() / gs.abs().max()).item()
        out["det_equal"] = det_equal
        out["det_same_on_ranks"] = det_same_on_ranks
        native.check_status()
        out["max_err"] = max(errs.values())
        out["errs"] = {k: v for k, v in errs.items() if v > 2e-2}
    elif mode == "grouped":
        # the mesh of record: ('dp', 'tp') = (2, 4) on 8 GPUs ((2, 2) on 4): every collective and every
        # fused GEMM + collective on the tp groups and on the dp groups, against NCCL on the same group
        from nabla_b200 import native
        from nabla_b200.parallel import symm

        tp = 4 if world >= 8 else 2
        mesh = nb.DeviceMesh("m", (world // tp, tp), ("dp", "tp"))
        errs = {}
        out["groups"] = {}
        for axes in (("tp",), ("dp",)):
            pg, ranks = mesh.process_group(axes)
            g = len(ranks)
            if g == 1:
                continue
            gi = ranks.index(rank)
            ws = symm.workspace(mesh, axes)
            out["groups"]["+".join(axes)] = {"ranks": ranks, "nvls": bool(ws.mc_ptr)}
            tag = axes[0]
            for dtype in (torch.bfloat16, torch.float32):
                for n in (4096, (1 << 20) + 8 * g, (1 << 22) + 24 * g):
                    torch.manual_seed(100 + rank)
                    x = torch.randn(n, device=dev, dtype=dtype)
                    ref = x.clone().float()
                    dist.all_reduce(ref, group=pg)
                    for algo in ["oneshot", "twoshot"] + (["multimem"] if ws.mc_ptr else []):
                        y = symm.all_reduce(x, mesh, axes, "sum", algo=algo)
                        errs[f"{tag}_ar_{algo}_{str(dtype)[6:]}_{n}"] = ((y.float() - ref).abs().max() / (ref.abs().max() + 1e-6)).item()
            x = torch.randn(64, 256, device=dev, dtype=torch.bfloat16)
            parts = [torch.empty_like(x) for _ in range(g)]
            dist.all_gather(parts, x, group=pg)
            errs[f"{tag}_all_gather"] = (symm.all_gather_dim0(x, mesh, axes).float() - torch.cat(parts).float()).abs().max().item()
            big = torch.randn(64 * g, 256, device=dev, dtype=torch.float32)
            rs_ref = torch.empty(64, 256, device=dev)
            dist.reduce_scatter_tensor(rs_ref, big.clone(), group=pg)
            errs[f"{tag}_reduce_scatter"] = (symm.reduce_scatter_dim0(big, mesh, axes) - rs_ref).abs().max().item()
            # fused GEMM -> all-reduce on this group
            for (M, N, K) in [(1000, 264, 328), (2048, 2048, 512)]:
                torch.manual_seed(7 + rank)
                a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
                b = torch.randn(K, N, device=dev, dtype=torch.bfloat16)
                ref = a.float() @ b.float()
                dist.all_reduce(ref, group=pg)
                for rep in range(2):
                    y = symm.gemm_all_reduce(a, b, mesh, axes).clone()
                    errs[f"{tag}_gemm_ar_{M}x{N}x{K}_{rep}"] = ((y.float() - ref).abs().max() / ref.abs().max()).item()
            # fused GEMM -> reduce-scatter and all-gather -> GEMM on this group
            for (M, N, K, cs) in [(256 * g, 512, 256, 128), (1024 * g, 264, 328, 256)]:
                torch.manual_seed(11 + rank)
                a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
                b = torch.randn(K, N, device=dev, dtype=torch.bfloat16)
                ref = a.float() @ b.float()
                dist.all_reduce(ref, group=pg)
                mine = ref.view(-1, g, cs, N)[:, gi].reshape(-1, N)
                for rep in range(2):
                    y = symm.gemm_reduce_scatter(a, b, mesh, axes, cs)
                    errs[f"{tag}_gemm_rs_{M}x{N}x{K}_{rep}"] = ((y.float() - mine).abs().max() / ref.abs().max()).item()
                torch.manual_seed(5)
                w = torch.randn(K, N, device=dev, dtype=torch.bfloat16) * 0.05
                torch.manual_seed(13 + rank)
                xs = torch.randn(M // g, K, device=dev, dtype=torch.bfloat16)
                parts = [torch.empty_like(xs) for _ in range(g)]
                dist.all_gather(parts, xs, group=pg)
                full = torch.stack([p_.view(-1, cs, K) for p_ in parts], 1).reshape(M, K)
                z_ref = full.float() @ w.float()
                ar = symm.arena(mesh, axes)
                for rep in range(3):
                    off = ar.alloc(M * K * 2) if (ar is not None and rep >= 1) else None      # reps 1, 2: push variant
                    a_full, y = symm.all_gather_gemm(xs, w, mesh, axes, cs, arena_off=off)
                    torch.cuda.synchronize()
                    errs[f"{tag}_ag_gather_{M}x{K}_{rep}"] = (a_full.float() - full.float()).abs().max().item()
                    errs[f"{tag}_ag_gemm_{M}x{N}x{K}_{rep}"] = ((y.float() - z_ref).abs().max() / z_ref.abs().max()).item()
                    if off is not None:
                        dist.barrier(group=pg)
                        ar.free(off)
            torch.cuda.synchronize()
            out.setdefault("canary_ok", True)
            out["canary_ok"] = out["canary_ok"] and ws.check_canary()
        native.check_status()
        out["max_err"] = max(errs.values())
        out["n_checks"] = len(errs)
        out["errs"] = {k: v for k, v in errs.items() if v > 2e-2}
    elif mode == "transformer":
        from nabla_b200.models import transformer as TR
        from nabla_b200.parallel import backend

        tp = 4 if world >= 8 else (2 if world % 2 == 0 else 1)
        cfg = TR.TransformerConfig(n_layers=2, d_model=512, n_heads=4, d_ff=1024, vocab=512, max_seq=256)
        with nb.default_device(nb.Accelerator(dev.index)):
            nb.seed(0)
            params = TR.init_params(cfg, device=nb.Accelerator(dev.index))
            rng = np.random.default_rng(0)
            tok = nb.constant(rng.integers(0, 512, (8, 256)), device=nb.Accelerator(dev.index))
            tgt = nb.constant(rng.integers(0, 512, (8, 256)), device=nb.Accelerator(dev.index))
            l0, g0 = nb.value_and_grad(lambda p: TR.loss_fn(p, tok, tgt, cfg), create_graph=False)(params)
            mesh = nb.DeviceMesh("m", (world // tp, tp), ("dp", "tp"))
            ps = TR.place_params(params, mesh, "tp")
            toks, tgts = tok.shard(mesh, ("dp", None)), tgt.shard(mesh, ("dp", None))
            # sequence-parallel layout (tokens split over 'tp' between the projections): this is what
            # puts the fused GEMM -> reduce-scatter and all-gather -> GEMM kernels on the model's path
            sp = TR.SeqParallel(mesh, "dp", "tp") if (tp > 1 and os.environ.get("NABLA_B200_SEQ_PARALLEL", "1") != "0") else None
            l1, g1 = nb.value_and_grad(lambda p: TR.loss_fn(p, toks, tgts, cfg, sp), create_graph=False)(ps)
            rel = []
            for a, b in zip(nb.tree_leaves(g0), nb.tree_leaves(g1)):
                ta, tb = torch.from_numpy(a.to_numpy()).float(), torch.from_numpy(b.to_numpy()).float()
                rel.append(((ta - tb).norm() / (ta.norm() + 1e-6)).item())
            out.update(loss0=l0.item(), loss1=l1.item(), grad_rel_err=max(rel), backend=dict(backend.stats),
                       mesh=[world // tp, tp], seq_parallel=sp is not None)
    elif mode == "lost_peer":
        import time

        from nabla_b200.parallel import health

        mesh = nb.DeviceMesh("m", (world,), ("x",))
        x = nb.Tensor.from_torch(torch.ones(4, 4, device=dev)).shard(mesh, ("x", None))
        nb.all_reduce(x, reduce_axes={"x"}).realize()
        torch.cuda.synchronize()
        if rank == world - 1:
            health.announce_exit()                         # leaves between steps, nothing in flight
            print("RESULT " + json.dumps({"rank": rank, "left": True}), flush=True)
            os._exit(0)
        try:
            deadline = time.time() + 30
            while time.time() < deadline:                  # the survivors look at the store before launching
                health.check_peers()
                time.sleep(0.2)
            out["detected"] = False
        except health.PeerLostError as e:
            out["detected"] = True
            out["error"] = type(e).__name__
            out["lost"] = e.ranks
    print("RESULT " + json.dumps(out), flush=True)
    if mode == "lost_peer":
        os._exit(0)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
