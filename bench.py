"""Headline benchmark: training throughput (tokens/s) of the dp x tp sharded decoder-only
transformer (24 layers, d_model 2048, 16 heads, MLP 8192 gelu, pre-LayerNorm, vocab 32000,
seq 2048, bf16 parameters, fp32 Adam state, random init, synthetic token ids).

    python bench.py --gpus N --steps K --warmup W          (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Weak scaling: 8 sequences per GPU, i.e. global batch 8*N (64 at N = 8, the configuration of
record, on a ('dp','tp') = (2,4) mesh; tp = min(N, 4), dp = N / tp). One timed step =
forward + backward + AdamW update through the public API (`nabla_b200.compile` of
`value_and_grad` + `nn.adamw_update`). Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "train tokens/sec dp x tp transformer (24L d2048 h16 ff8192 v32000 s2048), max over ranks"
SEQS_PER_GPU = 8


def reference_arm() -> None:
    """The reference (nabla-ml/nabla) needs the `modular` (MAX + Mojo) runtime, which is neither
    installed nor available offline; the package installs with --no-deps but cannot be imported."""
    why = "reference imports `modular`/MAX (nabla/__init__.py:9-19), not installable offline: PackageNotFoundError: modular"
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import nabla  # noqa: F401

        why = "reference imported but its MAX runtime path is not wired into this benchmark"
    except Exception as e:  # pragma: no cover
        why = f"reference cannot be imported here: {type(e).__name__}: {str(e)[:120]}"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler:
    """Samples SM clock / power / throttle reasons of this rank's GPU with nvidia-smi while a
    timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows: list[list[str]] = []
        self._stop = threading.Event()
        self._t: threading.Thread | None = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._loop, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)

    def summary(self) -> dict:
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.rows)}


def _collective_stats():
    from nabla_b200.parallel import backend

    return dict(backend.stats)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="transformer", choices=["transformer", "gpipe", "pp_dp", "lora"],
                    help="transformer = the headline dp x tp benchmark; the others time the pipeline / LoRA "
                         "configurations of nabla_b200.models.configs at their full sizes on the GPUs given")
    ap.add_argument("--layers", type=int, default=24, help="debug only: a run with fewer layers is not a valid number")
    ap.add_argument("--seqs-per-gpu", type=int, default=SEQS_PER_GPU)
    ap.add_argument("--tp", type=int, default=0, help="debug only: tensor-parallel width (default min(N, 4), the benchmark's mesh)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.config != "transformer":
        other_config(args)
        return

    import numpy as np
    import torch

    import nabla_b200 as nb
    from nabla_b200 import native, nn
    from nabla_b200.models import transformer as T
    from nabla_b200.parallel import init_distributed

    rank, world = init_distributed()
    if os.environ.get("NABLA_B200_BENCH_DEBUG"):
        import faulthandler

        faulthandler.dump_traceback_later(int(os.environ["NABLA_B200_BENCH_DEBUG"]), exit=False, file=sys.stderr)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    n = world
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = nb.Accelerator(local)
    tdev = dev.to_torch()
    cfg = T.TransformerConfig(n_layers=args.layers)
    tp = args.tp if args.tp > 0 else min(n, 4)
    dp = n // tp
    mesh = nb.DeviceMesh("mesh", (dp, tp), ("dp", "tp")) if n > 1 else None
    global_batch = args.seqs_per_gpu * n
    seq = cfg.max_seq
    # tokens stay split over 'tp' between the projections (reduce-scatter / all-gather fused
    # with their GEMMs) unless NABLA_B200_SEQ_PARALLEL=0 asks for the all-reduce layout
    sp = T.SeqParallel(mesh, "dp", "tp") if (mesh is not None and tp > 1
                                              and os.environ.get("NABLA_B200_SEQ_PARALLEL", "1") != "0") else None

    with nb.default_device(dev):
        nb.seed(1234)
        params = T.init_params(cfg, mesh=mesh, tp_axis="tp", device=dev)
        nb.realize_all(*nb.tensor_leaves(params))
        state = nn.adamw_init(params, state_dtype=nb.DType.float32)
        nb.realize_all(*nb.tensor_leaves(state))

        # the whole step (forward, backward, AdamW) is recorded once, captured into one CUDA graph
        # and replayed; params and optimizer state are donated, so AdamW updates them in place
        use_graph = os.environ.get("NABLA_B200_CUDA_GRAPH", "1") != "0"

        def step_fn(params, state, tokens, targets):
            loss, grads = nb.value_and_grad(lambda p: T.loss_fn(p, tokens, targets, cfg, sp), create_graph=False)(params)
            params, state = nn.adamw_update(params, grads, state, lr=1e-4, weight_decay=0.01, realize=False)
            return loss, params, state

        train_step = nb.compile(step_fn, cuda_graph=use_graph, donate_argnums=(0, 1))

        # synthetic data: every rank generates the same global batch (same seed) in pinned host
        # memory and keeps its dp slice; a fresh batch per step
        rng = np.random.default_rng(2024)
        n_batches = 2 * args.warmup + 3 * args.steps
        rows = global_batch // dp
        dp_idx = (rank // tp) if mesh is not None else 0
        host = []
        for _ in range(n_batches):
            ids = rng.integers(0, cfg.vocab, (global_batch, seq + 1), dtype=np.int64)[dp_idx * rows:(dp_idx + 1) * rows]
            host.append((torch.from_numpy(np.ascontiguousarray(ids[:, :-1])).pin_memory(),
                         torch.from_numpy(np.ascontiguousarray(ids[:, 1:])).pin_memory()))
        h2d_bytes = 2 * rows * seq * 8

        def to_device(pair):
            outs = []
            for h in pair:
                d = h.to(tdev, non_blocking=True)
                if mesh is None:
                    outs.append(nb.Tensor.from_torch(d))
                else:
                    from nabla_b200.core.sharding.spec import ShardingSpec
                    from nabla_b200.core.tensor.impl import TensorImpl

                    spec = ShardingSpec(mesh, ["dp", None])
                    outs.append(nb.Tensor(impl=TensorImpl([d], shape=(global_batch, seq), dtype=nb.DType.int64,
                                                          device=dev, sharding=spec)))
            return outs

        def sync():
            if world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize()

        def counters():
            from nabla_b200.native import attention, gemm, kernels
            from nabla_b200.parallel import backend

            return native.total_launches()

        # ---- warm-up (includes the one trace)
        it = iter(host)
        for _ in range(args.warmup):
            tok, tgt = to_device(next(it))
            loss, params, state = train_step(params, state, tok, tgt)
        loss.realize()
        sync()
        native.check_status()

        # ---- timed region 1: device time of K steps, inputs already on the device
        staged = [to_device(next(it)) for _ in range(args.steps)]
        sync()
        c0 = counters()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clk:
            e0.record()
            t_issue0 = time.perf_counter()
            for tok, tgt in staged:
                loss, params, state = train_step(params, state, tok, tgt)
            e1.record()
            host_issue_ms = 1e3 * (time.perf_counter() - t_issue0)     # host time to enqueue the K steps
            sync()
        launches = counters() - c0
        if train_step.stats.cuda_graphs:
            launches = train_step.stats.launches_per_graph * args.steps     # replayed from the captured graph
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], device=tdev)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_total = float(t.item())

        # ---- timed region 2: end to end through the public API, per step H2D of the inputs
        # from pinned memory and D2H of the loss
        sync()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_wall0 = time.perf_counter()
        e2.record()
        last = None
        for _ in range(args.steps):
            tok, tgt = to_device(next(it))
            loss, params, state = train_step(params, state, tok, tgt)
            last = loss.item()
        e3.record()
        sync()
        wall_ms = 1e3 * (time.perf_counter() - t_wall0)
        t2 = torch.tensor([max(e2.elapsed_time(e3), wall_ms)], device=tdev)
        if world > 1:
            torch.distributed.all_reduce(t2, op=torch.distributed.ReduceOp.MAX)
        e2e_ms_total = float(t2.item())
        native.check_status()

        # ---- exposed communication: the same step recorded with every collective replaced by its
        # communication-free local counterpart (same GEMM shapes, no byte crosses NVLink); the
        # difference to the real step is what the step fails to hide. Runs last: its numbers are garbage.
        exposed = None
        graph_used = bool(train_step.stats.cuda_graphs)
        launches_per_graph = train_step.stats.launches_per_graph
        if world > 1 and os.environ.get("NABLA_B200_EXPOSED_COMM", "1") != "0":
            from nabla_b200.parallel import symm

            try:
                train_step.release()
                symm.set_local_only(True)
                local_step = nb.compile(step_fn, cuda_graph=use_graph, donate_argnums=(0, 1))
                for _ in range(args.warmup):
                    tok, tgt = to_device(next(it))
                    loss, params, state = local_step(params, state, tok, tgt)
                staged = [to_device(next(it)) for _ in range(args.steps)]
                sync()
                e4, e5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e4.record()
                for tok, tgt in staged:
                    loss, params, state = local_step(params, state, tok, tgt)
                e5.record()
                sync()
                t3 = torch.tensor([e4.elapsed_time(e5)], device=tdev)
                torch.distributed.all_reduce(t3, op=torch.distributed.ReduceOp.MAX)
                local_ms = float(t3.item()) / args.steps
                exposed = {"exposed_comm_ms_per_step": ms_total / args.steps - local_ms,
                           "compute_only_ms_per_step": local_ms,
                           "exposed_comm_fraction": (ms_total / args.steps - local_ms) / (ms_total / args.steps)}
                local_step.release()
            except Exception as e:      # the measurement is optional: never lose the headline numbers to it
                exposed = {"exposed_comm_ms_per_step": None, "error": f"{type(e).__name__}: {str(e)[:160]}"}
            finally:
                symm.set_local_only(False)

        if os.environ.get("NABLA_B200_PROFILE_OPS") and not train_step.stats.cuda_graphs:
            # per-op device time of one more step (event pair around every replayed op), rank 0 -> stderr
            train_step.profile_ops = True
            tok, tgt = to_device(host[0])
            loss, params, state = train_step(params, state, tok, tgt)
            train_step.profile_ops = False
            if rank == 0:
                tot = sum(v[1] for v in train_step.op_profile.values())
                print(f"op profile (rank 0, {tot:.1f} ms summed):", file=sys.stderr)
                for k, v in sorted(train_step.op_profile.items(), key=lambda kv: -kv[1][1])[:40]:
                    print(f"  {v[1]:9.2f} ms {100 * v[1] / tot:5.1f}%  x{v[0]:4d}  {k}", file=sys.stderr)

    tokens_per_step = global_batch * seq
    value = tokens_per_step * args.steps / (ms_total / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms_total / 1e3)
    flops = cfg.flops_per_token(seq) * tokens_per_step
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        sustained = peaks.get("bf16_tflops_sustained", 1400.0)
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids ~U[0,32000), random-init weights",
            "config": {"model": f"decoder-only transformer {cfg.n_layers}L d{cfg.d_model} h{cfg.n_heads} ff{cfg.d_ff} "
                                f"vocab{cfg.vocab} pre-LN gelu, bf16 params + fp32 Adam state",
                       "global_batch": global_batch, "seq_len": seq, "parallelism": f"dp{dp}xtp{tp}" + ("+sp" if sp is not None else ""),
                       "l2": "inputs larger than L2 (per-step working set is tens of GB)",
                       "optimizer": "AdamW fused kernel, inside the timed step",
                       "cuda_graph": graph_used},
            "clocks": clk.summary(),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms_total / args.steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "host_issue_ms_per_step": host_issue_ms / args.steps,
            "final_loss": last,
            "model_tflops_per_gpu": flops / (ms_total / args.steps / 1e3) / 1e12 / n,
            "mfu_of_measured_sustained": flops / (ms_total / args.steps / 1e3) / 1e12 / n / sustained,
            "impl": "ours",
            "collectives": _collective_stats(),
        }
        if exposed is not None:
            out.update(exposed)
        print(json.dumps(out), flush=True)
    from nabla_b200.parallel import shutdown

    del params, state, loss
    shutdown(train_step)


def other_config(args) -> None:
    """`--config gpipe | pp_dp | lora`: the other multi-GPU configurations, same JSON contract."""
    import torch

    import nabla_b200 as nb
    from nabla_b200 import native
    from nabla_b200.models import configs
    from nabla_b200.parallel import init_distributed

    rank, world = init_distributed()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = nb.Accelerator(local)
    tdev = dev.to_torch()
    run = {"gpipe": configs.run_gpipe, "pp_dp": configs.run_pp_dp, "lora": configs.run_lora}[args.config]
    with nb.default_device(dev), ClockSampler(local) as clk:
        res = run(nb, rank, world, dev, tdev, args.steps, args.warmup)
        native.check_status()
    if rank == 0:
        unit = "tokens/s" if args.config == "lora" else "samples/s"
        value = res.get("tokens_per_s", res.get("samples_per_s"))
        metric = {"gpipe": "train samples/sec GPipe MLP (one bf16 Linear 4096 + relu per stage, 32 micro-batches of 64)",
                  "pp_dp": "train samples/sec PP x DP MLP (2 bf16 Linear 8192 + relu per stage, 16 micro-batches of 128 per replica, AdamW)",
                  "lora": "train tokens/sec LoRA rank 16 on q/k/v/o of the 24L d2048 transformer, tensor parallel, seq 2048 batch 32"}
        print(json.dumps({"metric": metric[args.config], "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                          "data": "synthetic N(0,1) activations / token ids ~U[0,32000), random-init weights",
                          "config": res, "clocks": clk.summary(), "gpu_launches": int(native.total_launches()),
                          "impl": "ours"}), flush=True)
    configs.finish()


if __name__ == "__main__":
    main()
