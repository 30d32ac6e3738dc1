"""The other multi-GPU training configurations besides the dp x tp transformer of ``bench.py``:

* ``gpipe``  GPipe MLP pipeline: S stages (one per GPU), bf16 Linear 4096 -> 4096 + relu per stage,
  ``vmap(spmd_axis_name='stage')`` + ``ppermute`` shift, 32 micro-batches of (64, 4096), MSE loss.
* ``pp_dp``  PP x DP MLP: ('stage', 'dp') mesh, bf16 Linear 8192 -> 8192 + relu stages, 16 micro-batches
  of (128, 8192) per replica, AdamW on the stage weights (gradients all-reduced over 'dp').
* ``lora``   LoRA fine-tuning of the 24-layer d=2048 transformer: frozen bf16 base, rank-16 adapters on
  q/k/v/o, tensor parallel over all GPUs, seq 2048, batch 32; only adapter gradients exist.

* ``cpu_mlp``  the CPU training configuration: fp32 MLP 64 -> 256 -> 256 -> 256 -> 1 with relu, x (512, 64)
  ~ U(0, 1) from seed 0, y = sin(2 pi mean(x, axis=1)), MSE, Adam lr 1e-3, 100 steps, one device
  (``python -m nabla_b200.models.configs cpu_mlp``; no torchrun, no GPU).

Run under torchrun, one rank per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m nabla_b200.models.configs gpipe --steps 5

Rank 0 prints one JSON line: samples (or tokens) per second over the timed steps (CUDA events, max
over ranks, after warm-up; the compiled step is recorded once and replayed).
(Reference recipes: examples/07_mlp_pipeline_parallel.ipynb, examples/08_mlp_pp_dp_training.ipynb,
nabla/nn/finetune/lora.py.)
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch


_COMPILED: list = []      # compiled step functions of this process, released by `finish`


def finish() -> None:
    """Release the recorded steps (and their CUDA graphs) and leave the process group in order."""
    from nabla_b200.parallel import shutdown

    shutdown(*_COMPILED)
    _COMPILED.clear()


def _graph() -> bool:
    """Replay the recorded step from one CUDA graph (default) unless NABLA_B200_CUDA_GRAPH=0."""
    return os.environ.get("NABLA_B200_CUDA_GRAPH", "1") != "0"


def _timed(step_fn, warmup: int, steps: int, world: int, dev) -> float:
    for _ in range(warmup):
        out = step_fn()
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step_fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item()) / steps, out


def run_gpipe(nb, rank, world, dev, tdev, steps, warmup, dim=4096, micro=32, batch=64):
    from nabla_b200.models import mlp_pipeline as P

    S = world
    mesh = nb.DeviceMesh("pipe", (S,), ("stage",))
    nb.seed(1)
    w = P.place_stage_params(nb.gaussian((S, dim, dim), 0.0, dim ** -0.5, dtype=nb.DType.bfloat16, device=dev), mesh)
    b = P.place_stage_params(nb.zeros((S, dim), dtype=nb.DType.bfloat16, device=dev), mesh)
    xs = nb.gaussian((micro, batch, dim), 0.0, 1.0, dtype=nb.DType.bfloat16, device=dev)
    ys = nb.gaussian((micro, batch, dim), 0.0, 1.0, dtype=nb.DType.bfloat16, device=dev)
    nb.realize_all(w, b, xs, ys)

    @nb.compile(cuda_graph=_graph())
    def step(w, b, xs, ys):
        loss, (gw, gb) = nb.value_and_grad(lambda w_, b_: P.gpipe_loss(w_, b_, xs, ys, mesh), argnums=(0, 1))(w, b)
        return loss, w - gw * 1e-3, b - gb * 1e-3

    state = [w, b]
    _COMPILED.append(step)

    def one():
        loss, state[0], state[1] = step(state[0], state[1], xs, ys)
        return loss

    ms, loss = _timed(one, warmup, steps, world, tdev)
    return {"config": "gpipe", "stages": S, "micro_batches": micro, "batch": batch, "dim": dim, "ms_per_step": ms,
            "samples_per_s": micro * batch / (ms / 1e3), "loss": float(loss.item())}


def run_pp_dp(nb, rank, world, dev, tdev, steps, warmup, dim=8192, micro=16, batch=128):
    from nabla_b200 import nn
    from nabla_b200.models import mlp_pipeline as P

    dp = 2 if world % 2 == 0 and world >= 4 else 1
    S = world // dp
    mesh = nb.DeviceMesh("ppdp", (S, dp), ("stage", "dp"))
    nb.seed(2)
    def wt():
        return P.place_stage_params(nb.gaussian((S, dim, dim), 0.0, dim ** -0.5, dtype=nb.DType.bfloat16, device=dev), mesh)

    def bs():
        return P.place_stage_params(nb.zeros((S, dim), dtype=nb.DType.bfloat16, device=dev), mesh)

    params = {"w1": wt(), "b1": bs(), "w2": wt(), "b2": bs()}      # two Linear + relu per stage
    xs = nb.gaussian((micro, batch * dp, dim), 0.0, 1.0, dtype=nb.DType.bfloat16, device=dev)
    ys = nb.gaussian((micro, batch * dp, dim), 0.0, 1.0, dtype=nb.DType.bfloat16, device=dev)
    if dp > 1:
        xs, ys = xs.shard(mesh, (None, "dp", None)), ys.shard(mesh, (None, "dp", None))
    nb.realize_all(*nb.tensor_leaves(params), xs, ys)
    state = nn.adamw_init(params, state_dtype=nb.DType.float32)
    nb.realize_all(*nb.tensor_leaves(state))

    @nb.compile(cuda_graph=_graph(), donate_argnums=(0, 1))
    def step(params, state, xs, ys):
        loss, grads = nb.value_and_grad(
            lambda p: P.gpipe_loss((p["w1"], p["w2"]), (p["b1"], p["b2"]), xs, ys, mesh, "stage",
                                   "dp" if dp > 1 else None))(params)
        params, state = nn.adamw_update(params, grads, state, lr=1e-4, weight_decay=0.0, realize=False)
        return loss, params, state

    box = [params, state]
    _COMPILED.append(step)

    def one():
        loss, box[0], box[1] = step(box[0], box[1], xs, ys)
        return loss

    ms, loss = _timed(one, warmup, steps, world, tdev)
    return {"config": "pp_dp", "stages": S, "dp": dp, "micro_batches": micro, "batch_per_replica": batch, "dim": dim,
            "ms_per_step": ms, "samples_per_s": micro * batch * dp / (ms / 1e3), "loss": float(loss.item())}


def run_lora(nb, rank, world, dev, tdev, steps, warmup, layers=24, batch=32, seq=2048):
    from nabla_b200 import nn
    from nabla_b200.models import transformer as T

    cfg = T.TransformerConfig(n_layers=layers, max_seq=seq)
    mesh = nb.DeviceMesh("tp", (world,), ("tp",)) if world > 1 else None
    nb.seed(3)
    params = T.init_params(cfg, mesh=mesh, tp_axis="tp", device=dev)
    lora = T.init_lora(params, cfg, rank=16, init_std=0.02, mesh=mesh, tp_axis="tp")
    nb.realize_all(*nb.tensor_leaves(params), *nb.tensor_leaves(lora))
    state = nn.adamw_init(lora, state_dtype=nb.DType.float32)
    nb.realize_all(*nb.tensor_leaves(state))
    rng = np.random.default_rng(7)
    ids = rng.integers(0, cfg.vocab, (batch, seq + 1), dtype=np.int64)
    tok = nb.Tensor.from_torch(torch.from_numpy(np.ascontiguousarray(ids[:, :-1])).to(tdev))
    tgt = nb.Tensor.from_torch(torch.from_numpy(np.ascontiguousarray(ids[:, 1:])).to(tdev))
    if mesh is not None:
        tok, tgt = tok.shard(mesh, (None, None)), tgt.shard(mesh, (None, None))

    @nb.compile(cuda_graph=_graph(), donate_argnums=(0, 1))
    def step(lora, state, tok, tgt):
        loss, grads = nb.value_and_grad(lambda a: T.loss_fn(params, tok, tgt, cfg, None, a), create_graph=False)(lora)
        lora, state = nn.adamw_update(lora, grads, state, lr=1e-4, weight_decay=0.0, realize=False)
        return loss, lora, state

    box = [lora, state]
    _COMPILED.append(step)

    def one():
        loss, box[0], box[1] = step(box[0], box[1], tok, tgt)
        return loss

    ms, loss = _timed(one, warmup, steps, world, tdev)
    return {"config": "lora", "tp": world, "layers": layers, "batch": batch, "seq": seq, "rank": 16, "ms_per_step": ms,
            "tokens_per_s": batch * seq / (ms / 1e3), "loss": float(loss.item())}


def run_cpu_mlp(steps: int = 100) -> dict:
    import time

    import nabla_b200 as nb
    from nabla_b200 import nn

    rng = np.random.default_rng(0)
    x_np = rng.uniform(0.0, 1.0, (512, 64)).astype(np.float32)
    y_np = np.sin(2 * np.pi * x_np.mean(axis=1, keepdims=True)).astype(np.float32)
    sizes = [64, 256, 256, 256, 1]
    with nb.default_device(nb.CPU()):
        x, y = nb.constant(x_np), nb.constant(y_np)
        params = []
        for fi, fo in zip(sizes[:-1], sizes[1:]):
            params.append({"w": nb.constant(rng.normal(0.0, fi ** -0.5, (fi, fo)).astype(np.float32)),
                           "b": nb.constant(np.zeros((1, fo), np.float32))})
        state = nn.adamw_init(params)

        def loss_fn(ps):
            h = x
            for i, p in enumerate(ps):
                h = h @ p["w"] + p["b"]
                if i + 1 < len(ps):
                    h = nb.relu(h)
            d = h - y
            return nb.mean(d * d)

        @nb.compile
        def step(params, state):
            loss, grads = nb.value_and_grad(loss_fn)(params)
            params, state = nn.adamw_update(params, grads, state, lr=1e-3, weight_decay=0.0, realize=False)
            return loss, params, state

        first = None
        t0 = time.perf_counter()
        for i in range(steps):
            loss, params, state = step(params, state)
            if i == 0:
                first = float(loss.item())
                t1 = time.perf_counter()          # the first call records the graph
        last = float(loss.item())
        t2 = time.perf_counter()
    return {"config": "cpu_mlp", "steps": steps, "first_loss": first, "final_loss": last,
            "steps_per_s_after_first": (steps - 1) / (t2 - t1), "total_s": t2 - t0}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", choices=["gpipe", "pp_dp", "lora", "cpu_mlp"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--small", action="store_true", help="reduced sizes (functional check, not a benchmark number)")
    ap.add_argument("--dump-plan", default=None, help="rank 0 writes the recorded schedule (one line per step) to this file")
    args = ap.parse_args()

    if args.config == "cpu_mlp":
        print(json.dumps(run_cpu_mlp(100 if args.steps == 5 else args.steps)), flush=True)
        return

    import nabla_b200 as nb
    from nabla_b200 import native
    from nabla_b200.parallel import init_distributed

    rank, world = init_distributed()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = nb.Accelerator(local)
    tdev = dev.to_torch()
    with nb.default_device(dev):
        if args.config == "gpipe":
            kw = dict(dim=512, micro=4, batch=16) if args.small else {}
            out = run_gpipe(nb, rank, world, dev, tdev, args.steps, args.warmup, **kw)
        elif args.config == "pp_dp":
            kw = dict(dim=512, micro=4, batch=16) if args.small else {}
            out = run_pp_dp(nb, rank, world, dev, tdev, args.steps, args.warmup, **kw)
        else:
            kw = dict(layers=2, batch=4, seq=256) if args.small else {}
            out = run_lora(nb, rank, world, dev, tdev, args.steps, args.warmup, **kw)
        native.check_status()
    out.update(n_gpus=world, steps=args.steps, warmup=args.warmup, small=bool(args.small), cuda_graph=_graph())
    if rank == 0:
        print(json.dumps(out), flush=True)
        if args.dump_plan:
            with open(args.dump_plan, "w") as f:
                for c in _COMPILED:
                    c.dump_plan(file=f)
    finish()


if __name__ == "__main__":
    main()
