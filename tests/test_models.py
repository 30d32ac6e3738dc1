"""Workload-level tests on CPU: the benchmark transformer (unsharded == dp x tp sharded, compiled
training step decreases the loss), the CPU MLP configuration, GPipe via vmap(spmd_axis_name) +
ppermute against a sequential oracle, PP x DP."""
import numpy as np
import pytest
import torch

import nabla_b200 as nb
from nabla_b200 import nn
from nabla_b200.models import mlp_pipeline as PP
from nabla_b200.models import transformer as TR
from common import T, close, rand


def _tiny_cfg():
    return TR.TransformerConfig(n_layers=2, d_model=32, n_heads=4, d_ff=64, vocab=48, max_seq=8, dtype=nb.DType.float32)


@pytest.mark.parametrize("fused", ["0", "1"])
def test_transformer_sharded_equals_unsharded(fused, monkeypatch):
    monkeypatch.setenv("NABLA_B200_FUSED", fused)
    cfg = _tiny_cfg()
    params = TR.init_params(cfg)
    rng = np.random.default_rng(0)
    tok, tgt = nb.constant(rng.integers(0, 48, (4, 8))), nb.constant(rng.integers(0, 48, (4, 8)))
    l, g = nb.value_and_grad(lambda p: TR.loss_fn(p, tok, tgt, cfg), create_graph=False)(params)
    mesh = nb.DeviceMesh("m", (2, 2), ("dp", "tp"))
    ps = TR.place_params(params, mesh, "tp")
    l2, g2 = nb.value_and_grad(lambda p: TR.loss_fn(p, tok.shard(mesh, ("dp", None)), tgt.shard(mesh, ("dp", None)), cfg),
                               create_graph=False)(ps)
    assert abs(l.item() - l2.item()) < 1e-5
    assert g2["layers"][0]["wqkv"].sharding.dim_specs[1].axes == ["tp"]
    for a, b in zip(nb.tree_leaves(g), nb.tree_leaves(g2)):
        close(b, a.to_numpy(), rtol=1e-4, atol=1e-5)
    # logits agree with a plain torch implementation of the same architecture
    logits = TR.forward(params, tok, cfg).to_numpy()
    close(TR.forward(ps, tok.shard(mesh, ("dp", None)), cfg), logits, rtol=1e-4, atol=1e-4)
    ref = TR.torch_reference_forward({k: v for k, v in params.items()}, torch.from_numpy(tok.to_numpy()), cfg)
    np.testing.assert_allclose(logits, ref.numpy(), rtol=1e-3, atol=1e-4)


def test_transformer_compiled_training_loss_decreases(monkeypatch):
    monkeypatch.setenv("NABLA_B200_FUSED", "1")
    cfg = _tiny_cfg()
    params = TR.init_params(cfg)
    state = nn.adamw_init(params)
    rng = np.random.default_rng(1)
    tok, tgt = nb.constant(rng.integers(0, 48, (4, 8))), nb.constant(rng.integers(0, 48, (4, 8)))

    @nb.compile
    def step(p, s, a, b):
        l, g = nb.value_and_grad(lambda q: TR.loss_fn(q, a, b, cfg), create_graph=False)(p)
        p, s = nn.adamw_update(p, g, s, lr=3e-3, realize=False)
        return l, p, s

    losses = []
    for _ in range(15):
        l, params, state = step(params, state, tok, tgt)
        losses.append(l.item())
    assert losses[-1] < 0.8 * losses[0] and step.stats.misses == 1


def test_baseline_cpu_mlp_config_trains():
    """CPU MLP configuration: fp32 MLP 64-256-256-256-1 relu, x (512,64) ~U(0,1), y = sin(2 pi mean x),
    MSE, Adam lr 1e-3 (shortened to 40 steps)."""
    rng = np.random.default_rng(0)
    xn = rng.random((512, 64), dtype=np.float32)
    x, y = nb.constant(xn), nb.constant(np.sin(2 * np.pi * xn.mean(1, keepdims=True)).astype(np.float32))
    dims = [64, 256, 256, 256, 1]
    params = [{"w": nb.gaussian((dims[i], dims[i + 1]), 0, 1 / np.sqrt(dims[i])), "b": nb.zeros((1, dims[i + 1]))} for i in range(4)]

    def fwd(p, h):
        for i, l in enumerate(p):
            h = h @ l["w"] + l["b"]
            if i < 3:
                h = nb.relu(h)
        return h

    state = nn.adamw_init(params)
    step = nb.compile(lambda p, s: (lambda lg: (lg[0],) + nn.adamw_update(p, lg[1], s, lr=1e-3))(
        nb.value_and_grad(lambda q: nn.mse_loss(fwd(q, x), y))(p)))
    first = last = None
    for i in range(40):
        l, params, state = step(params, state)
        first = l.item() if first is None else first
        last = l.item()
    assert last < first


def test_gpipe_matches_sequential_oracle():
    S, MB, B, D = 4, 6, 3, 8
    mesh = nb.DeviceMesh("pp", (S,), ("stage",))
    w, b = rand(S, D, D, seed=1, scale=0.5), rand(S, D, seed=2, scale=0.1)
    xs, ys = rand(MB, B, D, seed=3), rand(MB, B, D, seed=4)
    wt, bt = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    h = xs
    for s in range(S):
        h = torch.relu(h @ wt[s] + bt[s].unsqueeze(0))
    ref = ((h - ys) ** 2).mean()
    ref.backward()
    loss, (gw, gb) = nb.value_and_grad(lambda ww, bb: PP.gpipe_loss(ww, bb, T(xs), T(ys), mesh, "stage"), argnums=(0, 1))(
        PP.place_stage_params(T(w), mesh, "stage"), PP.place_stage_params(T(b), mesh, "stage"))
    assert abs(loss.item() - ref.item()) < 1e-5
    close(gw, wt.grad, rtol=1e-4, atol=1e-5)
    close(gb, bt.grad, rtol=1e-4, atol=1e-5)
    out = PP.gpipe_forward(PP.place_stage_params(T(w), mesh, "stage"), PP.place_stage_params(T(b), mesh, "stage"), T(xs), mesh, "stage")
    close(out, h.detach(), rtol=1e-4, atol=1e-5)


def test_pp_dp_matches_sequential_oracle():
    S, R, MB, B, D = 2, 2, 3, 4, 6
    mesh = nb.DeviceMesh("ppdp", (S, R), ("stage", "dp"))
    w, b = rand(S, D, D, seed=1, scale=0.5), rand(S, D, seed=2, scale=0.1)
    xs, ys = rand(MB, B, D, seed=3), rand(MB, B, D, seed=4)
    wt = w.clone().requires_grad_(True)
    h = xs
    for s in range(S):
        h = torch.relu(h @ wt[s] + b[s].unsqueeze(0))
    ((h - ys) ** 2).mean().backward()
    g = nb.grad(lambda ww: PP.gpipe_loss(ww, PP.place_stage_params(T(b), mesh, "stage"), T(xs), T(ys), mesh, "stage", dp_axis="dp"))(
        PP.place_stage_params(T(w), mesh, "stage"))
    close(g, wt.grad, rtol=1e-4, atol=1e-5)
