"""CPU tests of the sequence-parallel layout, reduce-scatter resharding, argument donation with
in-place optimizer updates, LoRA adapters on the transformer and the symmetric-arena allocator."""
import numpy as np
import pytest
import torch

import nabla_b200 as nb
from nabla_b200 import nn
from nabla_b200.models import transformer as T


def _tiny_cfg():
    return T.TransformerConfig(n_layers=2, d_model=32, n_heads=4, d_ff=64, vocab=48, max_seq=16, dtype=nb.DType.float32)


def _batch(cfg, b=4):
    rng = np.random.default_rng(0)
    return (nb.constant(rng.integers(0, cfg.vocab, (b, cfg.max_seq))), nb.constant(rng.integers(0, cfg.vocab, (b, cfg.max_seq))))


def _rel(ga, gb):
    out = []
    for a, b in zip(nb.tree_leaves(ga), nb.tree_leaves(gb)):
        ta, tb = torch.from_numpy(a.to_numpy()).float(), torch.from_numpy(b.to_numpy()).float()
        out.append(((ta - tb).norm() / (ta.norm() + 1e-9)).item())
    return max(out)


def test_sequence_parallel_matches_unsharded_and_uses_reduce_scatter():
    cfg = _tiny_cfg()
    nb.seed(0)
    params = T.init_params(cfg)
    tok, tgt = _batch(cfg)
    l0, g0 = nb.value_and_grad(lambda p: T.loss_fn(p, tok, tgt, cfg))(params)
    mesh = nb.DeviceMesh("m", (2, 2), ("dp", "tp"))
    ps = T.place_params(params, mesh, "tp")
    toks, tgts = tok.shard(mesh, ("dp", None)), tgt.shard(mesh, ("dp", None))
    sp = T.SeqParallel(mesh)
    from nabla_b200.core.graph import engine as E

    seen = []
    orig = E.run_node

    def spy(node):
        seen.append(node.op.name)
        return orig(node)

    E.run_node = spy
    try:
        l1, g1 = nb.value_and_grad(lambda p: T.loss_fn(p, toks, tgts, cfg, sp))(ps)
        err = _rel(g0, g1)
    finally:
        E.run_node = orig
    assert abs(l0.item() - l1.item()) < 1e-5 and err < 1e-4
    # row-parallel projections end in reduce-scatter, column-parallel ones start with all-gather
    assert seen.count("reduce_scatter") >= 2 * cfg.n_layers and seen.count("all_gather") >= 2 * cfg.n_layers


def test_partial_sum_to_split_dim_is_a_reduce_scatter():
    mesh = nb.DeviceMesh("m", (4,), ("x",))
    rng = np.random.default_rng(1)
    a = nb.constant(rng.normal(size=(8, 12)).astype(np.float32)).shard(mesh, (None, "x"))
    w = nb.constant(rng.normal(size=(12, 6)).astype(np.float32)).shard(mesh, ("x", None))
    y = a @ w                                   # pending partial sum over 'x'
    assert "x" in y._impl.sharding.partial_sum_axes
    z = y.shard(mesh, ("x", None))              # rows split over the same axis: one reduce-scatter
    assert z._impl.output_refs is not None and z._impl.output_refs.op.name == "reduce_scatter"
    np.testing.assert_allclose(z.to_numpy(), a.to_numpy() @ w.to_numpy(), rtol=1e-5, atol=1e-5)


def test_donated_arguments_are_updated_in_place_and_match(monkeypatch):
    monkeypatch.setenv("NABLA_B200_FUSED", "1")
    cfg = _tiny_cfg()
    tok, tgt = _batch(cfg)

    def run(donate):
        nb.seed(0)
        params = T.init_params(cfg)
        nb.realize_all(*nb.tensor_leaves(params))
        state = nn.adamw_init(params, state_dtype=nb.DType.float32)
        nb.realize_all(*nb.tensor_leaves(state))

        def step(params, state, tokens, targets):
            loss, grads = nb.value_and_grad(lambda p: T.loss_fn(p, tokens, targets, cfg), create_graph=False)(params)
            params, state = nn.adamw_update(params, grads, state, lr=1e-2, weight_decay=0.01, realize=False)
            return loss, params, state

        f = nb.compile(step, donate_argnums=(0, 1) if donate else ())
        first = params["layers"][0]["w1"]._impl._buffers[0].data_ptr()
        losses = []
        for _ in range(3):
            loss, params, state = f(params, state, tok, tgt)
            losses.append(loss.item())
        return losses, params["layers"][0]["w1"]._impl._buffers[0].data_ptr() == first

    plain, same_plain = run(False)
    donated, same_donated = run(True)
    np.testing.assert_allclose(plain, donated, rtol=1e-6)
    assert same_donated and not same_plain


def test_lora_adapter_gradients_sharded_match_unsharded():
    cfg = _tiny_cfg()
    nb.seed(0)
    params = T.init_params(cfg)
    lora = T.init_lora(params, cfg, rank=4)
    for L in lora:
        for k in ("qkv", "o"):
            L[k]["B"] = nb.gaussian(tuple(int(d) for d in L[k]["B"].shape), 0.0, 0.05)
    tok, tgt = _batch(cfg)
    l0, g0 = nb.value_and_grad(lambda a: T.loss_fn(params, tok, tgt, cfg, None, a))(lora)
    mesh = nb.DeviceMesh("m", (4,), ("tp",))
    ps = T.place_params(params, mesh, "tp")
    ls = [{"qkv": {"A": L["qkv"]["A"].shard(mesh, (None, None)), "B": L["qkv"]["B"].shard(mesh, (None, "tp"))},
           "o": {"A": L["o"]["A"].shard(mesh, ("tp", None)), "B": L["o"]["B"].shard(mesh, (None, None))}} for L in lora]
    l1, g1 = nb.value_and_grad(lambda a: T.loss_fn(ps, tok, tgt, cfg, None, a))(ls)
    assert abs(l0.item() - l1.item()) < 1e-5 and _rel(g0, g1) < 1e-4
    # the frozen base receives no gradient: only adapter leaves come back
    assert len(nb.tree_leaves(g1)) == 4 * cfg.n_layers


def test_arena_free_list_reuses_and_coalesces():
    from nabla_b200.parallel.symm import Arena

    ar = Arena.__new__(Arena)                 # allocator logic only: no device memory behind it
    ar.nbytes = 16 << 20
    ar.free_list = [[0, ar.nbytes]]
    ar.live = {}
    a = ar.alloc(3 << 20)
    b = ar.alloc(1)                           # rounded up to the 1 MiB granule
    c = ar.alloc(4 << 20)
    assert (a, b, c) == (0, 3 << 20, 4 << 20)
    ar.free(b)
    ar.free(a)                                # neighbours merge
    assert ar.free_list[0] == [0, 4 << 20]
    assert ar.alloc(4 << 20) == 0
    assert ar.alloc(9 << 20) is None          # only 8 MiB left
    ar.free(c)
    ar.free(0)
    assert ar.free_list == [[0, ar.nbytes]]
