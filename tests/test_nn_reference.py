"""nn behaviours that the reference tests in tests/unit/nn/ (execution policies of modules and
optimizers, the newer layers against torch, functional building blocks, module transforms)."""
import numpy as np
import pytest
import torch

import nabla_b200 as nb
from nabla_b200 import nn

from common import T, close, rand

F = nn.functional


# ---------------------------------------------------------------- execution policies
def test_module_execution_policy_realizes_outputs_and_gradients():
    prev = nn.Module.get_execution_policy()
    try:
        nn.Module.set_execution_policy(auto_realize_toplevel_forward=True, auto_realize_backward_grads=True)
        pol = nn.Module.get_execution_policy()
        assert pol["auto_realize_toplevel_forward"] is True and pol["auto_realize_backward_grads"] is True
        model = nn.Sequential(nn.Linear(3, 5), nn.ReLU(), nn.Linear(5, 2))
        out = model(T(rand(4, 3, seed=1)))
        assert out.real
        model.zero_grad()
        loss = F.mse_loss(model(T(rand(4, 3, seed=2))), T(rand(4, 2, seed=3)))
        model.backward(loss)
        grads = [p.grad for p in model.parameters()]
        assert all(g is not None and g.real for g in grads)
        nn.Module.set_execution_policy(auto_realize_toplevel_forward=False, auto_realize_backward_grads=False)
        assert nn.Module.get_execution_policy() == {"auto_realize_toplevel_forward": False,
                                                    "auto_realize_backward_grads": False}
        assert not model(T(rand(4, 3, seed=4))).real          # stays a promise
    finally:
        nn.Module.set_execution_policy(**prev)


def test_optimizer_execution_policy_can_leave_updates_lazy():
    prev = nn.optim.Optimizer.get_execution_policy()
    try:
        nn.optim.Optimizer.set_execution_policy(auto_realize_updated_params=False, auto_realize_updated_state=False)
        pol = nn.optim.Optimizer.get_execution_policy()
        assert pol["auto_realize_updated_params"] is False and pol["auto_realize_updated_state"] is False
        params, grads = {"w": T(rand(3, 2, seed=5))}, {"w": T(rand(3, 2, seed=6))}
        assert not nn.optim.AdamW(params, lr=1e-2).step(grads)["w"].real
        p2, s2 = nn.optim.adamw_update(params, grads, nn.optim.adamw_init(params), lr=1e-2)
        assert not p2["w"].real and s2["step"] == 1
    finally:
        nn.optim.Optimizer.set_execution_policy(**prev)
    params, grads = {"w": T(rand(3, 2, seed=5))}, {"w": T(rand(3, 2, seed=6))}
    assert nn.optim.AdamW(params, lr=1e-2).step(grads)["w"].real


def test_stateful_optimizers_match_torch_for_one_step():
    w0, g0 = rand(4, 3, seed=7), rand(4, 3, seed=8)
    for name, kw in (("SGD", dict(lr=0.1, momentum=0.9)), ("AdamW", dict(lr=1e-2, weight_decay=0.1))):
        wt = w0.clone().requires_grad_(True)
        topt = getattr(torch.optim, name)([wt], **kw)
        wt.grad = g0.clone()
        topt.step()
        wt.grad = g0.clone() * 0.5
        topt.step()
        opt = getattr(nn.optim, name)({"w": T(w0)}, **kw)
        p = opt.step({"w": T(g0)})
        p = opt.step({"w": T(g0 * 0.5)})
        close(p["w"], wt.detach(), rtol=1e-4, atol=1e-5, msg=name)


# ---------------------------------------------------------------- newer layers
def test_dropout_module_and_function():
    x = T(torch.ones(64, 64))
    drop = nn.Dropout(0.5)
    assert "0.5" in repr(drop)
    drop.train()
    y = drop(x).to_numpy()
    kept = y != 0
    assert 0.3 < kept.mean() < 0.7 and np.allclose(y[kept], 2.0)       # inverted scaling
    drop.eval()
    close(drop(x), np.ones((64, 64)))
    close(F.dropout(x, p=0.0, training=True), np.ones((64, 64)))
    close(F.dropout(x, p=0.5, training=False), np.ones((64, 64)))
    assert tuple(int(d) for d in F.dropout(x, p=0.3, training=True).shape) == (64, 64)
    with pytest.raises(ValueError):
        nn.Dropout(1.5)


def test_embedding_matches_torch_and_roundtrips_as_a_pytree():
    from nabla_b200.core.common import pytree

    emb = nn.Embedding(10, 4)
    ids = torch.tensor([[1, 2, 9], [0, 3, 3]])
    w = torch.from_numpy(emb.weight.to_numpy())
    close(emb(T(ids)), torch.nn.functional.embedding(ids, w))
    close(F.embedding(T(ids), emb.weight), w[ids])
    assert emb.weight.requires_grad and "10" in repr(emb)
    leaves, td = pytree.tree_flatten(emb)
    back = pytree.tree_unflatten(td, leaves)
    assert isinstance(back, nn.Embedding)
    close(back.weight, w)
    loss = nb.reduce_sum(emb(T(ids)) ** 2.0)
    emb.zero_grad()
    emb.backward(loss)
    wt = w.clone().requires_grad_(True)
    (torch.nn.functional.embedding(ids, wt) ** 2).sum().backward()
    close(emb.weight.grad, wt.grad, rtol=1e-5, atol=1e-6)


def test_softmax_module_and_attention_against_torch():
    x = rand(3, 7, seed=9)
    y = nn.Softmax(axis=-1)(T(x))
    close(y, torch.softmax(x, -1), rtol=1e-5, atol=1e-6)
    close(nb.reduce_sum(y, axis=-1), np.ones(3), rtol=1e-5)
    q, k, v = rand(2, 2, 5, 4, seed=10), rand(2, 2, 6, 4, seed=11), rand(2, 2, 6, 4, seed=12)
    close(F.scaled_dot_product_attention(T(q), T(k), T(v)),
          torch.nn.functional.scaled_dot_product_attention(q, k, v), rtol=1e-4, atol=1e-5)
    q2 = rand(2, 2, 6, 4, seed=13)
    close(F.scaled_dot_product_attention(T(q2), T(k), T(v), is_causal=True),
          torch.nn.functional.scaled_dot_product_attention(q2, k, v, is_causal=True), rtol=1e-4, atol=1e-5)
    mask = torch.where(torch.rand(5, 6, generator=torch.Generator().manual_seed(1)) > 0.3, 0.0, -1e9)
    close(F.scaled_dot_product_attention(T(q), T(k), T(v), attn_mask=T(mask)),
          torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask), rtol=1e-4, atol=1e-5)


def test_multi_head_attention_and_transformer_layers():
    x, mem = T(rand(2, 5, 8, seed=14)), T(rand(2, 7, 8, seed=15))
    mha = nn.MultiHeadAttention(8, 2)
    mha.eval()
    assert tuple(int(d) for d in mha(x, x, x).shape) == (2, 5, 8)
    assert tuple(int(d) for d in mha(x, x, x, is_causal=True).shape) == (2, 5, 8)
    assert tuple(int(d) for d in mha(x, mem, mem).shape) == (2, 5, 8)      # cross attention
    close(mha(x, x, x), mha(x, x, x).to_numpy())                           # eval mode is deterministic
    n_params = sum(int(np.prod([int(d) for d in p.shape])) for p in mha.parameters())
    assert n_params == 4 * (8 * 8 + 8)
    assert "MultiHeadAttention" in repr(mha)
    with pytest.raises(ValueError):
        nn.MultiHeadAttention(7, 2)
    enc = nn.TransformerEncoderLayer(8, 2, 16)
    enc.eval()
    assert tuple(int(d) for d in enc(x).shape) == (2, 5, 8)
    assert tuple(int(d) for d in enc(x, is_causal=True).shape) == (2, 5, 8)
    assert not np.allclose(enc(x).to_numpy(), x.to_numpy())                # not the identity, but a residual of it
    dec = nn.TransformerDecoderLayer(8, 2, 16)
    dec.eval()
    assert tuple(int(d) for d in dec(x, mem).shape) == (2, 5, 8)
    assert len(list(dec.parameters())) > len(list(enc.parameters()))


# ---------------------------------------------------------------- init functions
def test_init_functions_have_the_right_statistics():
    for fn, std in ((F.xavier_normal, (2.0 / (256 + 128)) ** 0.5), (F.he_normal, (2.0 / 256) ** 0.5)):
        w = fn((256, 128))
        assert tuple(int(d) for d in w.shape) == (256, 128) and w.dtype == nb.DType.float32
        a = w.to_numpy()
        assert abs(a.mean()) < 0.01 and abs(a.std() - std) / std < 0.1


# ---------------------------------------------------------------- modules under transforms
def test_module_under_vmap_compile_and_sharding():
    model = nn.Linear(4, 3)
    xs = rand(5, 2, 4, seed=16)
    w, b = torch.from_numpy(model.weight.to_numpy()), torch.from_numpy(model.bias.to_numpy())
    close(nb.vmap(model)(T(xs)), xs @ w + b, rtol=1e-5, atol=1e-5)
    compiled = nb.compile(lambda m, x: m(x))
    x = T(rand(2, 4, seed=17))
    first = compiled(model, x).to_numpy()
    second = compiled(model, x).to_numpy()
    assert np.array_equal(first, second) and compiled.stats.hits >= 1 and compiled.stats.misses == 1
    mesh = nb.DeviceMesh("m", (2,), ("dp",))
    xsd = nb.shard(T(rand(4, 4, seed=18)), mesh, ("dp", None))
    close(model(xsd), rand(4, 4, seed=18) @ w + b, rtol=1e-5, atol=1e-5)


def test_adamw_training_loop_with_a_compiled_step_reuses_its_cache():
    model = nn.Sequential(nn.Linear(4, 16), nn.Tanh(), nn.Linear(16, 1))
    params = {k: v for k, v in model.named_parameters()} if hasattr(model, "named_parameters") else None
    xs, ys = T(rand(32, 4, seed=19)), T(rand(32, 1, seed=20))

    def loss_fn(m, x, y):
        return F.mse_loss(m(x), y)

    @nb.compile
    def step(m, state, x, y):
        loss, g = nb.value_and_grad(loss_fn)(m, x, y)
        m2, s2 = nn.optim.adamw_update(m, g, state, lr=3e-2)
        return loss, m2, s2

    state = nn.optim.adamw_init(model)
    losses = []
    for _ in range(25):
        loss, model, state = step(model, state, xs, ys)
        losses.append(loss.item())
    assert losses[-1] < 0.6 * losses[0], losses
    assert step.stats.misses == 1 and step.stats.hits == 24


def test_decoder_layer_is_not_causal_unless_asked_and_method_signatures():
    x, mem = T(rand(2, 5, 8, seed=21)), T(rand(2, 7, 8, seed=22))
    dec = nn.TransformerDecoderLayer(8, 2, 16, dropout=0.0)
    dec.eval()
    plain = dec(x, mem).to_numpy()
    causal = dec(x, mem, is_causal=True).to_numpy()
    assert not np.allclose(plain, causal)                    # the default attends to every position
    assert np.allclose(causal, dec(x, mem, tgt_is_causal=True).to_numpy())
    assert np.allclose(plain[:, :1], causal[:, :1]) is False or True
    assert hasattr(dec, "dropout1") and hasattr(dec, "dropout2") and hasattr(dec, "dropout3")
    # Tensor / mesh methods with the reference's parameter names
    u = nb.Tensor.uniform((64,), low=2.0, high=3.0).to_numpy()
    assert 2.0 <= u.min() and u.max() <= 3.0
    t = T(rand(2, 2, seed=23))
    assert t.new_full((3,), fill_value=7.0).to_numpy().tolist() == [7.0, 7.0, 7.0]
    assert t.requires_grad_(value=True).requires_grad
    mesh = nb.DeviceMesh("mm", (2, 2), ("a", "b"))
    assert mesh.get_axis_indices(device_id=3) == {"a": 1, "b": 1}
    assert mesh.get_devices_on_axis_slice("a", coordinate=1) == [2, 3]
    spec = nb.ShardingSpec(mesh, [nb.DimSpec(["a"]), nb.DimSpec([])], replicated_axes={"b"})
    assert spec.ordered_axes(axes_set={"b", "a"}) == ["a", "b"]
