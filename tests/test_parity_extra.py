"""Extra parity checks modelled on the reference's unit-test areas: Hessians through all four
jacfwd/jacrev compositions, a CNN toy training run, context-variable isolation across threads,
custom pytree nodes, slice assignment, and vmap over collectives."""
import threading

import numpy as np
import pytest
import torch

import nabla_b200 as nb


def _f(x):
    return nb.sum(nb.tanh(x) * x * x)


def _hess_ref(x_np):
    x = torch.tensor(x_np, dtype=torch.float64, requires_grad=True)
    return torch.autograd.functional.hessian(lambda t: (torch.tanh(t) * t * t).sum(), x).numpy()


@pytest.mark.parametrize("outer,inner", [("jacfwd", "jacrev"), ("jacrev", "jacrev"), ("jacfwd", "jacfwd"), ("jacrev", "jacfwd")])
def test_hessian_all_four_compositions(outer, inner):
    x_np = np.array([0.3, -1.2, 0.7], dtype=np.float32)
    h = getattr(nb, outer)(getattr(nb, inner)(_f))(nb.constant(x_np))
    np.testing.assert_allclose(h.to_numpy(), _hess_ref(x_np), rtol=2e-4, atol=2e-4)


def test_hessian_through_matmul():
    rng = np.random.default_rng(0)
    a_np = rng.normal(size=(3, 3)).astype(np.float32)
    a = nb.constant(a_np)

    def g(x):
        return nb.sum(nb.sin(a @ x) * x)

    x_np = rng.normal(size=(3,)).astype(np.float32)
    h = nb.jacfwd(nb.jacrev(g))(nb.constant(x_np))
    xt = torch.tensor(x_np, dtype=torch.float64)
    at = torch.tensor(a_np, dtype=torch.float64)
    ref = torch.autograd.functional.hessian(lambda t: (torch.sin(at @ t) * t).sum(), xt).numpy()
    np.testing.assert_allclose(h.to_numpy(), ref, rtol=5e-4, atol=5e-4)


def test_cnn_toy_training_loss_decreases():
    from nabla_b200 import nn

    rng = np.random.default_rng(0)
    x = nb.constant(rng.normal(size=(8, 8, 8, 3)).astype(np.float32))          # NHWC
    y = nb.constant(rng.integers(0, 4, (8,)))
    params = {"k": nb.constant((rng.normal(size=(3, 3, 3, 6)) * 0.2).astype(np.float32)),   # HWIO
              "w": nb.constant((rng.normal(size=(6 * 3 * 3, 4)) * 0.1).astype(np.float32)),
              "b": nb.constant(np.zeros((1, 4), np.float32))}

    def loss_fn(p):
        h = nb.relu(nb.conv2d(x, p["k"], stride=(1, 1), padding=(0, 0, 0, 0)))    # (8, 6, 6, 6)
        h = nb.max_pool2d(h, kernel_size=(2, 2), stride=(2, 2))                      # (8, 3, 3, 6)
        logits = nb.reshape(h, (8, -1)) @ p["w"] + p["b"]
        return nn.functional.cross_entropy_loss(logits, y)

    state = nn.adamw_init(params)
    losses = []
    for _ in range(25):
        loss, grads = nb.value_and_grad(loss_fn)(params)
        params, state = nn.adamw_update(params, grads, state, lr=2e-2, weight_decay=0.0)
        losses.append(loss.item())
    assert losses[-1] < 0.6 * losses[0], losses


def test_context_variables_are_isolated_between_threads():
    seen = {}

    def worker(name, dt):
        with nb.default_dtype(dt):
            barrier.wait()
            seen[name] = nb.ones((2,)).dtype

    barrier = threading.Barrier(2)
    ts = [threading.Thread(target=worker, args=("a", nb.DType.float32)),
          threading.Thread(target=worker, args=("b", nb.DType.float64))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert seen["a"] is nb.DType.float32 and seen["b"] is nb.DType.float64


def test_custom_pytree_node_roundtrip_and_grad():
    class Pair:
        def __init__(self, a, b):
            self.a, self.b = a, b

    nb.register_pytree_node(Pair, lambda p: ((p.a, p.b), None), lambda aux, ch: Pair(*ch))
    p = Pair(nb.constant(np.array([1.0, 2.0], np.float32)), nb.constant(np.array([3.0], np.float32)))
    leaves, td = nb.tree_flatten(p)
    q = nb.tree_unflatten(td, leaves)
    assert isinstance(q, Pair) and len(leaves) == 2
    g = nb.grad(lambda t: nb.sum(t.a * t.a) + nb.sum(t.b))(p)
    assert isinstance(g, Pair)
    np.testing.assert_allclose(g.a.to_numpy(), [2.0, 4.0])
    np.testing.assert_allclose(g.b.to_numpy(), [1.0])


def test_slice_assignment_and_gradient_through_slice_update():
    x = nb.constant(np.arange(12, dtype=np.float32).reshape(3, 4))
    x[1:3, 0:2] = nb.constant(np.full((2, 2), -1.0, np.float32))
    ref = np.arange(12, dtype=np.float32).reshape(3, 4)
    ref[1:3, 0:2] = -1.0
    np.testing.assert_allclose(x.to_numpy(), ref)

    def f(u):
        base = nb.zeros((3, 4))
        return nb.sum(nb.slice_update(base, u, (0, 1), (2, 2)) * 2.0)

    g = nb.grad(f)(nb.ones((2, 2)))
    np.testing.assert_allclose(g.to_numpy(), np.full((2, 2), 2.0))


def test_vmap_over_all_reduce_on_simulated_mesh():
    mesh = nb.DeviceMesh("m", (2,), ("x",))
    xs = nb.constant(np.arange(24, dtype=np.float32).reshape(3, 4, 2))

    def per_example(x):
        xs_ = x.shard(mesh, ("x", None))
        return nb.all_reduce(xs_ * 1.0, reduce_axes={"x"})

    out = nb.vmap(per_example)(xs)
    ref = xs.to_numpy()[:, :2] + xs.to_numpy()[:, 2:]
    np.testing.assert_allclose(out.to_numpy(), ref)
