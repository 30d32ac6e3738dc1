"""grad / value_and_grad / vjp / jvp / jacobians / Hessians / vmap / compile
(reference: tests/unit/test_vjp.py, test_jvp.py, test_jacobians.py, test_hessian_*.py,
test_transforms_composition.py, test_compile*.py)."""
import numpy as np
import pytest
import torch

import nabla_b200 as nb
from common import T, close, rand


def test_grad_argnums_and_pytrees():
    a, b = rand(3, 4, seed=1), rand(4, seed=2)
    f = lambda p, s: nb.reduce_sum(nb.tanh(p["w"] @ p["v"]) * s)  # noqa: E731
    at, bt = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    (torch.tanh(at @ bt) * 2.0).sum().backward()
    g = nb.grad(f)({"w": T(a), "v": T(b)}, 2.0)
    close(g["w"], at.grad, rtol=1e-5, atol=1e-6)
    close(g["v"], bt.grad, rtol=1e-5, atol=1e-6)
    g0, g1 = nb.grad(lambda x, y: nb.reduce_sum(x * y * y), argnums=(0, 1))(T(a), T(a))
    close(g0, a * a)
    close(g1, 2 * a * a)
    v, g = nb.value_and_grad(lambda x: nb.mean(x * x))(T(a))
    assert abs(v.item() - (a * a).mean().item()) < 1e-6
    # a non-scalar output is pulled back with ones, i.e. the gradient of its sum (reference behaviour)
    close(nb.grad(lambda x: x * x * 2.0)(T(a)), 4.0 * a)


def test_has_aux():
    (v, aux), g = nb.value_and_grad(lambda x: (nb.reduce_sum(x * x), {"n": x.shape}), has_aux=True)(T(rand(3)))
    assert aux["n"] == [3]
    close(g, 2 * rand(3))


def test_vjp_jvp_match_torch():
    x = rand(5, seed=3)
    out, pull = nb.vjp(lambda t: nb.sin(t) * nb.exp(t), T(x))
    (g,) = pull(nb.ones_like(out))
    close(g, (torch.cos(x) + torch.sin(x)) * torch.exp(x), rtol=1e-5, atol=1e-6)
    out, tan = nb.jvp(lambda t: nb.sin(t) * nb.exp(t), (T(x),), (nb.ones_like(T(x)),))
    close(tan, (torch.cos(x) + torch.sin(x)) * torch.exp(x), rtol=1e-5, atol=1e-6)


def test_jacobians_and_hessians():
    x = T(torch.tensor([1.0, 2.0]))
    f = lambda v: nb.reduce_sum(v * v * v) + v[0] * v[1] * 2.0  # noqa: E731
    H = torch.tensor([[6.0, 2.0], [2.0, 12.0]])
    for h in (nb.jacrev(nb.grad(f)), nb.jacfwd(nb.grad(f)), nb.jacfwd(nb.jacrev(f)), nb.jacrev(nb.jacfwd(f))):
        close(h(x), H, rtol=1e-5, atol=1e-5)
    A = rand(3, 2, seed=4)
    g = lambda v: nb.tanh(T(A) @ v)  # noqa: E731
    J = torch.autograd.functional.jacobian(lambda v: torch.tanh(A @ v), torch.tensor([1.0, 2.0]))
    close(nb.jacrev(g)(x), J, rtol=1e-5, atol=1e-6)
    close(nb.jacfwd(g)(x), J, rtol=1e-5, atol=1e-6)
    # matrix input: jacobian shape (*out, *in)
    W = rand(2, 3, seed=5)
    Jm = nb.jacrev(lambda w: nb.reduce_sum(w * w, axis=1))(T(W))
    assert tuple(int(d) for d in Jm.shape) == (2, 2, 3)


def test_third_derivative_by_nesting():
    f = lambda x: x * x * x * x  # noqa: E731
    d3 = nb.grad(lambda x: nb.reduce_sum(nb.grad(lambda y: nb.reduce_sum(nb.grad(lambda z: nb.reduce_sum(f(z)))(y)))(x)))
    close(d3(T(torch.tensor([2.0]))), torch.tensor([48.0]))


def test_vmap_in_axes_out_axes_nested_and_pytrees():
    A, x = rand(5, 3, 4, seed=1), rand(5, 4, seed=2)
    close(nb.vmap(lambda a, v: a @ v)(T(A), T(x)), torch.einsum("bij,bj->bi", A, x), rtol=1e-5, atol=1e-5)
    close(nb.vmap(lambda a, v: a @ v, in_axes=(0, None))(T(A), T(x[0])), A @ x[0], rtol=1e-5, atol=1e-5)
    close(nb.vmap(lambda a, v: a @ v, in_axes=(None, 0), out_axes=1)(T(A[0]), T(x)), (x @ A[0].T).T, rtol=1e-5, atol=1e-5)
    nested = nb.vmap(nb.vmap(lambda a, b: nb.reduce_sum(a * b)))
    close(nested(T(A[:, :, :2]), T(A[:, :, 2:])), (A[:, :, :2] * A[:, :, 2:]).sum(-1), rtol=1e-5, atol=1e-5)
    tree = nb.vmap(lambda p: p["a"] * 2.0 + p["b"][0])({"a": T(x), "b": [T(x)]})
    close(tree, 3 * x)

    @nb.vmap
    def dec(v):
        return nb.softmax(v, axis=0)

    close(dec(T(x)), torch.softmax(x, -1), rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        nb.vmap(lambda a, b: a + b)(T(A), T(rand(4, 3, 4)))
    close(nb.vmap(lambda v: nb.constant(1.0) + 0.0 * nb.reduce_sum(v), axis_size=5)(T(x)), torch.ones(5))


def test_vmap_of_grad_per_example_gradients():
    w, xs, ys = rand(4, seed=1), rand(6, 4, seed=2), rand(6, seed=3)
    loss = lambda ww, x, y: (nb.reduce_sum(ww * x) - y) ** 2.0  # noqa: E731
    per = nb.vmap(nb.grad(loss), in_axes=(None, 0, 0))(T(w), T(xs), T(ys))
    ref = 2 * ((xs @ w) - ys).unsqueeze(1) * xs
    close(per, ref, rtol=1e-5, atol=1e-5)


def test_compile_cache_and_stats():
    calls = {"n": 0}

    @nb.compile
    def f(a, b):
        calls["n"] += 1
        return nb.relu(a @ b) + 1.0

    a, b = rand(4, 5, seed=1), rand(5, 3, seed=2)
    for i in range(4):
        close(f(T(a + i), T(b)), torch.relu((a + i) @ b) + 1.0, rtol=1e-5, atol=1e-5)
    assert calls["n"] == 1 and f.stats.misses == 1 and f.stats.hits == 3
    f(T(rand(7, 5)), T(b))
    assert calls["n"] == 2 and f.stats.misses == 2
    assert "hits=3" in repr(f.stats)


def test_compile_dynamic_dims_share_one_entry():
    f = nb.compile(lambda x: nb.reduce_sum(x * 2.0, axis=0), dynamic_dims={0: {0: "batch"}})
    for n in (3, 5, 3, 8):
        x = rand(n, 4, seed=n)
        close(f(T(x)), (x * 2).sum(0), rtol=1e-5, atol=1e-5)
    assert f.stats.misses == 1 and f.stats.hits == 3 and len(f._cache) == 1


def test_compile_training_step_with_optimizer_state_and_module():
    from nabla_b200 import nn

    torch.manual_seed(0)
    x, y = rand(32, 4, seed=1), rand(32, 1, seed=2)

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(4, 8)
            self.b = nn.Linear(8, 1)

        def forward(self, t):
            return self.b(nb.relu(self.a(t)))

    model = MLP()
    state = nn.adamw_init(model)

    @nb.compile
    def step(m, s, xx, yy):
        l, g = nb.value_and_grad(lambda mm: nn.mse_loss(mm(xx), yy))(m)
        m, s = nn.adamw_update(m, g, s, lr=1e-2)
        return l, m, s

    losses = []
    for _ in range(25):
        l, model, state = step(model, state, T(x), T(y))
        losses.append(l.item())
    assert losses[-1] < losses[0] * 0.7
    assert step.stats.misses == 1 and step.stats.hits == 24
    assert isinstance(model, MLP) and abs(state["step"].item() - 25.0) < 1e-6


def test_compile_random_ops_draw_fresh_numbers():
    f = nb.compile(lambda x: x + nb.uniform((4,)))
    a = f(T(torch.zeros(4))).to_numpy()
    b = f(T(torch.zeros(4))).to_numpy()
    assert not np.allclose(a, b)


def test_compile_sharded(mesh_2x4):
    x, w = rand(8, 16, seed=1), rand(16, 8, seed=2)
    f = nb.compile(lambda a, b: nb.exp((a @ b) * 0.01))
    xs, ws = nb.shard(T(x), mesh_2x4, nb.P("dp", "tp")), nb.shard(T(w), mesh_2x4, nb.P("tp", None))
    for _ in range(2):
        out = f(xs, ws)
    assert out.sharding is not None and f.stats.hits == 1
    close(out, torch.exp((x @ w) * 0.01), rtol=1e-4, atol=1e-5)


def test_backward_api_accumulates_grad():
    w = T(rand(3, seed=1))
    w.requires_grad = True
    loss = nb.reduce_sum(w * w)
    loss.backward()
    close(w.grad, 2 * rand(3, seed=1))
    nb.reduce_sum(w * 3.0).backward()
    close(w.grad, 2 * rand(3, seed=1) + 3.0)
    with pytest.raises(ValueError):
        (w * 2.0).backward()


# ---------------------------------------------------------------- compile: data-dependent control flow, RNG, dynamic dims
def test_compiled_cond_follows_its_predicate():
    """A compiled `cond` decides again on every call (reference: ops.cond lowered into the graph,
    nabla/ops/control_flow.py:302-307); the branch taken while tracing is not baked in."""
    g = nb.compile(lambda a: nb.cond(nb.reduce_sum(a) > 0, lambda x: x * 2, lambda x: x - 1, a))
    pos = nb.constant(np.array([1., 2., 3.], dtype=np.float32))
    neg = nb.constant(np.array([-1., -2., -3.], dtype=np.float32))
    assert np.allclose(g(pos).to_numpy(), [2, 4, 6])
    assert np.allclose(g(neg).to_numpy(), [-2, -3, -4])
    assert np.allclose(g(pos).to_numpy(), [2, 4, 6])
    assert g.stats.misses == 1 and g.stats.retraces == 0


def test_compiled_cond_closure_and_select_lowering():
    """Branches may close over tensors computed earlier in the traced function; with
    cuda_graph=True the same function lowers to both branches + `where` and gives the same values."""
    def f(a, b):
        s = a + b
        return nb.cond(nb.reduce_sum(a) > 0, lambda x: x * s, lambda x: x - s, a)
    a1 = nb.constant(np.array([1., 2.], dtype=np.float32))
    a2 = nb.constant(np.array([-1., -2.], dtype=np.float32))
    b = nb.constant(np.array([10., 20.], dtype=np.float32))
    for kw in ({}, {"cuda_graph": True}):
        g = nb.compile(f, **kw)
        assert np.allclose(g(a1, b).to_numpy(), [11, 44])
        assert np.allclose(g(a2, b).to_numpy(), [-10, -20])
        assert np.allclose(g(a1, b).to_numpy(), [11, 44])


def test_compiled_cond_rejects_mismatched_branches():
    g = nb.compile(lambda a: nb.cond(nb.reduce_sum(a) > 0, lambda x: x * 2, lambda x: nb.reduce_sum(x), a))
    with pytest.raises(ValueError):
        g(nb.constant(np.ones(3, dtype=np.float32)))


def test_compiled_while_loop_trip_count_follows_the_input():
    def f(x):
        return nb.while_loop(lambda v, i: nb.reduce_sum(v) < 100.0, lambda v, i: (v * 2, i + 1),
                             (x, nb.constant(np.float32(0))))
    h = nb.compile(f)
    for start, trips in ((1., 6), (10., 3), (40., 1), (200., 0), (1., 6)):
        v, i = h(nb.constant(np.array([start, start], dtype=np.float32)))
        assert int(i.to_numpy()) == trips
        assert np.allclose(v.to_numpy(), start * 2 ** trips)
    assert h.stats.misses == 1 and h.stats.retraces == 0


def test_compiled_dropout_draws_a_new_mask_on_every_replay():
    nb.seed(5)
    g = nb.compile(lambda x: nb.nn.functional.dropout(x, p=0.5, training=True))
    x = nb.constant(np.ones((64, 64), dtype=np.float32))
    a, b, c = (g(x).to_numpy() for _ in range(3))
    assert g.stats.hits == 2
    assert (a != b).any() and (b != c).any()
    assert set(np.unique(a)) <= {0.0, 2.0}


def test_dynamic_dims_serves_new_sizes_without_rerunning_python():
    """dynamic_dims: four sizes, the Python function runs for the first one only (plus one
    shape-only probe); shape-valued arguments follow the size (reference: one executable with
    symbolic dims, nabla/transforms/compile.py:276-301, tests/unit/test_compile.py:46)."""
    calls = {"n": 0}

    def f(x, w):
        calls["n"] += 1
        b = int(x.shape[0])
        y = nb.reshape(nb.matmul(x, w), (b * 2, 4))
        z = nb.concatenate([y, nb.zeros((b, 4), dtype=y.dtype, device=y.device)], axis=0)
        return nb.reduce_sum(nb.relu(z), axis=0), z[: b // 2]

    g = nb.compile(f, dynamic_dims={0: {0: "batch"}})
    rng = np.random.default_rng(0)
    w = rng.standard_normal((6, 8)).astype(np.float32)
    for b in (4, 8, 2, 16, 8):
        x = rng.standard_normal((b, 6)).astype(np.float32)
        out, head = g(nb.constant(x), nb.constant(w))
        z = np.concatenate([(x @ w).reshape(b * 2, 4), np.zeros((b, 4), np.float32)], 0)
        assert np.allclose(out.to_numpy(), np.maximum(z, 0).sum(0), atol=1e-4)
        assert np.allclose(head.to_numpy(), z[: b // 2], atol=1e-5)
    assert calls["n"] == 3                      # the real trace and two shape-only probes (2x and 3x the size)
    assert g.stats.retraces == 0 and g.stats.respecialisations == 3 and g.stats.misses == 1


def test_dynamic_dims_falls_back_when_a_size_is_not_affine():
    """b // 2 recorded at b = 4 and probed at b = 8 has slope 1/2: an odd size has no integer value
    on that line, so that size is traced on its own and counted as a retrace."""
    g = nb.compile(lambda x: x[: int(x.shape[0]) // 2] * 2.0, dynamic_dims={0: {0: "n"}})
    for n in (4, 6, 5):
        x = np.arange(n, dtype=np.float32)
        assert np.allclose(g(nb.constant(x)).to_numpy(), x[: n // 2] * 2)
    assert g.stats.respecialisations == 1 and g.stats.retraces == 1


def test_dynamic_dims_records_per_size_when_a_value_is_computed_from_the_size_in_python():
    """Only integers that move on a line with the size are re-evaluated. A float (``mean`` over the
    dynamic axis scales by ``1.0 / n``), a constant tensor built from the size, or an integer that is
    not linear in it (checked with a third, shape-only recording) make the function one that is
    recorded per size: slower, never wrong."""
    rng = np.random.default_rng(1)
    g = nb.compile(lambda x: nb.reduce_sum(x * x, axis=0) * (1.0 / int(x.shape[0])), dynamic_dims={0: {0: "n"}})
    for n in (4, 8, 6, 8):
        x = rng.standard_normal((n, 3)).astype(np.float32)
        assert np.allclose(g(nb.constant(x)).to_numpy(), (x * x).mean(0), atol=1e-5)
    assert g.stats.respecialisations == 0 and g.stats.retraces == 2
    # `mean` itself divides by an integer count, which follows the size: no second run of Python
    g = nb.compile(nb.value_and_grad(lambda x: nb.mean(nb.reduce_sum(x * x, axis=1))), dynamic_dims={0: {0: "n"}})
    for n in (4, 8, 6, 10):
        x = rng.standard_normal((n, 3)).astype(np.float32)
        v, gr = g(nb.constant(x))
        assert np.allclose(v.to_numpy(), (x * x).sum(1).mean(), atol=1e-5) and np.allclose(gr.to_numpy(), 2 * x / n, atol=1e-5)
    assert g.stats.respecialisations == 3 and g.stats.retraces == 0

    def last_and_first(x):
        n = int(x.shape[0])
        return nb.gather(x, nb.constant(np.array([n - 1, 0], dtype=np.int32)), axis=0)

    g = nb.compile(last_and_first, dynamic_dims={0: {0: "n"}})
    for n in (4, 8, 5):
        x = rng.standard_normal((n, 2)).astype(np.float32)
        assert np.allclose(g(nb.constant(x)).to_numpy(), x[[n - 1, 0]])
    assert g.stats.respecialisations == 0

    g = nb.compile(lambda x: x[: (int(x.shape[0]) * int(x.shape[0])) // 8 + 1], dynamic_dims={0: {0: "n"}})
    for n in (4, 8, 6):                                   # n*n // 8 + 1 = 3, 9 -> 8, 5: not a line
        x = rng.standard_normal((n,)).astype(np.float32)
        assert np.allclose(g(nb.constant(x)).to_numpy(), x[: n * n // 8 + 1])
    assert g.stats.respecialisations == 0

    g = nb.compile(lambda x, w: nb.reduce_sum(nb.relu(x @ w), axis=1), dynamic_dims={0: {0: "n"}})
    w = rng.standard_normal((3, 5)).astype(np.float32)
    for n in (4, 8, 6, 10):                               # the usual case still needs no second run of Python
        x = rng.standard_normal((n, 3)).astype(np.float32)
        assert np.allclose(g(nb.constant(x), nb.constant(w)).to_numpy(), np.maximum(x @ w, 0).sum(1), atol=1e-5)
    assert g.stats.respecialisations == 3 and g.stats.retraces == 0


def test_reverse_mode_through_cond_and_while_loop_recorded_by_compile():
    """The recorded node of a ``cond`` / ``while_loop`` has a backward node: at replay it runs the
    taken branch (the loop) of THAT call again with autograd on. Gradients follow the data of each
    call, also for tensors the branch functions close over; forward mode says it is not available."""
    w = nb.constant(np.array([0.5, -1.0], np.float32))
    xs = nb.constant(np.ones((3, 2), np.float32))

    def f_cond(c, xs):
        p = nb.greater(nb.reduce_sum(c), 0.0)
        r = nb.cond(p, lambda a, b: nb.tanh(a) * w + nb.reduce_sum(b, axis=0), lambda a, b: a * 2.0 + w, c, xs)
        return nb.reduce_sum(r)

    def f_while(c, xs):
        i, a = nb.while_loop(lambda s: nb.less(s[0], nb.reduce_sum(nb.abs(c))), lambda s: (s[0] + 1.0, nb.tanh(s[1]) * w),
                             (nb.constant(np.float32(0.0)), c))
        return nb.reduce_sum(a)

    for f in (f_cond, f_while):
        g = nb.compile(nb.value_and_grad(f))
        for vals in ([1.0, 2.0], [-3.0, 0.5], [0.2, 0.3], [1.0, 2.0]):
            c = np.array(vals, np.float32)
            v_ref, g_ref = nb.value_and_grad(f)(nb.constant(c), xs)
            v, gr = g(nb.constant(c), xs)
            assert np.allclose(v.to_numpy(), v_ref.to_numpy(), atol=1e-5) and np.allclose(gr.to_numpy(), g_ref.to_numpy(), atol=1e-5)
        assert g.stats.misses == 1 and g.stats.hits == 3

    def f_w(c, w2):
        p = nb.greater(nb.reduce_sum(c), 0.0)
        return nb.reduce_sum(nb.cond(p, lambda a: nb.tanh(a) * w2, lambda a: a * 2.0 + w2 * w2, c))

    g = nb.compile(nb.grad(f_w, argnums=(0, 1)))
    for vals in ([1.0, 2.0], [-3.0, 0.5]):
        c = np.array(vals, np.float32)
        for a, b in zip(g(nb.constant(c), w), nb.grad(f_w, argnums=(0, 1))(nb.constant(c), w)):
            assert np.allclose(a.to_numpy(), b.to_numpy(), atol=1e-5)
    with pytest.raises(NotImplementedError, match="forward mode"):
        nb.compile(nb.jacfwd(f_cond, argnums=0))(nb.constant(np.array([1.0, 2.0], np.float32)), xs)


def test_cond_and_while_loop_under_vmap_with_a_predicate_per_example():
    """vmap over examples that take different branches / different numbers of iterations: ``cond``
    evaluates both branches and selects, ``while_loop`` runs while any example wants to and freezes
    the others; values and gradients equal the per-example runs."""
    C = np.array([[0.5, 0.2], [-1.5, 1.0], [3.0, 0.4]], np.float32)

    def f_cond(c):
        p = nb.greater(nb.reduce_sum(c), 0.0)
        return nb.reduce_sum(nb.cond(p, lambda a: nb.tanh(a) * 3.0, lambda a: a * a, c))

    def f_while(c):
        i, a = nb.while_loop(lambda s: nb.less(s[0], nb.reduce_sum(nb.abs(c))), lambda s: (s[0] + 1.0, nb.tanh(s[1]) + 0.1),
                             (nb.constant(np.float32(0.0)), c))
        return nb.reduce_sum(a)

    for f in (f_cond, f_while):
        ref = np.array([f(nb.constant(C[i])).to_numpy() for i in range(3)])
        g_ref = np.stack([nb.grad(f)(nb.constant(C[i])).to_numpy() for i in range(3)])
        assert np.allclose(nb.vmap(f)(nb.constant(C)).to_numpy(), ref, atol=1e-5)
        assert np.allclose(nb.vmap(nb.grad(f))(nb.constant(C)).to_numpy(), g_ref, atol=1e-5)
