"""Sharding model, factor propagation, communication ops (simulated meshes), deferred partial
sums incl. negative oracles (reference: tests/unit/test_communication*.py,
test_stress_partial_propagation.py)."""
import numpy as np
import pytest
import torch

import nabla_b200 as nb
from nabla_b200.core.sharding.propagation import OpShardingRuleTemplate, infer_from_rule
from nabla_b200.core.sharding.spec import compute_global_shape, local_slice, parse_sub_axis
from common import T, close, rand


def test_mesh_geometry_and_groups():
    m = nb.DeviceMesh("m", (2, 4), ("dp", "tp"))
    assert m.get_axis_size("tp") == 4 and m.get_coordinate(6, "dp") == 1 and m.get_coordinate(6, "tp") == 2
    assert m.group_of(5, ["tp"]) == [4, 5, 6, 7] and m.group_of(5, ["dp"]) == [1, 5]
    assert m.groups(["dp"]) == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert not m.is_distributed and m.local_ids == list(range(8))
    assert parse_sub_axis("tp:(2)2") == ("tp", 2, 2)
    assert m.get_axis_size("tp:(2)2") == 2 and m.get_coordinate(3, "tp:(2)2") == 1 and m.get_coordinate(3, "tp:(1)2") == 1


def test_spec_validation_and_repr():
    m = nb.DeviceMesh("m", (2, 4), ("dp", "tp"))
    s = nb.ShardingSpec(m, ["dp", None], partial_sum_axes={"tp"})
    assert repr(s) == "sharding<@m, [{'dp'}, {}], partial={'tp'}>"
    with pytest.raises(ValueError):
        nb.ShardingSpec(m, ["dp", "dp"])
    with pytest.raises(ValueError):
        nb.ShardingSpec(m, ["dp", None], partial_sum_axes={"dp"})
    with pytest.raises(ValueError):
        nb.ShardingSpec(m, ["tp:(1)2", "tp:(1)4"])
    assert nb.compute_local_shape((8, 6), nb.ShardingSpec(m, ["dp", "tp"]), 7) == (4, 0)   # 6 over 4: 2,2,2,0
    assert local_slice(10, 3, 4) == (9, 1)
    assert compute_global_shape((4, 2), nb.ShardingSpec(m, ["dp", "tp"])) == (8, 8)


def test_factor_propagation_matmul():
    m = nb.DeviceMesh("m", (2, 4), ("dp", "tp"))
    rule = OpShardingRuleTemplate.parse("... m k, ... k n -> ... m n").instantiate([(8, 16), (16, 32)])
    out, partial = infer_from_rule(rule, [nb.ShardingSpec(m, ["dp", None]), nb.ShardingSpec(m, [None, "tp"])], m)
    assert [d.axes for d in out.dim_specs] == [["dp"], ["tp"]] and partial == set()
    out, partial = infer_from_rule(rule, [nb.ShardingSpec(m, ["dp", "tp"]), nb.ShardingSpec(m, ["tp", None])], m)
    assert [d.axes for d in out.dim_specs] == [["dp"], []] and partial == {"tp"} and out.partial_sum_axes == {"tp"}
    assert rule.get_contracting_factors() == {"k"}


@pytest.mark.parametrize("shape,axes", [((2,), ("x",)), ((4,), ("x",)), ((8,), ("x",)), ((2, 2), ("a", "b")),
                                        ((2, 4), ("dp", "tp")), ((4, 2), ("a", "b")), ((3, 2), ("a", "b")),
                                        ((2, 2, 2), ("a", "b", "c"))])
def test_shard_gather_roundtrip_all_meshes(shape, axes):
    m = nb.DeviceMesh("m", shape, axes)
    x = rand(12, 10, seed=2)
    xs = nb.shard(T(x), m, [axes[0], axes[-1] if len(axes) > 1 else None])
    assert xs.num_shards == m.size
    close(xs, x)
    close(nb.all_gather(xs, axis=0), x)
    y = nb.reshard(xs, m, [None, axes[0]])
    assert [d.axes for d in y.sharding.dim_specs] == [[], [axes[0]]]
    close(y, x)


def test_collectives_semantics(mesh_2x4):
    x = rand(8, 4, seed=1)
    xs = nb.shard(T(x), mesh_2x4, nb.P("dp", None))
    # psum over dp of a dp-sharded tensor: sums the two row blocks
    r = nb.all_reduce(xs, reduce_axes={"dp"})
    close(r, x[:4] + x[4:])
    # grouped max over tp of replicated values is the value itself
    close(nb.all_reduce(xs, reduce_axes={"tp"}, reduce_op="max"), x)
    # pmean over tp of replicated values is the value; psum multiplies by 4
    close(nb.pmean(xs, "tp"), x)
    close(nb.all_reduce(xs, reduce_axes={"tp"}), 4 * x)
    rs = nb.reduce_scatter(nb.shard(T(x), mesh_2x4, nb.P(None, None)), axis=0, scatter_axes={"tp"})
    assert [d.axes for d in rs.sharding.dim_specs] == [["tp"], []]
    close(rs, 4 * x)
    a2a = nb.all_to_all(nb.shard(T(x), mesh_2x4, nb.P("tp", None)), split_axis=1, concat_axis=0)
    assert [d.axes for d in a2a.sharding.dim_specs] == [[], ["tp"]]
    close(a2a, x)
    idx = nb.axis_index(mesh_2x4, "tp")
    assert idx.to_numpy().tolist() == [0, 1, 2, 3]
    close(nb.distributed_broadcast(T(x), mesh_2x4), x)


def test_ppermute_and_its_vjp():
    m = nb.DeviceMesh("pp", (4,), ("stage",))
    x = rand(4, 3, seed=3)
    xs = nb.shard(T(x), m, ["stage", None])
    perm = [(i, (i + 1) % 4) for i in range(4)]
    close(nb.ppermute(xs, perm), torch.roll(x, 1, 0))
    # partial permutation: unaddressed destinations receive zeros
    ref = torch.zeros_like(x)
    ref[1] = x[0]
    close(nb.ppermute(xs, perm=[(0, 1)]), ref)
    g = nb.grad(lambda t: nb.reduce_sum(nb.ppermute(t, perm) * T(torch.arange(12.0).reshape(4, 3)).shard(m, ["stage", None])))(xs)
    close(g, torch.roll(torch.arange(12.0).reshape(4, 3), -1, 0))
    with pytest.raises(ValueError):
        nb.ppermute(xs, [(0, 1), (2, 1)])


def test_tp_mlp_deferred_partial_and_lazy_allreduce(mesh_2x4):
    x, w1, w2 = rand(8, 16, seed=1), rand(16, 32, seed=2), rand(32, 16, seed=3)
    xs = nb.shard(T(x), mesh_2x4, nb.P("dp", None))
    w1s = nb.shard(T(w1), mesh_2x4, nb.P(None, "tp"))
    w2s = nb.shard(T(w2), mesh_2x4, nb.P("tp", None))
    h = nb.relu(xs @ w1s)
    assert [d.axes for d in h.sharding.dim_specs] == [["dp"], ["tp"]] and not h.sharding.partial_sum_axes
    y = h @ w2s
    assert y.sharding.partial_sum_axes == {"tp"}                    # reduction deferred
    z = (-y) * 2.0 + y                                               # linear ops keep it deferred
    assert z.sharding.partial_sum_axes == {"tp"}
    e = nb.exp(z * 0.01)                                             # non-linear: reduced first
    assert not e.sharding.partial_sum_axes
    ref = torch.exp((-(torch.relu(x @ w1) @ w2) * 2 + torch.relu(x @ w1) @ w2) * 0.01)
    close(e, ref, rtol=1e-4, atol=1e-4)
    tr = str(nb.trace(lambda a, b, c: nb.exp((nb.relu(a @ b) @ c) * 0.01), xs, w1s, w2s))
    assert tr.count("all_reduce(") == 1 and "spmd @mesh" in tr


def test_partial_policies_negative_oracle(mesh_2x4):
    """A wrong reduction schedule gives a different number: adding a replicated bias to a
    pending partial sum must reduce first (else the bias is counted tp times)."""
    x, w, b = rand(8, 16, seed=1), rand(16, 8, seed=2), rand(1, 8, seed=3)
    xs = nb.shard(T(x), mesh_2x4, nb.P(None, "tp"))
    ws = nb.shard(T(w), mesh_2x4, nb.P("tp", None))
    y = xs @ ws
    assert y.sharding.partial_sum_axes == {"tp"}
    out = y + T(b)
    assert not out.sharding.partial_sum_axes
    good = x @ w + b
    wrong = x @ w + 4 * b
    close(out, good, rtol=1e-4, atol=1e-4)
    assert not np.allclose(out.to_numpy(), wrong.numpy(), rtol=1e-3)
    # mul by a replicated tensor is linear in the partial operand: stays deferred and is right
    m = y * T(b)
    assert m.sharding.partial_sum_axes == {"tp"}
    close(m, (x @ w) * b, rtol=1e-4, atol=1e-4)
    # partial * partial is not allowed to stay deferred
    pp = y * y
    assert not pp.sharding.partial_sum_axes
    close(pp, (x @ w) ** 2, rtol=1e-4, atol=1e-3)
    # division: only the numerator may be partial
    close(T(b) / (y + 100.0), b / (x @ w + 100.0), rtol=1e-4, atol=1e-5)
    assert (y / T(b + 3.0)).sharding.partial_sum_axes == {"tp"}
    # cast never carries a partial sum
    assert not nb.cast(y, nb.DType.float64).sharding.partial_sum_axes
    # reduce_sum carries it, reduce_max resolves it
    assert nb.reduce_sum(y, axis=0).sharding.partial_sum_axes == {"tp"}
    close(nb.reduce_max(y, axis=1), (x @ w).amax(1), rtol=1e-4, atol=1e-4)


def test_dp_weight_grads_are_allreduced(mesh_2x4):
    x, w, t = rand(8, 6, seed=1), rand(6, 3, seed=2), rand(8, 3, seed=3)
    xs = nb.shard(T(x), mesh_2x4, nb.P("dp", None))
    ts = nb.shard(T(t), mesh_2x4, nb.P("dp", None))
    wt = w.clone().requires_grad_(True)
    ((x @ wt - t) ** 2).mean().backward()
    g = nb.grad(lambda ww: nb.mean((xs @ ww - ts) ** 2.0))(T(w))
    close(g, wt.grad, rtol=1e-5, atol=1e-6)


def test_sharded_softmax_axis_and_reshape_head_split(mesh_2x4):
    x = rand(4, 8, seed=5)
    xs = nb.shard(T(x), mesh_2x4, nb.P(None, "tp"))
    close(nb.softmax(xs, axis=-1), torch.softmax(x, -1), rtol=1e-5, atol=1e-6)
    close(nb.logsoftmax(xs, axis=-1), torch.log_softmax(x, -1), rtol=1e-5, atol=1e-6)
    # splitting a tp-sharded hidden dim into (heads, head_dim) keeps the heads sharded
    h = nb.reshape(xs, (4, 4, 2))
    assert [d.axes for d in h.sharding.dim_specs] == [[], ["tp"], []]
    close(h, x.reshape(4, 4, 2))
    # a reshape that mixes the sharded dim with others gathers it
    m = nb.reshape(xs, (8, 4))
    close(m, x.reshape(8, 4))


def test_vmap_spmd_axis_name_pipeline_stage():
    m = nb.DeviceMesh("pp", (4,), ("stage",))
    w = rand(4, 5, 5, seed=1)
    x = rand(4, 3, 5, seed=2)
    f = nb.vmap(lambda xx, ww: nb.relu(xx @ ww), spmd_axis_name="stage", mesh=m)
    out = f(T(x), T(w))
    assert out.sharding is not None and out.sharding.dim_specs[0].axes == ["stage"]
    close(out, torch.relu(torch.bmm(x, w)), rtol=1e-5, atol=1e-5)


def test_shard_map_and_auto_sharding(mesh_2x4):
    x, w = rand(8, 16, seed=1), rand(16, 32, seed=2)
    f = nb.shard_map(lambda a, b: nb.relu(a @ b), mesh_2x4, in_specs=(nb.P("dp", None), nb.P(None, "tp")),
                     out_specs=nb.P("dp", None))
    out = f(T(x), T(w))
    assert [d.axes for d in out.sharding.dim_specs] == [["dp"], []]
    close(out, torch.relu(x @ w), rtol=1e-5, atol=1e-5)
    g = nb.shard_map(lambda a, b: a @ b, mesh_2x4, in_specs=(None, None), auto_sharding=True)
    close(g(T(x), T(w)), x @ w, rtol=1e-5, atol=1e-4)


def test_sharded_creation_and_like(mesh_2x4):
    xs = nb.shard(T(rand(8, 4)), mesh_2x4, nb.P("dp", "tp"))
    z = nb.zeros_like(xs)
    assert z.sharding == xs.sharding and tuple(z.local_shape) == (4, 1)
    close(nb.ones_like(xs) + xs, 1 + rand(8, 4))


def test_to_numpy_all_and_gather(mesh_2x4):
    x = rand(8, 4, seed=9)
    xs = nb.shard(T(x), mesh_2x4, nb.P("dp", None))
    a, b = nb.Tensor.to_numpy_all(xs, xs * 2.0)
    np.testing.assert_allclose(a, x.numpy())
    np.testing.assert_allclose(b, 2 * x.numpy())
    assert "shard(0)" in repr(xs)


def test_one_mesh_axis_serves_one_factor_of_an_op():
    """``x @ x.T`` with the rows of ``x`` split over an axis: both output dims would want that axis.
    The output keeps it on the rows, the transposed operand is gathered, and the values, later
    reductions and gradients match the unsharded run."""
    mesh = nb.DeviceMesh("cf", (2,), ("a",))
    x = np.random.RandomState(0).randn(4, 8, 8).astype(np.float32)
    ref = x @ x.transpose(0, 2, 1)
    xs = nb.shard(nb.Tensor.from_dlpack(x), mesh, (None, "a", None))
    t = xs @ nb.swap_axes(xs, -1, -2)
    assert tuple(int(d) for d in t.shape) == (4, 8, 8)
    assert [d.axes for d in t.sharding.dim_specs] == [[], ["a"], []]
    np.testing.assert_allclose(t.to_numpy(), ref, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(nb.reduce_max(nb.mean(t, axis=1), axis=0).to_numpy(), ref.mean(1).max(0), rtol=1e-5, atol=1e-5)

    def f(u):
        return nb.reduce_sum(nb.tanh(u @ nb.swap_axes(u, -1, -2)))

    g_ref = nb.grad(f)(nb.Tensor.from_dlpack(x)).to_numpy()
    np.testing.assert_allclose(nb.grad(f)(xs).to_numpy(), g_ref, rtol=1e-4, atol=1e-5)
    mesh2 = nb.DeviceMesh("cf2", (2, 2), ("a", "b"))
    y = np.random.RandomState(1).randn(8, 4).astype(np.float32)
    a = nb.shard(nb.Tensor.from_dlpack(y), mesh2, ("a", None))
    b = nb.shard(nb.Tensor.from_dlpack(y), mesh2, ("b", None))
    s = nb.softmax(a, axis=1)
    out = nb.broadcast_to(nb.unsqueeze(s, axis=0), (2, 8, 4))
    out = out @ nb.swap_axes(out, -1, -2)
    e = np.exp(y - y.max(1, keepdims=True))
    sm = e / e.sum(1, keepdims=True)
    np.testing.assert_allclose(out.to_numpy(), np.broadcast_to(sm @ sm.T, (2, 8, 8)), rtol=1e-5, atol=1e-6)
    assert b.sharding is not None


def test_a_pending_sum_is_taken_before_its_axis_splits_a_dim_of_the_next_op():
    """``(a @ a.T) @ a`` with ``a`` split over "b" along its columns: the first product is pending
    over "b", and the second one wants "b" for its output columns. The sum comes first."""
    mesh = nb.DeviceMesh("ps", (2, 2), ("a", "b"))
    rs = np.random.RandomState(0)
    A, B = rs.randn(8, 4).astype(np.float32), rs.randn(8, 4).astype(np.float32)
    a = nb.shard(nb.Tensor.from_dlpack(A), mesh, (None, "b"))
    b = nb.shard(nb.Tensor.from_dlpack(B), mesh, ("b", "a"))
    t1 = a @ nb.swap_axes(a, -1, -2)
    assert t1.sharding.partial_sum_axes == {"b"}
    for o, O in ((a, A), (b, B)):
        t2 = t1 @ o
        np.testing.assert_allclose(t2.to_numpy(), (A @ A.T) @ O, rtol=1e-4, atol=1e-4)
    g = nb.grad(lambda u: nb.reduce_sum((u @ nb.swap_axes(u, -1, -2)) @ u))(a)
    g_ref = nb.grad(lambda u: nb.reduce_sum((u @ nb.swap_axes(u, -1, -2)) @ u))(nb.Tensor.from_dlpack(A))
    np.testing.assert_allclose(g.to_numpy(), g_ref.to_numpy(), rtol=1e-4, atol=1e-4)


def test_an_operand_split_along_an_extent_one_dim_is_gathered_before_the_op():
    """A (1, n) bias split over an axis along its first dim lives on one device only. Ops never keep
    an axis on such a dim in their output label, so the operand is gathered first: a training step
    with that layout matches the unsharded one."""
    mesh = nb.DeviceMesh("e1", (2,), ("tp",))
    bn = np.arange(16, dtype=np.float32).reshape(1, 16)
    b = nb.shard(nb.Tensor.from_dlpack(bn), mesh, ("tp", None))
    for t, ref in ((b * 0.9, bn * 0.9), (b + b, bn * 2), (nb.tanh(b), np.tanh(bn))):
        t.realize()
        assert [tuple(x.shape) for x in t._impl._buffers] == [(1, 16), (1, 16)]
        assert not any(d.axes for d in t.sharding.dim_specs)
        np.testing.assert_allclose(t.to_numpy(), ref, rtol=1e-6)
    x = np.random.RandomState(0).randn(4, 4).astype(np.float32)
    w = np.random.RandomState(1).randn(4, 16).astype(np.float32)

    def loss(wt, bt):
        d = nb.nn.functional.linear(nb.Tensor.from_dlpack(x), wt, bt)
        return nb.mean(d * d)

    g_ref = nb.grad(loss, argnums=(0, 1))(nb.Tensor.from_dlpack(w), nb.Tensor.from_dlpack(bn))
    g_got = nb.grad(loss, argnums=(0, 1))(nb.shard(nb.Tensor.from_dlpack(w), mesh, (None, "tp")), b)
    for a, r in zip(g_got, g_ref):
        np.testing.assert_allclose(a.to_numpy(), r.to_numpy(), rtol=1e-5, atol=1e-6)
    step = (b - g_got[1] * 0.1) * 0.9 + g_got[1]              # what an SGD-with-momentum update does
    np.testing.assert_allclose(step.to_numpy(), (bn - g_ref[1].to_numpy() * 0.1) * 0.9 + g_ref[1].to_numpy(), rtol=1e-5)


def test_pending_sum_meeting_a_sequence_parallel_residual_becomes_one_reduce_scatter():
    """Row-parallel product (pending over "tp") + a residual split over "tp" along the rows: the sum
    and the split are done by one reduce-scatter, not an all-reduce followed by a slice."""
    from nabla_b200.core.graph.tracing import trace

    mesh = nb.DeviceMesh("sp", (2,), ("tp",))
    rs = np.random.RandomState(0)
    X, W, R = rs.randn(8, 6).astype(np.float32), rs.randn(6, 4).astype(np.float32), rs.randn(8, 4).astype(np.float32)
    x = nb.shard(nb.Tensor.from_dlpack(X), mesh, (None, "tp"))
    w = nb.shard(nb.Tensor.from_dlpack(W), mesh, ("tp", None))
    r = nb.shard(nb.Tensor.from_dlpack(R), mesh, ("tp", None))
    f = lambda a, b, c: nb.tanh((a @ b) + c)      # noqa: E731
    text = str(trace(f, x, w, r))
    assert "reduce_scatter" in text and "all_reduce" not in text
    out = f(x, w, r)
    assert [d.axes for d in out.sharding.dim_specs] == [["tp"], []] and not out.sharding.partial_sum_axes
    np.testing.assert_allclose(out.to_numpy(), np.tanh(X @ W + R), rtol=1e-5, atol=1e-6)


def test_forward_mode_on_sharded_operands_with_tangents_laid_out_differently():
    """Input tangents are laid out like their primals before the rules run, and the tangent of a
    max / min over a sharded axis is the SUM of the devices' addends (the primal is combined with
    max): both against the unsharded JVP."""
    mesh = nb.DeviceMesh("fw", (2, 2), ("a", "b"))
    rs = np.random.RandomState(0)
    X, TX = rs.randn(8, 8).astype(np.float32), rs.randn(8, 8).astype(np.float32)
    mk = lambda v, s: nb.shard(nb.Tensor.from_dlpack(v.copy()), mesh, s)      # noqa: E731
    for red in (nb.reduce_max, nb.reduce_min):
        for spec in ((None, "a"), ("a", None), ("b", "a"), (("a", "b"), None)):
            for axis in (0, 1):
                f = lambda t: red(t, axis=axis, keepdims=True)      # noqa: E731
                _, t_ref = nb.jvp(f, (nb.Tensor.from_dlpack(X.copy()),), (nb.Tensor.from_dlpack(TX.copy()),))
                _, t_got = nb.jvp(f, (mk(X, spec),), (mk(TX, spec),))
                np.testing.assert_allclose(t_got.to_numpy(), t_ref.to_numpy(), rtol=1e-5, atol=1e-6)

    def g(u, v):
        return nb.softmax(u @ nb.swap_axes(v, -1, -2), axis=-1) - nb.reduce_max(u, axis=-1, keepdims=True)

    plain = [nb.Tensor.from_dlpack(a.copy()) for a in (X, TX, TX, X)]
    o_ref, t_ref = nb.jvp(g, (plain[0], plain[1]), (plain[2], plain[3]))
    o, t = nb.jvp(g, (mk(X, ("b", "a")), mk(TX, (None, None))), (mk(TX, ("a", None)), mk(X, (None, "b"))))
    np.testing.assert_allclose(o.to_numpy(), o_ref.to_numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(t.to_numpy(), t_ref.to_numpy(), rtol=1e-4, atol=1e-5)


def test_jacobians_and_hessians_of_a_sharded_input_match_the_plain_ones():
    """jacrev hands unsharded basis cotangents to rules whose operands are on a mesh (the VJP of a
    reduce-scatter among them); all four forward / reverse Hessian constructions agree."""
    mesh = nb.DeviceMesh("jc", (2,), ("a",))
    x = np.random.RandomState(3).randn(2, 2).astype(np.float32) * 0.5
    y = nb.Tensor.from_dlpack(np.random.RandomState(4).randn(2, 2).astype(np.float32) * 0.5)

    def f(a):
        t = a @ nb.swap_axes(a, -1, -2)
        t = nb.cumsum(t, axis=0) + y
        return t - nb.reduce_max(t, axis=-1, keepdims=True)

    plain = lambda: nb.Tensor.from_dlpack(x.copy())                 # noqa: E731
    split = lambda: nb.shard(nb.Tensor.from_dlpack(x.copy()), mesh, ("a", None))      # noqa: E731
    j_ref = nb.jacrev(f)(plain()).to_numpy()
    np.testing.assert_allclose(nb.jacrev(f)(split()).to_numpy(), j_ref, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(nb.jacfwd(f)(split()).to_numpy(), j_ref, rtol=1e-4, atol=1e-5)
    s = lambda a: nb.reduce_sum(nb.tanh(f(a)))                      # noqa: E731
    h_ref = nb.jacrev(nb.jacrev(s))(plain()).to_numpy()
    for outer, inner in ((nb.jacrev, nb.jacrev), (nb.jacfwd, nb.jacfwd), (nb.jacfwd, nb.jacrev), (nb.jacrev, nb.jacfwd)):
        np.testing.assert_allclose(outer(inner(s))(split()).to_numpy(), h_ref, rtol=2e-3, atol=2e-4)
