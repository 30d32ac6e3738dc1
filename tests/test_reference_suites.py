"""Behaviour suites that the reference keeps in files of their own (tests/unit/test_tensor_index_update_api.py,
test_hessian_per_op.py, test_hessian_four_combos_ops.py, test_multi_output.py, test_pooling.py,
test_pytree_custom.py, test_indexing_creation.py), written against this package with torch / numpy
oracles: in-place and functional index updates under grad / vmap / sharding, second derivatives of
single ops through all four forward / reverse combinations, multi-output ops on sharded inputs,
pooling derivatives, custom pytree nodes, gather / scatter with sharding."""
import numpy as np
import pytest
import torch

import nabla_b200 as nb
from nabla_b200 import P

from common import T, close, rand


def _mesh(n=2, name="x"):
    return nb.DeviceMesh("m", (n,), (name,))


# ---------------------------------------------------------------- index updates
def test_setitem_slice_rebinds_the_tensor():
    x = T(np.arange(6, dtype=np.float32).reshape(2, 3))
    x[:, 1:3] = T(np.array([[10.0, 11.0], [12.0, 13.0]], dtype=np.float32))
    close(x, np.array([[0.0, 10.0, 11.0], [3.0, 12.0, 13.0]]))


def test_setitem_with_tensor_indices_broadcasts_a_scalar():
    x = T(np.arange(5, dtype=np.float32))
    x[T(np.array([0, 2, 4], dtype=np.int32))] = 9.0
    close(x, np.array([9.0, 1.0, 9.0, 3.0, 9.0]))


def test_at_set_and_add_are_functional():
    x = T(np.arange(5, dtype=np.float32))
    idx = T(np.array([1, 3], dtype=np.int32))
    y = x.at[idx].set(7.0)
    z = x.at[idx].add(2.0)
    close(x, np.arange(5))
    close(y, np.array([0.0, 7.0, 2.0, 7.0, 4.0]))
    close(z, np.array([0.0, 3.0, 2.0, 5.0, 4.0]))


def test_chained_updates_match_numpy_and_leave_the_input_alone():
    base = np.arange(12, dtype=np.float32).reshape(3, 4)
    x = T(base)
    y = x.at[0, :].set(1.0).at[:, 1:3].add(T(np.full((3, 2), 0.5, dtype=np.float32))).at[2, 3].set(-4.0)
    ref = base.copy()
    ref[0, :] = 1.0
    ref[:, 1:3] += 0.5
    ref[2, 3] = -4.0
    close(y, ref)
    close(x, base)
    x2 = T(base)
    x2[0, :] = 1.0
    x2[:, 1:3] = x2[:, 1:3] + 0.5
    x2[2, 3] = -4.0
    close(x2, ref)


def test_grad_through_setitem_and_at():
    u0 = rand(2, 2, seed=3)
    x0 = rand(3, 4, seed=4)

    def loss_setitem(x, u):
        y = x * 2.0
        y[1:3, 0:2] = u * u
        return nb.reduce_sum(y * y)

    def loss_at(x, u):
        y = (x * 2.0).at[1:3, 0:2].set(u * u).at[0, 3].add(1.0)
        return nb.reduce_sum(y * y)

    def oracle(with_add):
        xt, ut = x0.clone().requires_grad_(True), u0.clone().requires_grad_(True)
        y = (xt * 2.0).clone()
        y[1:3, 0:2] = ut * ut
        if with_add:
            y = y.clone()
            y[0, 3] = y[0, 3] + 1.0
        (y * y).sum().backward()
        return xt.grad, ut.grad

    gx, gu = nb.grad(loss_setitem, argnums=(0, 1))(T(x0), T(u0))
    rx, ru = oracle(False)
    close(gx, rx, rtol=1e-4, atol=1e-4)
    close(gu, ru, rtol=1e-4, atol=1e-4)
    gx, gu = nb.grad(loss_at, argnums=(0, 1))(T(x0), T(u0))
    rx, ru = oracle(True)
    close(gx, rx, rtol=1e-4, atol=1e-4)
    close(gu, ru, rtol=1e-4, atol=1e-4)


def test_vmap_of_an_index_update_and_of_its_gradient():
    xs = rand(4, 5, seed=5)
    us = rand(4, 2, seed=6)

    def f(x, u):
        return x.at[1:3].set(u * 3.0)

    out = nb.vmap(f)(T(xs), T(us))
    ref = xs.clone()
    ref[:, 1:3] = us * 3.0
    close(out, ref)

    def loss(x, u):
        y = x.at[1:3].set(u * u)
        return nb.reduce_sum(y * y)

    g = nb.vmap(nb.grad(loss, argnums=1))(T(xs), T(us))
    close(g, 4.0 * us ** 3, rtol=1e-4, atol=1e-4)


def test_sharded_index_update_and_its_gradient():
    mesh = _mesh(2)
    x0 = rand(4, 6, seed=7)
    u0 = rand(4, 2, seed=8)

    def loss(x, u):
        xs = nb.shard(x, mesh, ("x", None))
        y = xs.at[:, 1:3].set(nb.shard(u, mesh, ("x", None)) * 2.0)
        return nb.reduce_sum(y * y)

    xt, ut = x0.clone().requires_grad_(True), u0.clone().requires_grad_(True)
    y = xt.clone()
    y[:, 1:3] = ut * 2.0
    (y * y).sum().backward()
    val, (gx, gu) = nb.value_and_grad(loss, argnums=(0, 1))(T(x0), T(u0))
    close(val, (y * y).sum().detach(), rtol=1e-4)
    close(gx, xt.grad, rtol=1e-4, atol=1e-4)
    close(gu, ut.grad, rtol=1e-4, atol=1e-4)
    xs = nb.shard(T(x0), mesh, ("x", None))
    xs[:, 1:3] = nb.shard(T(u0), mesh, ("x", None))
    ref = x0.clone()
    ref[:, 1:3] = u0
    close(xs, ref)


# ---------------------------------------------------------------- second derivatives of single ops
def _hessian(f, mode):
    return {"rev_rev": lambda: nb.jacrev(nb.jacrev(f)), "fwd_fwd": lambda: nb.jacfwd(nb.jacfwd(f)),
            "rev_fwd": lambda: nb.jacrev(nb.jacfwd(f)), "fwd_rev": lambda: nb.jacfwd(nb.jacrev(f)),
            "fwd_grad": lambda: nb.jacfwd(nb.grad(f)), "rev_grad": lambda: nb.jacrev(nb.grad(f))}[mode]()


_W = rand(3, 3, seed=11)
_HESSIAN_CASES = {
    "exp_sum": ((5,), lambda a: nb.reduce_sum(nb.exp(a)), lambda a: a.exp().sum()),
    "exp_sum_2d": ((2, 3), lambda a: nb.reduce_sum(nb.exp(a)), lambda a: a.exp().sum()),
    "poly": ((4,), lambda a: nb.reduce_sum(a * a * a + 2.0 * a * a), lambda a: (a ** 3 + 2 * a ** 2).sum()),
    "matmul_quadratic": ((3,), lambda a: nb.reduce_sum(nb.matmul(nb.reshape(a, (1, 3)), T(_W)) * a),
                         lambda a: ((a.reshape(1, 3) @ _W) * a).sum()),
    "reduce_axis_chain": ((2, 3), lambda a: nb.reduce_sum(nb.reduce_sum(a * a, axis=0) * nb.mean(a, axis=0)),
                          lambda a: ((a * a).sum(0) * a.mean(0)).sum()),
    "view_chain": ((2, 3), lambda a: nb.reduce_sum(nb.swap_axes(nb.reshape(a * a, (3, 2)), 0, 1) * nb.moveaxis(
        nb.reshape(a, (3, 2)), 0, 1)), lambda a: ((a * a).reshape(3, 2).transpose(0, 1) * a.reshape(3, 2).movedim(0, 1)).sum()),
    "broadcast_chain": ((3,), lambda a: nb.reduce_sum(nb.broadcast_to(nb.unsqueeze(a, axis=0), (4, 3)) ** 2.0
                                                     * nb.squeeze(nb.unsqueeze(nb.sin(a), axis=1), axis=1)),
                        lambda a: ((a.unsqueeze(0).expand(4, 3) ** 2) * a.sin()).sum()),
    "getitem_scalar": ((4,), lambda a: a[1] * a[1] * a[2] + nb.reduce_sum(a[0:2] * a[2:4]),
                       lambda a: a[1] * a[1] * a[2] + (a[0:2] * a[2:4]).sum()),
}


@pytest.mark.parametrize("mode", ["rev_rev", "fwd_fwd", "rev_fwd", "fwd_rev", "fwd_grad", "rev_grad"])
@pytest.mark.parametrize("case", sorted(_HESSIAN_CASES))
def test_hessian_of_single_ops_through_every_combination(case, mode):
    shape, f, ft = _HESSIAN_CASES[case]
    a0 = rand(*shape, seed=13) * 0.7
    ref = torch.autograd.functional.hessian(ft, a0)
    got = _hessian(f, mode)(T(a0))
    close(got, ref, rtol=2e-4, atol=2e-4, msg=f"{case}/{mode}")


# ---------------------------------------------------------------- multi-output ops
def test_split_chunk_unbind_on_sharded_inputs():
    mesh = _mesh(2)
    a = rand(4, 6, seed=21)
    xs = nb.shard(T(a), mesh, ("x", None))
    parts = nb.split(xs, 3, axis=1)                       # the split axis is not the sharded one
    for p, r in zip(parts, torch.split(a, 2, dim=1)):
        close(p, r)
    parts = nb.split(xs, 2, axis=0)                       # the split axis is the sharded one
    for p, r in zip(parts, torch.split(a, 2, dim=0)):
        close(p, r)
    parts = nb.split(xs, [1, 2, 3], axis=1)
    for p, r in zip(parts, torch.split(a, [1, 2, 3], dim=1)):
        close(p, r)
    for p, r in zip(nb.chunk(xs, 3, axis=1), torch.chunk(a, 3, dim=1)):
        close(p, r)
    uneven = nb.chunk(T(rand(7, 2, seed=22)), 3, axis=0)
    assert [tuple(int(d) for d in u.shape) for u in uneven] == [(3, 2), (2, 2), (2, 2)]      # numpy array_split sizes
    for p, r in zip(nb.unbind(xs, axis=0), torch.unbind(a, 0)):
        close(p, r)
    b = rand(2, 4, 3, seed=23)
    for p, r in zip(nb.unbind(nb.shard(T(b), mesh, (None, "x", None)), axis=1), torch.unbind(b, 1)):
        close(p, r)


def test_split_on_a_two_axis_mesh_and_minmax():
    mesh = nb.DeviceMesh("m2", (2, 2), ("a", "b"))
    a = rand(4, 8, seed=24)
    xs = nb.shard(T(a), mesh, ("a", "b"))
    for p, r in zip(nb.split(xs, 2, axis=1), torch.split(a, 4, dim=1)):
        close(p, r)
    mm = nb.minmax(T(a), axis=1)
    close(mm["min"], a.min(1).values)
    close(mm["max"], a.max(1).values)
    mm = nb.minmax(nb.shard(T(a), _mesh(2), ("x", None)), axis=0)
    close(mm["min"], a.min(0).values)
    close(mm["max"], a.max(0).values)
    for t in (T(a), nb.shard(T(a), _mesh(2), ("x", None))):      # no axis: over the whole tensor
        mm = nb.minmax(t)
        assert tuple(mm["min"].shape) == ()
        close(mm["min"], a.min())
        close(mm["max"], a.max())


def test_vmap_over_multi_output_ops_and_edge_cases():
    a = rand(3, 4, 6, seed=25)
    outs = nb.vmap(lambda t: nb.split(t, 2, axis=1))(T(a))
    for p, r in zip(outs, torch.split(a, 3, dim=2)):
        close(p, r)
    outs = nb.vmap(lambda t: tuple(nb.chunk(t, 2, axis=0)))(T(a))
    for p, r in zip(outs, torch.chunk(a, 2, dim=1)):
        close(p, r)
    outs = nb.vmap(lambda t: nb.unbind(t, axis=0))(T(a))
    for p, r in zip(outs, torch.unbind(a, 1)):
        close(p, r)
    one = nb.split(T(a), 1, axis=0)
    assert len(one) == 1
    close(one[0], a)
    many = nb.chunk(T(rand(2, 3, seed=26)), 5, axis=0)     # more chunks than elements
    assert len(many) == 2
    single = nb.unbind(T(rand(1, 3, seed=27)), axis=0)
    assert len(single) == 1 and tuple(int(d) for d in single[0].shape) == (3,)


def test_gradient_through_split_and_unbind():
    a = rand(4, 6, seed=28)

    def f(t):
        p, q, r = nb.split(t, 3, axis=1)
        u = nb.unbind(p * q, axis=0)
        return nb.reduce_sum(u[0] * u[1]) + nb.reduce_sum(r * r * r)

    at = a.clone().requires_grad_(True)
    p, q, r = torch.split(at, 2, dim=1)
    u = torch.unbind(p * q, 0)
    ((u[0] * u[1]).sum() + (r ** 3).sum()).backward()
    close(nb.grad(f)(T(a)), at.grad, rtol=1e-4, atol=1e-4)


# ---------------------------------------------------------------- pooling (NHWC)
def _pool_ref(fn, x, k, s, p):
    return fn(x.permute(0, 3, 1, 2), k, s, padding=p).permute(0, 2, 3, 1)


@pytest.mark.parametrize("kind", ["avg", "max"])
def test_pool2d_forward_vjp_and_jvp_match_torch(kind):
    op = nb.avg_pool2d if kind == "avg" else nb.max_pool2d
    ref_fn = torch.nn.functional.avg_pool2d if kind == "avg" else torch.nn.functional.max_pool2d
    x0 = rand(2, 6, 7, 3, seed=31)
    k, s, p = (3, 2), (2, 1), (1, 0)
    y = op(T(x0), k, stride=s, padding=p)
    xt = x0.clone().requires_grad_(True)
    yt = _pool_ref(ref_fn, xt, k, s, p)
    close(y, yt.detach(), rtol=1e-5, atol=1e-5)
    cot = rand(*yt.shape, seed=32)
    yt.backward(cot)
    _, pull = nb.vjp(lambda t: op(t, k, stride=s, padding=p), T(x0))
    (gx,) = pull(T(cot))
    close(gx, xt.grad, rtol=1e-4, atol=1e-5)
    tan = rand(*x0.shape, seed=33)
    _, jt = torch.autograd.functional.jvp(lambda t: _pool_ref(ref_fn, t, k, s, p), x0, tan)
    _, tout = nb.jvp(lambda t: op(t, k, stride=s, padding=p), (T(x0),), (T(tan),))
    close(tout, jt, rtol=1e-4, atol=1e-5)


def test_avg_pool2d_under_nested_vmap_and_bad_parameters():
    x0 = rand(2, 3, 1, 4, 4, 2, seed=34)
    f = lambda t: nb.avg_pool2d(t, (2, 2), stride=(2, 2))
    out = nb.vmap(nb.vmap(f))(T(x0))
    ref = torch.stack([torch.stack([_pool_ref(torch.nn.functional.avg_pool2d, x0[i, j], 2, 2, 0) for j in range(3)])
                       for i in range(2)])
    close(out, ref, rtol=1e-5, atol=1e-5)
    with pytest.raises(Exception):
        nb.avg_pool2d(T(rand(1, 4, 4, 1)), (0, 2))
    with pytest.raises(Exception):
        nb.max_pool2d(T(rand(4, 4, 1)), (2, 2))           # not NHWC


# ---------------------------------------------------------------- custom pytree nodes
def test_custom_pytree_node_roundtrip_map_and_grad():
    from nabla_b200.core.common import pytree

    class Pair:
        def __init__(self, a, b, tag):
            self.a, self.b, self.tag = a, b, tag

    pytree.register_pytree_node(Pair, lambda p: ((p.a, p.b), p.tag), lambda tag, ch: Pair(ch[0], ch[1], tag))
    tree = {"p": Pair(T(rand(2, seed=41)), T(rand(2, seed=42)), "meta"), "k": [T(rand(3, seed=43)), 5]}
    leaves, td = pytree.tree_flatten(tree)
    assert sum(isinstance(l, nb.Tensor) for l in leaves) == 3
    back = pytree.tree_unflatten(td, leaves)
    assert isinstance(back["p"], Pair) and back["p"].tag == "meta" and back["k"][1] == 5
    doubled = pytree.tree_map(lambda t: t * 2.0 if isinstance(t, nb.Tensor) else t, tree)
    close(doubled["p"].a, tree["p"].a.to_numpy() * 2.0)
    g = nb.grad(lambda pr: nb.reduce_sum(pr.a * pr.b * pr.b))(tree["p"])
    assert isinstance(g, Pair)
    close(g.a, tree["p"].b.to_numpy() ** 2, rtol=1e-5)
    close(g.b, 2.0 * tree["p"].a.to_numpy() * tree["p"].b.to_numpy(), rtol=1e-5)


# ---------------------------------------------------------------- gather / scatter with sharding and vmap
def test_gather_and_scatter_on_sharded_inputs():
    mesh = _mesh(2)
    a = rand(4, 6, seed=51)
    idx = torch.tensor([2, 0, 5], dtype=torch.int64)
    close(nb.gather(T(a), T(idx), axis=1), a[:, idx])
    close(nb.gather(nb.shard(T(a), mesh, ("x", None)), T(idx), axis=1), a[:, idx])       # sharded on the other axis
    close(nb.gather(nb.shard(T(a), mesh, ("x", None)), T(torch.tensor([3, 1])), axis=0), a[[3, 1]])
    b = rand(2, 4, 3, seed=52)
    close(nb.gather(nb.shard(T(b), mesh, ("x", None, None)), T(torch.tensor([1, 3, 3])), axis=1), b[:, [1, 3, 3]])
    close(nb.gather(T(b), T(torch.tensor([2, 0])), axis=-1), b[..., [2, 0]])
    upd = rand(4, 3, seed=53)
    ref = a.clone()
    ref[:, idx] = upd
    close(nb.scatter(T(a), T(idx), T(upd), axis=1), ref)
    close(nb.scatter(nb.shard(T(a), mesh, ("x", None)), T(idx), nb.shard(T(upd), mesh, ("x", None)), axis=1), ref)
    # gather then scatter of the same rows gives the original back
    rows = torch.tensor([3, 0, 2, 1])
    close(nb.scatter(T(torch.zeros(4, 6)), T(rows), nb.gather(T(a), T(rows), axis=0), axis=0), a)


@pytest.mark.parametrize("batch", [2, 4])
def test_vmap_gather_with_shared_and_batched_indices(batch):
    a = rand(batch, 5, 3, seed=54)
    idx = torch.tensor([4, 0, 2])
    close(nb.vmap(lambda t: nb.gather(t, T(idx), axis=0))(T(a)), a[:, idx])
    bidx = torch.stack([torch.randperm(5, generator=torch.Generator().manual_seed(i))[:2] for i in range(batch)])
    out = nb.vmap(lambda t, i: nb.gather(t, i, axis=0))(T(a), T(bidx))
    close(out, torch.stack([a[i][bidx[i]] for i in range(batch)]))


def test_random_creation_does_not_depend_on_the_sharding():
    mesh = _mesh(2)
    nb.seed(123)
    full = nb.uniform((4, 6)).to_numpy()
    nb.seed(123)
    sharded = nb.shard(nb.uniform((4, 6)), mesh, ("x", None)).to_numpy()
    assert np.array_equal(full, sharded)
    assert 0.0 <= full.min() and full.max() <= 1.0 and full.std() > 0.1


# ---------------------------------------------------------------- vmap over collectives
def _rng_array(*shape, seed=0):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def test_vmap_over_all_gather_all_reduce_and_reduce_scatter():
    mesh = nb.DeviceMesh("mesh_tp", (2,), ("tp",))
    x0 = _rng_array(4, 16, seed=61)
    r = nb.vmap(lambda x: nb.all_gather(x.shard(mesh, P("tp")), axis=0))(T(x0))
    assert tuple(int(d) for d in r.shape) == (4, 16) and r.sharding.is_fully_replicated()
    close(r, x0)
    # all_reduce of a spatially split vector adds the halves (the op's own semantics)
    r = nb.vmap(lambda x: nb.all_reduce(x.shard(mesh, P("tp")), reduce_op="sum"))(T(x0))
    assert tuple(int(d) for d in r.shape) == (4, 8)
    close(r, x0[:, :8] + x0[:, 8:])
    r = nb.vmap(lambda x: nb.reduce_scatter(x.shard(mesh, P("tp")), axis=0))(T(x0))
    assert tuple(int(d) for d in r.shape) == (4, 8)


def test_vmap_on_a_dp_axis_with_tp_communication_inside():
    mesh = nb.DeviceMesh("mesh_hybrid", (2, 2), ("dp", "tp"))
    x0 = _rng_array(4, 16, seed=62)
    r = nb.vmap(lambda x: nb.all_gather(x.shard(mesh, P("tp")), axis=0))(T(x0).shard(mesh, P("dp", None)))
    close(r, x0)
    assert "dp" in r.sharding.dim_specs[0].axes


def test_nested_vmap_and_shifted_in_axes_over_all_gather():
    mesh = nb.DeviceMesh("mesh_n", (2,), ("tp",))
    x0 = _rng_array(2, 3, 8, seed=63)
    f = lambda x: nb.all_gather(x.shard(mesh, P("tp")), axis=0) * 2.0
    close(nb.vmap(nb.vmap(f))(T(x0)), 2.0 * x0)
    x1 = _rng_array(8, 5, seed=64)                      # the mapped axis is the second one
    r = nb.vmap(f, in_axes=1, out_axes=1)(T(x1))
    close(r, 2.0 * x1)
    x3 = _rng_array(3, 4, 4, seed=65)
    r = nb.vmap(lambda x: nb.all_to_all(x.shard(mesh, P("tp", None)), 0, 1))(T(x3))
    assert tuple(int(d) for d in r.shape) == (3, 4, 4)
    close(r, x3)


def test_gradient_through_vmapped_collectives():
    mesh = nb.DeviceMesh("mesh_g", (2,), ("tp",))
    x0 = _rng_array(4, 16, seed=66)

    def loss_ar(x):
        y = nb.vmap(lambda t: nb.all_reduce(t.shard(mesh, P("tp")), reduce_op="sum"))(x)
        return nb.reduce_sum(y * y)

    s = x0[:, :8] + x0[:, 8:]
    close(nb.grad(loss_ar)(T(x0)), np.concatenate([2 * s, 2 * s], 1), rtol=1e-5, atol=1e-5)

    def loss_ag(x):
        y = nb.vmap(lambda t: nb.all_gather(t.shard(mesh, P("tp")), axis=0))(x)
        return nb.reduce_sum(y * y * y)

    close(nb.grad(loss_ag)(T(x0)), 3.0 * x0 * x0, rtol=1e-4, atol=1e-5)


# ---------------------------------------------------------------- physical-shape ops on sharded inputs
def test_reductions_and_view_ops_keep_or_resolve_the_sharding():
    mesh = _mesh(2)
    a = rand(4, 6, seed=71)
    xs = nb.shard(T(a), mesh, ("x", None))
    r = nb.reduce_sum(xs, axis=1)                        # the reduced axis is not the sharded one
    close(r, a.sum(1))
    assert r.sharding is not None and "x" in r.sharding.dim_specs[0].axes
    close(nb.reduce_sum(xs, axis=0), a.sum(0))           # the reduced axis is the sharded one
    close(nb.mean(xs, axis=1), a.mean(1))
    close(nb.mean(xs, axis=0), a.mean(0), rtol=1e-5, atol=1e-6)
    b = rand(4, 1, 6, seed=72)
    sq = nb.squeeze(nb.shard(T(b), mesh, ("x", None, None)), axis=1)
    close(sq, b.squeeze(1))
    assert "x" in sq.sharding.dim_specs[0].axes
    un = nb.unsqueeze(xs, axis=0)
    close(un, a.unsqueeze(0))
    assert "x" in un.sharding.dim_specs[1].axes
    bc = nb.broadcast_to(nb.unsqueeze(xs, axis=0), (3, 4, 6))
    close(bc, a.unsqueeze(0).expand(3, 4, 6))
    assert "x" in bc.sharding.dim_specs[1].axes


# ---------------------------------------------------------------- a small CNN trained for a few steps
def test_cnn_training_loop_realizes_every_step_and_learns():
    rng = np.random.default_rng(5)
    xb = rng.standard_normal((16, 8, 8, 1)).astype(np.float32)
    yb = (xb.mean(axis=(1, 2, 3)) > 0).astype(np.int64)
    params = {"w1": T(rng.standard_normal((3, 3, 1, 4)).astype(np.float32) * 0.3), "b1": T(np.zeros(4, np.float32)),
              "w2": T(rng.standard_normal((4 * 4 * 4, 2)).astype(np.float32) * 0.1), "b2": T(np.zeros(2, np.float32))}
    onehot = T(np.eye(2, dtype=np.float32)[yb])

    def loss_fn(p, x):
        h = nb.relu(nb.conv2d(x, p["w1"], stride=(1, 1), padding=(1, 1)) + p["b1"])
        h = nb.max_pool2d(h, (2, 2), stride=(2, 2))
        logits = nb.reshape(h, (16, 4 * 4 * 4)) @ p["w2"] + p["b2"]
        logp = logits - nb.unsqueeze(nb.logsumexp(logits, axis=1), axis=1) if hasattr(nb, "logsumexp") else nb.logsoftmax(logits, axis=1)
        return -nb.mean(nb.reduce_sum(logp * onehot, axis=1))

    losses = []
    for _ in range(12):
        loss, g = nb.value_and_grad(loss_fn)(params, T(xb))
        params = {k: params[k] - 0.5 * g[k] for k in params}
        nb.realize_all(*params.values())                 # the lazy graph is cut every step
        assert all(v.is_realized for v in params.values())
        losses.append(loss.item())
    assert losses[-1] < losses[0] * 0.8, losses


# ---------------------------------------------------------------- control flow, reference calling conventions
def test_while_loop_passes_the_whole_state_as_one_argument():
    def cond_fn(state):
        i, _ = state
        return i < 11.0

    def body_fn(state):
        i, acc = state
        return (i + 1.0, acc + i)

    i, acc = nb.while_loop(cond_fn, body_fn, (T(np.float32(1.0)), T(np.float32(0.0))))
    assert i.item() == 11.0 and acc.item() == 55.0
    assert nb.while_loop(lambda c: c < 10.0, lambda c: c + 1.0, T(np.float32(0.0))).item() == 10.0
    # a sharded tensor in the loop state keeps its value and its shape
    mesh = _mesh(2)
    a = rand(8, 4, seed=81)
    n, out = nb.while_loop(lambda st: st[0] < 5.0, lambda st: (st[0] + 1.0, st[1] + 1.0),
                           (T(np.float32(0.0)), nb.shard(T(a), mesh, ("x", None))))
    assert n.item() == 5.0 and tuple(int(d) for d in out.shape) == (8, 4)
    close(out, a + 5.0)
    # the loop leaves as soon as the condition fails, also when that is before the first iteration
    v = nb.while_loop(lambda t: nb.reduce_sum(t) < 0.0, lambda t: t * 2.0, T(np.ones(3, np.float32)))
    close(v, np.ones(3))
    # a dict inside the state
    st = nb.while_loop(lambda s: s[0]["k"] < 3.0, lambda s: ({"k": s[0]["k"] + 1.0}, s[1] * 2.0),
                       ({"k": T(np.float32(0.0))}, T(np.ones(2, np.float32))))
    assert st[0]["k"].item() == 3.0
    close(st[1], np.full(2, 8.0))


def test_cond_and_scan_conventions():
    a = rand(4, 6, seed=82)
    yes, no = nb.constant(np.array(True)), nb.constant(np.array(False))
    close(nb.cond(yes, lambda u, v: u + v, lambda u, v: u - v, T(a), T(a)), 2 * a)
    close(nb.cond(no, lambda u, v: u + v, lambda u, v: u - v, T(a), T(a)), 0 * a)
    out = nb.cond(yes, lambda u: {"a": u * 2.0, "b": [u + 1.0]}, lambda u: {"a": u, "b": [u]}, T(a))
    close(out["a"], 2 * a)
    close(out["b"][0], a + 1)
    mesh = _mesh(2)
    xs = nb.shard(T(a), mesh, ("x", None))
    r = nb.cond(no, lambda u: u * 2.0, lambda u: nb.reduce_sum(u, axis=0, keepdims=True) + u, xs)
    close(r, a.sum(0, keepdim=True) + a, rtol=1e-5, atol=1e-5)
    carry, ys = nb.scan(lambda c, v: (c + v, c + v), T(np.zeros(6, np.float32)), T(a))
    close(ys, torch.cumsum(a, 0), rtol=1e-5, atol=1e-5)
    close(carry, a.sum(0), rtol=1e-5, atol=1e-5)
    carry, ys = nb.scan(lambda c, v: (c * v, c * v), T(np.ones(6, np.float32)), nb.shard(T(a), mesh, (None, "x")))
    close(ys, torch.cumprod(a, 0), rtol=1e-4, atol=1e-5)
    seqs = rand(3, 5, 2, seed=83)
    f = lambda seq: nb.scan(lambda c, v: ({"s": c["s"] + v, "n": c["n"] + 1.0}, c["s"]),
                            {"s": T(np.zeros(2, np.float32)), "n": nb.constant(np.float32(0.0))}, seq)
    carry, ys = nb.vmap(f)(T(seqs))
    close(carry["s"], seqs.sum(1), rtol=1e-5, atol=1e-5)
    close(carry["n"], np.full(3, 5.0))
    rev_carry, rev = nb.scan(lambda c, v: (c + v, c), T(np.zeros(6, np.float32)), T(a), reverse=True)
    close(rev_carry, a.sum(0), rtol=1e-5, atol=1e-5)
    close(rev[0], a[1:].sum(0), rtol=1e-5, atol=1e-5)


# ---------------------------------------------------------------- behaviours the reference's older suites rely on
def test_backward_on_trace_gives_gradients_for_the_trace_inputs_after_trace_returned():
    """`trace()` restores `is_traced` when it returns; the inputs named to it still get gradients
    (reference: tests/depr/test_dp_vs_mp_vjp.py, test_sharded_comm_vjp.py)."""
    from nabla_b200.core.autograd import backward_on_trace
    from nabla_b200.core.graph.tracing import trace

    mesh = _mesh(2, "tp")
    xn, wn = rand(4, 8, seed=90), rand(8, 4, seed=91)
    x = nb.shard(T(xn), mesh, ("tp", None))
    w = nb.shard(T(wn), mesh, (None, None))
    t = trace(lambda a, b: nb.reduce_sum(nb.matmul(a, b), axis=0), x, w)
    assert not x.is_traced
    g = backward_on_trace(t, nb.full_like(t.outputs, 1.0))
    close(g[x], wn.sum(1).expand(4, 8), rtol=1e-5, atol=1e-5)
    close(g[w], xn.sum(0)[:, None].expand(8, 4), rtol=1e-5, atol=1e-5)


def test_from_dlpack_keeps_a_zero_dim_array_zero_dim():
    t = nb.Tensor.from_dlpack(np.array(1.5, dtype=np.float32))
    assert tuple(int(d) for d in t.shape) == ()
    assert t.item() == 1.5


def test_vmapped_matmul_broadcasts_logical_batch_dims_of_unequal_rank():
    """Per-stage `x @ W` with x (stages, batch, s, d) and W (stages, d, n): under vmap the mapped dim
    is in front of both, and W has to broadcast over x's batch dim, sharded or not
    (reference: tests/depr/test_pp_transformer.py)."""
    xn, wn = rand(2, 4, 6, 8, seed=92), rand(2, 8, 5, seed=93)
    ref = torch.einsum("sbik,skn->sbin", xn, wn)
    f = nb.vmap(lambda a, b: a @ b)
    close(f(T(xn), T(wn)), ref, rtol=1e-5, atol=1e-5)
    ga, gb = nb.grad(lambda a, b: nb.reduce_sum(f(a, b)), argnums=(0, 1))(T(xn), T(wn))
    close(ga, wn.sum(-1)[:, None, None, :].expand(2, 4, 6, 8), rtol=1e-5, atol=1e-5)
    close(gb, xn.sum((1, 2))[:, :, None].expand(2, 8, 5), rtol=1e-4, atol=1e-4)
    mesh = nb.DeviceMesh("pp_dp", (2, 2), ("data", "stage"))
    xs = nb.shard(T(xn), mesh, ("stage", "data", None, None))
    ws = nb.shard(T(wn), mesh, ("stage", None, None))
    y = f(xs, ws)
    assert [d.axes for d in y.sharding.dim_specs][:2] == [["stage"], ["data"]]
    close(y, ref, rtol=1e-5, atol=1e-5)


def test_sharding_rule_template_takes_the_dict_form_and_shapes():
    from nabla_b200.core.sharding.propagation import OpShardingRuleTemplate

    m = {0: ["d0"], 1: ["d1"]}
    rule = OpShardingRuleTemplate([m], [m]).instantiate([(4, 8)], [(4, 8)])
    assert rule.input_mappings == [m] and rule.output_mappings == [m]
    assert rule.factor_sizes == {"d0": 4, "d1": 8}
    tpl = OpShardingRuleTemplate.parse("... m k, ... k n -> ... m n", [(3, 4, 5), (5, 6)])
    assert len(tpl.input_mappings[0]) == 3 and len(tpl.input_mappings[1]) == 2 and len(tpl.output_mappings[0]) == 3
    assert tpl.input_mappings[0][0] == tpl.output_mappings[0][0]
    # a size-1 batch dim that broadcasts never shares the other operand's factor
    r = OpShardingRuleTemplate.parse("... m k, ... k n -> ... m n").instantiate([(7, 4, 5), (1, 5, 6)])
    assert r.input_mappings[0][0] != r.input_mappings[1][0]
    assert r.input_mappings[0][0] == r.output_mappings[0][0]


def test_memory_cost_counts_output_bytes():
    from nabla_b200.ops.binary import MatmulOp
    from nabla_b200.ops.reduction import ReduceSumOp

    assert MatmulOp().memory_cost([(8, 32, 64), (8, 64, 128)], [(8, 32, 128)]) == 8 * 32 * 128 * 4
    assert ReduceSumOp().memory_cost([(32, 64, 128)], [(32, 128)], dtype_bytes=2) == 32 * 128 * 2


def test_compile_cache_key_separates_replicated_partial_and_explicitly_replicated():
    from nabla_b200.core.sharding.spec import DimSpec, ShardingSpec
    from nabla_b200.transforms.compile import CompiledFunction

    mesh = _mesh(2, "tp")
    dims = [DimSpec([]), DimSpec([])]
    c = CompiledFunction(lambda x: x)
    keys = {c._extract_sharding_key(ShardingSpec(mesh, dims)),
            c._extract_sharding_key(ShardingSpec(mesh, dims, partial_sum_axes={"tp"})),
            c._extract_sharding_key(ShardingSpec(mesh, dims, replicated_axes={"tp"}))}
    assert len(keys) == 3 and c._extract_sharding_key(None) is None


def test_broadcast_to_physical_adds_logical_dims_and_all_hessian_modes_agree():
    """reference: tests/unit/test_hessian_physical_ops.py (broadcast_to_physical, batch-dims chain)."""
    from nabla_b200.ops.view import broadcast_batch_dims

    a = rand(2, 3, seed=94)
    y = nb.broadcast_to_physical(T(a), (4, 2, 3))
    assert y.batch_dims == 0 and tuple(int(d) for d in y.shape) == (4, 2, 3)

    def f(x):
        z = nb.broadcast_to_physical(x, (4, 2, 3))
        return nb.reduce_sum(z * z)

    def g(x):
        z = broadcast_batch_dims(x, (3,))
        z = nb.reduce_sum_physical(z * z, axis=0, keepdims=False)      # sums a vmap dim away again
        return nb.reduce_sum(z)

    eye = torch.eye(6).reshape(2, 3, 2, 3)
    for fn, scale in ((f, 8.0), (g, 6.0)):
        close(nb.grad(fn)(T(a)), scale * a, rtol=1e-5, atol=1e-5)
        for outer, inner in ((nb.jacrev, nb.jacrev), (nb.jacfwd, nb.jacfwd), (nb.jacrev, nb.jacfwd), (nb.jacfwd, nb.jacrev)):
            close(outer(inner(fn))(T(a)), scale * eye, rtol=1e-5, atol=1e-5)


def test_tensor_global_and_local_shape_include_vmap_dims():
    seen = {}

    def f(row):
        seen["g"], seen["l"], seen["s"] = tuple(row.global_shape), tuple(row.local_shape), tuple(row.shape)
        return row * 2.0

    nb.vmap(f)(T(rand(4, 6, seed=95)))
    assert seen == {"g": (4, 6), "l": (4, 6), "s": (6,)}


def test_distributed_broadcast_gradient_counts_every_copy_and_all_to_all_checks_divisibility():
    """reference: tests/unit/test_communication_rigorous.py:104-123,
    test_vmap_communication_comprehensive.py:80-96."""
    mesh = _mesh(2, "tp")
    u = rand(4, seed=96)

    def f(t):
        r = nb.distributed_broadcast(t, mesh=mesh)
        return nb.reduce_sum(r * r)

    close(f(T(u)), (u * u).sum(), rtol=1e-5, atol=1e-5)
    close(nb.grad(f)(T(u)), 2 * u * 2, rtol=1e-5, atol=1e-5)
    x = nb.shard(T(rand(3, 4, seed=97)), mesh, ("tp", None))
    with pytest.raises(ValueError, match="divisible"):
        nb.all_to_all(x, split_axis=0, concat_axis=1)


def test_index_updates_record_which_api_asked_and_tensor_trace_returns_the_tensor():
    """reference: tests/unit/test_tensor_index_update_api.py:44-108."""
    x = T(np.arange(6, dtype=np.float32).reshape(2, 3))
    upd = T(np.array([[10.0, 11.0], [12.0, 13.0]], dtype=np.float32))
    y = x.at[:, 1:3].set(upd)
    assert y.op_kwargs.get("use_buffer_ops") is False
    t = T(np.arange(6, dtype=np.float32).reshape(2, 3)).trace()
    assert isinstance(t, nb.Tensor) and t.is_traced
    t[:, 1:3] = upd
    assert t.is_traced and t.op_kwargs.get("use_buffer_ops") is True
    close(t, np.array([[0.0, 10.0, 11.0], [3.0, 12.0, 13.0]]))


def test_edge_cases_from_the_reference_older_suites():
    """An int device is a mesh device id; `broadcast` of an unsharded tensor without a mesh is the
    tensor itself; a scatter onto a shard that an uneven split left empty writes nothing
    (reference: tests/depr/test_streaming_pipeline.py, test_communication_ops.py)."""
    from nabla_b200.ops.communication import broadcast

    z = nb.zeros((2, 3), device=0)
    assert tuple(int(d) for d in z.shape) == (2, 3)
    a = rand(8, 4, seed=98)
    close(broadcast(T(a), root=0), a)
    mesh = nb.DeviceMesh("pd", (2, 4), ("stage", "data"))
    state = nb.shard(T(np.zeros((2, 2, 8), np.float32)), mesh, ("stage", "data", None))   # 2 rows over 4 devices
    fresh = rand(1, 2, 8, seed=99)
    out = nb.scatter(state, nb.constant(np.array([0], dtype=np.int32)), T(fresh), axis=0)
    ref = torch.zeros(2, 2, 8)
    ref[0] = fresh[0]
    close(out, ref)
