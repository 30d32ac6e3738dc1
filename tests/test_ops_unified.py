"""Every registered op x {baseline, vjp, jvp, vmap} against a torch oracle; and the same ops on
inputs sharded along axis 0 of a (2,4) mesh must equal the unsharded result (the reference's
unified op x transform matrix, tests/unit/test_unified.py)."""
import numpy as np
import pytest
import torch

import nabla_b200 as nb
from common import T, close, rand

U = lambda name, tfn, pos=False, nfn=None: (name, nfn or getattr(nb, name), tfn, pos)  # noqa: E731

UNARY = [
    U("relu", torch.relu), U("sigmoid", torch.sigmoid), U("tanh", torch.tanh), U("exp", torch.exp),
    U("neg", torch.neg), U("abs", torch.abs), U("log", torch.log, True), U("sqrt", torch.sqrt, True),
    U("cos", torch.cos), U("sin", torch.sin), U("erf", torch.erf), U("log1p", torch.log1p, True),
    U("rsqrt", torch.rsqrt, True), U("silu", torch.nn.functional.silu), U("gelu", torch.nn.functional.gelu),
    ("gelu_tanh", lambda x: nb.gelu(x, approximate="tanh"), lambda x: torch.nn.functional.gelu(x, approximate="tanh"), False),
    ("acos", lambda x: nb.acos(x * 0.3), lambda x: torch.acos(x * 0.3), False),
    ("atanh", lambda x: nb.atanh(x * 0.3), lambda x: torch.atanh(x * 0.3), False),
    ("softmax", lambda x: nb.softmax(x, axis=-1), lambda x: torch.softmax(x, -1), False),
    ("logsoftmax", lambda x: nb.logsoftmax(x, axis=0), lambda x: torch.log_softmax(x, 0), False),
    ("sum_axis", lambda x: nb.reduce_sum(x, axis=1), lambda x: x.sum(1), False),
    ("sum_all", lambda x: nb.reduce_sum(x), lambda x: x.sum(), False),
    ("mean_keep", lambda x: nb.mean(x, axis=(0, 1), keepdims=True), lambda x: x.mean((0, 1), keepdim=True), False),
    ("max_axis", lambda x: nb.reduce_max(x, axis=0), lambda x: x.amax(0), False),
    ("min_axis", lambda x: nb.reduce_min(x, axis=-1, keepdims=True), lambda x: x.amin(-1, keepdim=True), False),
    ("cumsum", lambda x: nb.cumsum(x, axis=1), lambda x: x.cumsum(1), False),
    ("cumsum_rev_excl", lambda x: nb.cumsum(x, axis=0, exclusive=True, reverse=True),
     lambda x: x.flip(0).cumsum(0).flip(0) - x, False),
    ("reshape", lambda x: nb.reshape(x, (6, 4)), lambda x: x.reshape(6, 4), False),
    ("swap_axes", lambda x: nb.swap_axes(x, 0, 1), lambda x: x.transpose(0, 1), False),
    ("permute", lambda x: nb.permute(x, (1, 0)), lambda x: x.permute(1, 0), False),
    ("unsqueeze", lambda x: nb.unsqueeze(x, axis=1), lambda x: x.unsqueeze(1), False),
    ("flip", lambda x: nb.flip(x, 1), lambda x: x.flip(1), False),
    ("moveaxis", lambda x: nb.moveaxis(x, 0, -1), lambda x: x.movedim(0, -1), False),
    ("broadcast_to", lambda x: nb.broadcast_to(x, (2, 4, 6)), lambda x: x.expand(2, 4, 6), False),
    ("slice", lambda x: x[1:3, 2:5], lambda x: x[1:3, 2:5], False),
    ("pad", lambda x: nb.pad(x, [(1, 0), (0, 2)]), lambda x: torch.nn.functional.pad(x, (0, 2, 1, 0)), False),
    ("flatten", lambda x: nb.flatten(x), lambda x: x.flatten(), False),
    ("tril", lambda x: nb.tril(x), lambda x: torch.tril(x), False),
    ("triu1", lambda x: nb.triu(x, 1), lambda x: torch.triu(x, 1), False),
    ("concat_self", lambda x: nb.concatenate([x, x * 2.0], axis=1), lambda x: torch.cat([x, x * 2], 1), False),
    ("stack_self", lambda x: nb.stack([x, x + 1.0], axis=0), lambda x: torch.stack([x, x + 1], 0), False),
    ("split_sum", lambda x: nb.split(x, 2, axis=1)[0] * nb.split(x, 2, axis=1)[1], lambda x: x[:, :3] * x[:, 3:], False),
    ("unbind", lambda x: nb.unbind(x, axis=0)[1] + nb.unbind(x, axis=0)[3], lambda x: x[1] + x[3], False),
    ("pow_scalar", lambda x: x ** 3.0, lambda x: x ** 3, False),
    ("div_scalar", lambda x: 2.0 / (x * x + 1.0), lambda x: 2.0 / (x * x + 1.0), False),
    ("where", lambda x: nb.where(x > 0.0, x * 2.0, x * x), lambda x: torch.where(x > 0, x * 2, x * x), False),
    ("cast_f64", lambda x: nb.cast(x, nb.DType.float64) * 2.0, lambda x: x.double() * 2, False),
]

BINARY = [
    ("add", nb.add, torch.add), ("sub", nb.sub, torch.sub), ("mul", nb.mul, torch.mul), ("div", nb.div, torch.div),
    ("matmul", lambda a, b: nb.matmul(a, nb.swap_axes(b, 0, 1)), lambda a, b: a @ b.T),
    ("outer", lambda a, b: nb.outer(a[0], b[1]), lambda a, b: torch.outer(a[0], b[1])),
    ("bcast_add", lambda a, b: a + b[0], lambda a, b: a + b[0]),
    ("pow", lambda a, b: nb.pow(nb.abs(a) + 0.5, b), lambda a, b: torch.pow(a.abs() + 0.5, b)),
    ("mod", lambda a, b: nb.mod(a, nb.abs(b) + 1.0), lambda a, b: torch.remainder(a, b.abs() + 1.0)),
]


def _x(pos):
    return rand(4, 6, seed=3, positive=pos)


@pytest.mark.parametrize("name,fn,tfn,pos", UNARY, ids=[u[0] for u in UNARY])
def test_unary_baseline_vjp_jvp(name, fn, tfn, pos):
    x = _x(pos)
    close(fn(T(x)), tfn(x), msg=f"{name} baseline")
    # vjp against torch autograd
    xt = x.clone().requires_grad_(True)
    yt = tfn(xt)
    ct = rand(*yt.shape, seed=11).to(yt.dtype) if yt.dim() else torch.tensor(1.3, dtype=yt.dtype)
    (gt,) = torch.autograd.grad(yt, xt, ct, allow_unused=True)
    out, pull = nb.vjp(fn, T(x))
    (g,) = pull(T(ct))
    close(g, gt if gt is not None else torch.zeros_like(x), rtol=1e-4, atol=1e-5, msg=f"{name} vjp")
    # jvp against torch forward-mode via double-backward trick
    v = rand(4, 6, seed=5)
    _, jt = torch.autograd.functional.jvp(tfn, (x,), (v,))
    _, tan = nb.jvp(fn, (T(x),), (T(v),))
    close(tan, jt, rtol=1e-4, atol=1e-5, msg=f"{name} jvp")


@pytest.mark.parametrize("name,fn,tfn", BINARY, ids=[b[0] for b in BINARY])
def test_binary_baseline_vjp_jvp(name, fn, tfn):
    a, b = rand(4, 6, seed=1), rand(4, 6, seed=2)
    close(fn(T(a), T(b)), tfn(a, b), rtol=1e-5, atol=1e-5, msg=f"{name} baseline")
    at, bt = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    yt = tfn(at, bt)
    ct = rand(*yt.shape, seed=9)
    ga, gb = torch.autograd.grad(yt, (at, bt), ct, allow_unused=True)
    _, pull = nb.vjp(fn, T(a), T(b))
    g1, g2 = pull(T(ct))
    if name != "mod":
        close(g1, ga, rtol=1e-4, atol=1e-4, msg=f"{name} vjp a")
        close(g2, gb if gb is not None else torch.zeros_like(b), rtol=1e-4, atol=1e-4, msg=f"{name} vjp b")
        va, vb = rand(4, 6, seed=21), rand(4, 6, seed=22)
        _, jt = torch.autograd.functional.jvp(tfn, (a, b), (va, vb))
        _, tan = nb.jvp(fn, (T(a), T(b)), (T(va), T(vb)))
        close(tan, jt, rtol=1e-4, atol=1e-4, msg=f"{name} jvp")


VMAPPABLE = [u for u in UNARY if u[0] not in ("broadcast_to", "reshape", "slice", "split_sum")]


@pytest.mark.parametrize("name,fn,tfn,pos", VMAPPABLE, ids=[u[0] for u in VMAPPABLE])
def test_unary_vmap_and_vmap_vjp(name, fn, tfn, pos):
    xb = rand(3, 4, 6, seed=8, positive=pos)
    ref = torch.stack([tfn(xb[i]) for i in range(3)])
    close(nb.vmap(fn)(T(xb)), ref, rtol=1e-5, atol=1e-5, msg=f"{name} vmap")
    # vmap over axis 1 with output on the last axis
    xb2 = xb.permute(1, 0, 2).contiguous()
    got = nb.vmap(fn, in_axes=1, out_axes=-1)(T(xb2))
    close(got, torch.movedim(ref, 0, -1), rtol=1e-5, atol=1e-5, msg=f"{name} vmap axes")
    # grad of a vmapped function
    xt = xb.clone().requires_grad_(True)
    tot = torch.stack([tfn(xt[i]) for i in range(3)]).double().pow(2).sum()
    (gt,) = torch.autograd.grad(tot, xt, allow_unused=True)
    g = nb.grad(lambda z: nb.reduce_sum(nb.cast(nb.vmap(fn)(z), nb.DType.float64) ** 2.0))(T(xb))
    close(g, gt if gt is not None else torch.zeros_like(xb), rtol=2e-4, atol=2e-4, msg=f"{name} grad(vmap)")


@pytest.mark.parametrize("name,fn,tfn,pos", UNARY, ids=[u[0] for u in UNARY])
def test_unary_sharded_equals_unsharded(name, fn, tfn, pos, mesh_2x4):
    x = rand(8, 6, seed=4, positive=pos)
    if name in ("reshape", "broadcast_to"):
        fn2 = {"reshape": lambda t: nb.reshape(t, (12, 4)), "broadcast_to": lambda t: nb.broadcast_to(t, (2, 8, 6))}[name]
        tf2 = {"reshape": lambda t: t.reshape(12, 4), "broadcast_to": lambda t: t.expand(2, 8, 6)}[name]
    else:
        fn2, tf2 = fn, tfn
    xs = nb.shard(T(x), mesh_2x4, nb.P(("dp", "tp"), None))
    assert xs.is_sharded and tuple(xs.local_shape) == (1, 6)
    close(fn2(xs), tf2(x), rtol=1e-5, atol=1e-5, msg=f"{name} sharded axis0")
    xs1 = nb.shard(T(x), mesh_2x4, nb.P("dp", "tp"))
    # 6 columns over 4 devices: uneven shards (2,2,2,0)
    close(fn2(xs1), tf2(x), rtol=1e-5, atol=1e-5, msg=f"{name} sharded 2d uneven")
    # gradient through the sharded computation equals the unsharded gradient
    xt = x.clone().requires_grad_(True)
    (gt,) = torch.autograd.grad(tf2(xt).double().pow(2).sum(), xt, allow_unused=True)
    g = nb.grad(lambda z: nb.reduce_sum(nb.cast(fn2(z), nb.DType.float64) ** 2.0))(xs)
    close(g, gt if gt is not None else torch.zeros_like(x), rtol=2e-4, atol=2e-4, msg=f"{name} sharded grad")


def test_comparisons_and_logical():
    a, b = rand(5, seed=1), rand(5, seed=2)
    for f, tf in ((nb.equal, torch.eq), (nb.not_equal, torch.ne), (nb.greater, torch.gt), (nb.greater_equal, torch.ge),
                  (nb.less, torch.lt), (nb.less_equal, torch.le)):
        r = f(T(a), T(b))
        assert r.dtype is nb.DType.bool
        np.testing.assert_array_equal(r.to_numpy(), tf(a, b).numpy())
    p, q = T(a > 0), T(b > 0)
    np.testing.assert_array_equal(nb.logical_and(p, q).to_numpy(), ((a > 0) & (b > 0)).numpy())
    np.testing.assert_array_equal(nb.logical_xor(p, q).to_numpy(), ((a > 0) ^ (b > 0)).numpy())
    np.testing.assert_array_equal((~p).to_numpy(), (~(a > 0)).numpy())
    np.testing.assert_array_equal((T(a) > 0.0).to_numpy(), (a > 0).numpy())


def test_argmax_argmin_minmax_chunk_misc():
    x = rand(4, 7, seed=6)
    np.testing.assert_array_equal(nb.argmax(T(x), axis=1).to_numpy(), x.argmax(1).numpy())
    np.testing.assert_array_equal(nb.argmin(T(x), axis=0, keepdims=True).to_numpy(), x.argmin(0, keepdim=True).numpy())
    mm = nb.minmax(T(x), axis=1)
    close(mm["min"], x.amin(1))
    close(mm["max"], x.amax(1))
    parts = nb.chunk(T(x), 3, axis=1)
    assert [int(p.shape[1]) for p in parts] == [3, 2, 2]      # sizes differ by at most one, larger first
    close(nb.floor(T(x)), x.floor())
    close(nb.trunc(T(x)), x.trunc())
    close(nb.round(T(x)), x.round())
    assert nb.is_nan(T(torch.tensor([1.0, float("nan")]))).to_numpy().tolist() == [False, True]
    assert nb.is_inf(T(torch.tensor([1.0, float("inf")]))).to_numpy().tolist() == [False, True]
    close(nb.arange(2, 11, 3), np.arange(2, 11, 3, dtype=np.float32))
    close(nb.hann_window(8), torch.hann_window(8))
    close(nb.full_like(T(x), 2.5), torch.full_like(x, 2.5))
    close(nb.sum(T(x)), x.sum())


def test_gather_scatter_and_grads():
    w = rand(7, 3, seed=1)
    idx = torch.tensor([[1, 3], [3, 6]])
    close(nb.gather(T(w), T(idx), axis=0), w[idx])
    wt = w.clone().requires_grad_(True)
    (gt,) = torch.autograd.grad((wt[idx] ** 2).sum(), wt)
    g = nb.grad(lambda t: nb.reduce_sum(nb.gather(t, T(idx), axis=0) ** 2.0))(T(w))
    close(g, gt, rtol=1e-5, atol=1e-5)
    upd = rand(2, 3, seed=2)
    ref = w.clone()
    ref[torch.tensor([0, 5])] = upd
    close(nb.scatter(T(w), T(torch.tensor([0, 5])), T(upd), axis=0), ref)
    close(nb.take(T(w), T(torch.tensor([2, 2, 0])), axis=1), w[:, [2, 2, 0]])


def test_control_flow():
    x = T(torch.tensor([1.0, -2.0]))
    r = nb.cond(nb.reduce_sum(x) > 0.0, lambda a: a * 2.0, lambda a: a - 1.0, x)
    close(r, torch.tensor([0.0, -3.0]))
    i, acc = nb.while_loop(lambda i, a: i < 5.0, lambda i, a: (i + 1.0, a + i), (nb.constant(0.0), nb.constant(0.0)))
    assert acc.item() == 10.0 and i.item() == 5.0
    carry, ys = nb.scan(lambda c, xt: (c + xt, c * xt), nb.constant(1.0), T(torch.tensor([1.0, 2.0, 3.0])))
    assert carry.item() == 7.0
    close(ys, torch.tensor([1.0, 4.0, 12.0]))
    g = nb.grad(lambda v: nb.scan(lambda c, xt: (c * xt, c), nb.constant(1.0), v)[0])(T(torch.tensor([2.0, 3.0, 4.0])))
    close(g, torch.tensor([12.0, 8.0, 6.0]))
    carry, ys = nb.scan(lambda c, xt: (c + xt, c), nb.constant(0.0), T(torch.tensor([1.0, 2.0, 3.0])), reverse=True)
    assert carry.item() == 6.0
    close(ys, torch.tensor([5.0, 3.0, 0.0]))       # ys[t] belongs to xs[t]: the carry before element t, coming from the end


def test_complex_views():
    x = rand(3, 2, seed=1)
    c = nb.as_interleaved_complex(T(x))
    back = nb.view_as_real_interleaved(c)
    close(back, x)


# ---------------------------------------------------------------- further transform tiers
# (reference: tests/unit/test_unified.py:306-381: vmap(jvp), jacrev, jacfwd per op)
@pytest.mark.parametrize("name,fn,tfn,pos", VMAPPABLE, ids=[u[0] for u in VMAPPABLE])
def test_unary_vmap_of_jvp(name, fn, tfn, pos):
    """vmap(jvp(f)) with all-ones tangents against per-example torch forward mode."""
    xb = rand(3, 4, 6, seed=12, positive=pos)

    def tan_of(x):
        return nb.jvp(fn, (x,), (nb.ones_like(x),))[1]

    got = nb.vmap(tan_of)(T(xb))
    ref = torch.stack([torch.autograd.functional.jvp(tfn, (xb[i],), (torch.ones_like(xb[i]),))[1] for i in range(3)])
    close(got, ref, rtol=1e-4, atol=1e-5, msg=f"{name} vmap(jvp)")


JAC_OPS = [u for u in UNARY if u[0] not in ("cast_f64",)]


@pytest.mark.parametrize("name,fn,tfn,pos", JAC_OPS, ids=[u[0] for u in JAC_OPS])
def test_unary_jacrev_and_jacfwd(name, fn, tfn, pos):
    """Full Jacobians, reverse and forward mode, against torch.autograd.functional.jacobian."""
    x = rand(4, 6, seed=13, positive=pos)
    ref = torch.autograd.functional.jacobian(tfn, x)
    close(nb.jacrev(fn)(T(x)), ref, rtol=1e-4, atol=1e-5, msg=f"{name} jacrev")
    close(nb.jacfwd(fn)(T(x)), ref, rtol=1e-4, atol=1e-5, msg=f"{name} jacfwd")


@pytest.mark.parametrize("name,fn,tfn", [b for b in BINARY if b[0] != "mod"], ids=[b[0] for b in BINARY if b[0] != "mod"])
def test_binary_vmap_of_jvp_and_jacobians(name, fn, tfn):
    a, b = rand(3, 4, 6, seed=14), rand(3, 4, 6, seed=15)

    def tan_of(x, y):
        return nb.jvp(fn, (x, y), (nb.ones_like(x), nb.ones_like(y)))[1]

    got = nb.vmap(tan_of)(T(a), T(b))
    ref = torch.stack([torch.autograd.functional.jvp(tfn, (a[i], b[i]), (torch.ones_like(a[i]), torch.ones_like(b[i])))[1]
                       for i in range(3)])
    close(got, ref, rtol=1e-4, atol=1e-4, msg=f"{name} vmap(jvp)")
    ja, jb = torch.autograd.functional.jacobian(tfn, (a[0], b[0]))
    r = nb.jacrev(fn, argnums=(0, 1))(T(a[0]), T(b[0]))
    f = nb.jacfwd(fn, argnums=(0, 1))(T(a[0]), T(b[0]))
    for got_j, ref_j in ((r[0], ja), (r[1], jb), (f[0], ja), (f[1], jb)):
        close(got_j, ref_j, rtol=1e-4, atol=1e-4, msg=f"{name} jacobian")


def test_python_scalars_promote_bool_and_integer_tensors_like_numpy():
    a = nb.Tensor.from_torch(torch.tensor([True, False]))
    assert (a + 2).to_torch().tolist() == [3, 2] and (a + 2).dtype is nb.DType.int32
    assert (2 * a).to_torch().tolist() == [2, 0]
    assert (a / 2).to_torch().tolist() == [0.5, 0.0]
    assert (a + True).dtype is nb.DType.bool
    assert (a + 2.5).dtype is nb.DType.float32
    b = nb.Tensor.from_torch(torch.tensor([1, 2], dtype=torch.int32))
    assert (b + 2).dtype is nb.DType.int32 and (b * 2.5).dtype is nb.DType.float32
