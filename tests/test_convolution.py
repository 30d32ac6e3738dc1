"""conv2d / conv2d_transpose under every transform, against torch (fp32, CPU): forward, VJP, JVP,
strides > 1, vmap of each, nested vmap(jvp(vjp)), sharded batch, argument validation, and
conv2d_transpose against finite differences (the reference's tests/unit/test_convolution.py, 22 cases,
with torch standing in for jax as the oracle)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as TF

import nabla_b200 as nb
from common import T, close, rand


def _torch_conv(x, w, stride=(1, 1), padding=(0, 0, 0, 0), bias=None):
    """NHWC x RSCF reference through torch's NCHW conv2d."""
    pt, pb, pl, pr = padding
    xp = TF.pad(x.permute(0, 3, 1, 2), (pl, pr, pt, pb))
    y = TF.conv2d(xp, w.permute(3, 2, 0, 1), bias=bias, stride=stride)
    return y.permute(0, 2, 3, 1)


def _torch_conv_transpose(x, w, stride=(1, 1), padding=(0, 0, 0, 0), bias=None):
    """x (N,H,W,Cin), w (R,S,Cout,Cin)."""
    pt, pb, pl, pr = padding
    y = TF.conv_transpose2d(x.permute(0, 3, 1, 2), w.permute(3, 2, 0, 1), stride=stride)
    y = y[:, :, pt:y.shape[2] - pb, pl:y.shape[3] - pr].permute(0, 2, 3, 1)
    return y if bias is None else y + bias


X = lambda *s, seed=0: rand(*s, seed=seed)  # noqa: E731


@pytest.mark.parametrize("stride,padding", [((1, 1), (0, 0, 0, 0)), ((1, 1), (1, 1, 1, 1)), ((2, 2), (1, 0, 0, 1)),
                                            ((2, 1), (2, 2, 0, 0))])
def test_conv2d_forward_matches_torch(stride, padding):
    x, w, b = X(2, 8, 7, 3), X(3, 2, 3, 5, seed=1), X(5, seed=2)
    close(nb.conv2d(T(x), T(w), stride=stride, padding=padding), _torch_conv(x, w, stride, padding), rtol=1e-4, atol=1e-5)
    close(nb.conv2d(T(x), T(w), stride=stride, padding=padding, bias=T(b)), _torch_conv(x, w, stride, padding, b),
          rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("stride", [(1, 1), (2, 2), (3, 2)])
def test_conv2d_vjp_matches_torch(stride):
    x, w = X(2, 9, 8, 3), X(3, 3, 3, 4, seed=1)
    pad = (1, 1, 0, 2)
    xt, wt = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    yt = _torch_conv(xt, wt, stride, pad)
    ct = X(*yt.shape, seed=5)
    gx, gw = torch.autograd.grad(yt, (xt, wt), ct)
    _, pull = nb.vjp(lambda a, b: nb.conv2d(a, b, stride=stride, padding=pad), T(x), T(w))
    g1, g2 = pull(T(ct))
    close(g1, gx, rtol=1e-4, atol=1e-4)
    close(g2, gw, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("stride", [(1, 1), (2, 2)])
def test_conv2d_jvp_matches_torch(stride):
    x, w = X(2, 8, 8, 2), X(3, 3, 2, 3, seed=1)
    vx, vw = X(2, 8, 8, 2, seed=3), X(3, 3, 2, 3, seed=4)
    pad = (1, 1, 1, 1)
    _, jt = torch.autograd.functional.jvp(lambda a, b: _torch_conv(a, b, stride, pad), (x, w), (vx, vw))
    _, tan = nb.jvp(lambda a, b: nb.conv2d(a, b, stride=stride, padding=pad), (T(x), T(w)), (T(vx), T(vw)))
    close(tan, jt, rtol=1e-4, atol=1e-4)


def test_conv2d_bias_gradient():
    x, w, b = X(2, 6, 6, 2), X(3, 3, 2, 4, seed=1), X(4, seed=2)
    bt = b.clone().requires_grad_(True)
    (gb,) = torch.autograd.grad(_torch_conv(x, w, bias=bt).pow(2).sum(), bt)
    g = nb.grad(lambda bb: nb.reduce_sum(nb.conv2d(T(x), T(w), bias=bb) ** 2.0))(T(b))
    close(g, gb, rtol=1e-4, atol=1e-4)


def test_conv2d_vmap_forward_vjp_jvp():
    xb, w = X(3, 2, 7, 7, 2), X(3, 3, 2, 3, seed=1)
    f = lambda a: nb.conv2d(a, T(w), stride=(2, 2), padding=(1, 1, 1, 1))  # noqa: E731
    ref = torch.stack([_torch_conv(xb[i], w, (2, 2), (1, 1, 1, 1)) for i in range(3)])
    close(nb.vmap(f)(T(xb)), ref, rtol=1e-4, atol=1e-5)
    # vmap of a gradient
    xt = xb.clone().requires_grad_(True)
    (gt,) = torch.autograd.grad(torch.stack([_torch_conv(xt[i], w, (2, 2), (1, 1, 1, 1)) for i in range(3)]).pow(2).sum(), xt)
    g = nb.vmap(nb.grad(lambda a: nb.reduce_sum(f(a) ** 2.0)))(T(xb))
    close(g, gt, rtol=1e-4, atol=1e-4)
    # vmap of a jvp
    v = X(3, 2, 7, 7, 2, seed=9)
    jt = torch.stack([torch.autograd.functional.jvp(lambda a: _torch_conv(a, w, (2, 2), (1, 1, 1, 1)), (xb[i],), (v[i],))[1]
                      for i in range(3)])
    tan = nb.vmap(lambda a, t: nb.jvp(f, (a,), (t,))[1])(T(xb), T(v))
    close(tan, jt, rtol=1e-4, atol=1e-4)


def test_conv2d_nested_vmap_jvp_of_vjp():
    """vmap(jvp(grad(f))): second-order through the convolution gradients."""
    xb, w = X(2, 1, 5, 5, 2), X(3, 3, 2, 2, seed=1)
    v = X(2, 1, 5, 5, 2, seed=7)
    loss = lambda a: nb.reduce_sum(nb.conv2d(a, T(w), padding=(1, 1, 1, 1)) ** 3.0)  # noqa: E731
    got = nb.vmap(lambda a, t: nb.jvp(nb.grad(loss), (a,), (t,))[1])(T(xb), T(v))

    def tloss(a):
        return _torch_conv(a, w, padding=(1, 1, 1, 1)).pow(3).sum()

    refs = []
    for i in range(2):
        g = lambda a: torch.autograd.grad(tloss(a), a, create_graph=True)[0]  # noqa: E731
        refs.append(torch.autograd.functional.jvp(g, (xb[i].clone().requires_grad_(True),), (v[i],))[1])
    close(got, torch.stack(refs), rtol=1e-3, atol=1e-3)


def test_conv2d_sharded_batch_forward_jvp_and_vjp(mesh_2x4):
    x, w = X(8, 6, 6, 2), X(3, 3, 2, 4, seed=1)
    xs = nb.shard(T(x), mesh_2x4, nb.P(("dp", "tp"), None, None, None))
    ref = _torch_conv(x, w, (1, 1), (1, 1, 1, 1))
    close(nb.conv2d(xs, T(w), padding=(1, 1, 1, 1)), ref, rtol=1e-4, atol=1e-5)
    v = X(8, 6, 6, 2, seed=3)
    _, jt = torch.autograd.functional.jvp(lambda a: _torch_conv(a, w, (1, 1), (1, 1, 1, 1)), (x,), (v,))
    _, tan = nb.jvp(lambda a: nb.conv2d(a, T(w), padding=(1, 1, 1, 1)), (xs,),
                    (nb.shard(T(v), mesh_2x4, nb.P(("dp", "tp"), None, None, None)),))
    close(tan, jt, rtol=1e-4, atol=1e-4)
    # gradients: the filter gradient is a sum over the sharded batch (all-reduced), the input gradient stays sharded
    xt, wt = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    gx, gw = torch.autograd.grad(_torch_conv(xt, wt, (1, 1), (1, 1, 1, 1)).pow(2).sum(), (xt, wt))
    g1, g2 = nb.grad(lambda a, b: nb.reduce_sum(nb.conv2d(a, b, padding=(1, 1, 1, 1)) ** 2.0), argnums=(0, 1))(xs, T(w))
    close(g1, gx, rtol=1e-4, atol=1e-4)
    close(g2, gw, rtol=1e-4, atol=1e-3)


def test_conv2d_argument_validation():
    x, w = T(X(1, 5, 5, 2)), T(X(3, 3, 2, 4, seed=1))
    with pytest.raises(ValueError, match="groups"):
        nb.conv2d(x, w, groups=2)
    with pytest.raises(ValueError, match="dilation"):
        nb.conv2d(x, w, dilation=(2, 2))
    with pytest.raises(ValueError, match="channels"):
        nb.conv2d(x, T(X(3, 3, 3, 4)))
    with pytest.raises(ValueError, match="bias"):
        nb.conv2d(x, w, bias=T(X(5)))
    with pytest.raises(ValueError):
        nb.conv2d(x, w, stride=(0, 1))
    with pytest.raises(ValueError):
        nb.conv2d(x, w, padding=(1, 2, 3))
    with pytest.raises(ValueError, match="rank-4"):
        nb.conv2d(T(X(5, 5, 2)), w)
    with pytest.raises(ValueError, match="layouts"):
        nb.conv2d(x, w, input_layout="NCHW")


# ---------------------------------------------------------------- conv2d_transpose
@pytest.mark.parametrize("stride,padding", [((1, 1), (0, 0, 0, 0)), ((2, 2), (0, 0, 0, 0)), ((2, 2), (1, 1, 1, 1)),
                                            ((3, 2), (1, 0, 0, 1))])
def test_conv2d_transpose_forward_and_shape(stride, padding):
    x, w, b = X(2, 5, 4, 3), X(3, 3, 4, 3, seed=1), X(4, seed=2)
    ref = _torch_conv_transpose(x, w, stride, padding)
    got = nb.conv2d_transpose(T(x), T(w), stride=stride, padding=padding)
    assert tuple(int(d) for d in got.shape) == tuple(ref.shape)
    close(got, ref, rtol=1e-4, atol=1e-5)
    close(nb.conv2d_transpose(T(x), T(w), stride=stride, padding=padding, bias=T(b)),
          _torch_conv_transpose(x, w, stride, padding, b), rtol=1e-4, atol=1e-5)


def _finite_difference(f, x, v, eps=1e-3):
    return (f(x + eps * v) - f(x - eps * v)) / (2 * eps)


def test_conv2d_transpose_jvp_and_vjp_match_finite_differences():
    x, w = X(1, 4, 4, 2).double(), X(3, 3, 3, 2, seed=1).double()
    vx, vw = X(1, 4, 4, 2, seed=3).double(), X(3, 3, 3, 2, seed=4).double()
    f = lambda a, b: nb.conv2d_transpose(a, b, stride=(2, 2), padding=(1, 0, 0, 1))  # noqa: E731
    fd = _finite_difference(lambda a: _torch_conv_transpose(a, w, (2, 2), (1, 0, 0, 1)), x, vx) + \
        _finite_difference(lambda b: _torch_conv_transpose(x, b, (2, 2), (1, 0, 0, 1)), w, vw)
    _, tan = nb.jvp(f, (T(x), T(w)), (T(vx), T(vw)))
    close(tan, fd, rtol=1e-5, atol=1e-6)
    # <cot, J v> == <J^T cot, v>
    y, pull = nb.vjp(f, T(x), T(w))
    cot = X(*[int(d) for d in y.shape], seed=6).double()
    gx, gw = pull(T(cot))
    lhs = (cot * fd).sum().item()
    rhs = (torch.from_numpy(gx.to_numpy()) * vx).sum().item() + (torch.from_numpy(gw.to_numpy()) * vw).sum().item()
    assert abs(lhs - rhs) < 1e-6 * max(1.0, abs(lhs))


def test_conv2d_transpose_vmap_jvp_and_vjp():
    xb, w = X(3, 1, 4, 4, 2), X(2, 2, 3, 2, seed=1)
    v = X(3, 1, 4, 4, 2, seed=2)
    f = lambda a: nb.conv2d_transpose(a, T(w), stride=(2, 2))  # noqa: E731
    ref = torch.stack([_torch_conv_transpose(xb[i], w, (2, 2)) for i in range(3)])
    close(nb.vmap(f)(T(xb)), ref, rtol=1e-4, atol=1e-5)
    jt = torch.stack([_torch_conv_transpose(v[i], w, (2, 2)) for i in range(3)])          # linear in x
    close(nb.vmap(lambda a, t: nb.jvp(f, (a,), (t,))[1])(T(xb), T(v)), jt, rtol=1e-4, atol=1e-5)
    xt = xb.clone().requires_grad_(True)
    (gt,) = torch.autograd.grad(torch.stack([_torch_conv_transpose(xt[i], w, (2, 2)) for i in range(3)]).pow(2).sum(), xt)
    g = nb.vmap(nb.grad(lambda a: nb.reduce_sum(f(a) ** 2.0)))(T(xb))
    close(g, gt, rtol=1e-4, atol=1e-4)


def test_conv2d_transpose_argument_validation():
    x, w = T(X(1, 4, 4, 2)), T(X(3, 3, 5, 2, seed=1))
    with pytest.raises(ValueError, match="output_paddings"):
        nb.conv2d_transpose(x, w, output_paddings=(1, 1))
    with pytest.raises(ValueError, match="dilation"):
        nb.conv2d_transpose(x, w, dilation=(2, 1))
    with pytest.raises(ValueError, match="Input channels"):
        nb.conv2d_transpose(x, T(X(3, 3, 5, 3)))
    with pytest.raises(ValueError, match="layouts"):
        nb.conv2d_transpose(x, w, filter_layout="OIHW")
