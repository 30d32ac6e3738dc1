"""Numerics of every hand-written CUDA kernel against a plain PyTorch fp32 reference of the
same op, on small / odd shapes. Needs a B200 (sm_100a)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(got, ref):
    got, ref = got.float(), ref.float()
    return ((got - ref).abs().max() / (ref.abs().max() + 1e-6)).item()


@pytest.fixture(autouse=True)
def _check_status():
    yield
    from nabla_b200 import native

    torch.cuda.synchronize()
    native.check_status()


def test_gemm_on_cta_pairs_matches_lone_ctas_and_fp32():
    """Wide-tile GEMMs run on CTA pairs (cta_group::2) by default: the pair kernel must have been the
    one that ran, agree with the lone-CTA kernel (to bf16 rounding) and with an fp32 reference, for every operand layout, for an odd number of 128-row tiles and
    through the fused epilogues."""
    from nabla_b200 import native
    from nabla_b200.native import gemm

    lib = native.load("libnb_gemm.so")
    assert gemm.set_pair_mode(True)
    a0, b0 = gemm.pair_alloc_probe()
    assert a0 == b0
    torch.manual_seed(4)
    for (M, N, K) in [(4096, 4608, 320), (19072, 2048, 1024), (4224, 4616, 136)]:
        for layout in ("NN", "NT", "TN", "TT"):
            A = torch.randn(K, M, device="cuda", dtype=torch.bfloat16).t() if layout[0] == "T" else \
                torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16).t() if layout[1] == "T" else \
                torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
            gemm.set_pair_mode(True)
            c_pair = gemm.gemm_bf16(A, B)
            assert lib.nb_gemm_pair_max_clusters() > 0          # the pair kernel has been launched
            gemm.set_pair_mode(False)
            c_lone = gemm.gemm_bf16(A, B)
            ref = A.float() @ B.float()
            assert _rel(c_pair, ref) < 1e-2
            assert _rel(c_pair, c_lone) < 4e-3, (M, N, K, layout)
    gemm.set_pair_mode(True)
    A = torch.randn(8192, 1024, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(1024, 8192, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(8192, device="cuda", dtype=torch.bfloat16)
    y, z = gemm.gemm_bf16(A, B, bias=bias, epilogue="gelu", aux="store_preact")
    zr = A.float() @ B.float() + bias.float()
    assert _rel(z, zr) < 1e-2 and _rel(y, torch.nn.functional.gelu(zr)) < 1e-2
    acc = torch.randn(8192, 8192, device="cuda", dtype=torch.float32)
    want = acc + A.float() @ B.float()
    got = gemm.gemm_bf16(A, B, out=acc, out_dtype=torch.float32, accumulate=True)
    assert _rel(got, want) < 1e-2
    native.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (100, 72, 40), (333, 520, 136), (1, 8, 8),
                                   (2048, 2048, 2048), (64, 4096, 1024)])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN", "TT"])
def test_gemm_layouts(M, N, K, layout):
    from nabla_b200.native.gemm import gemm_bf16

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    A = a.t().contiguous().t() if layout[0] == "T" else a
    B = b.t().contiguous().t() if layout[1] == "T" else b
    ref = a.float() @ b.float()
    for bn in (0, 256, 128, 64):
        assert _rel(gemm_bf16(A, B, block_n=bn), ref) < 2e-2


def test_gemm_epilogues_and_batched():
    from nabla_b200.native.gemm import gemm_bf16

    torch.manual_seed(1)
    M, N, K = 520, 776, 264
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(K, N, device="cuda", dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    aux = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    zz = a.float() @ w.float()
    z = zz + bias.float()
    F = torch.nn.functional
    assert _rel(gemm_bf16(a, w, bias=bias), z) < 2e-2
    assert _rel(gemm_bf16(a, w, bias=bias, epilogue="relu"), torch.relu(z)) < 2e-2
    assert _rel(gemm_bf16(a, w, bias=bias, epilogue="gelu"), F.gelu(z)) < 2e-2
    assert _rel(gemm_bf16(a, w, bias=bias, epilogue="gelu", gelu_tanh=True), F.gelu(z, approximate="tanh")) < 2e-2
    o, pre = gemm_bf16(a, w, bias=bias, epilogue="gelu", aux="store_preact")
    assert _rel(o, F.gelu(z)) < 2e-2 and _rel(pre, z) < 2e-2
    assert _rel(gemm_bf16(a, w, aux="add", aux_in=aux), zz + aux.float()) < 2e-2
    assert _rel(gemm_bf16(a, w, aux="drelu", aux_in=aux), zz * (aux.float() > 0)) < 2e-2
    x = aux.float().requires_grad_(True)
    F.gelu(x).sum().backward()
    assert _rel(gemm_bf16(a, w, aux="dgelu", aux_in=aux), zz * x.grad) < 2e-2
    acc = torch.ones(M, N, device="cuda")
    gemm_bf16(a, w, out=acc, accumulate=True)
    assert _rel(acc, zz + 1) < 1e-2
    assert _rel(gemm_bf16(a, w, out_dtype=torch.float32, alpha=0.125), zz * 0.125) < 1e-2
    ab = torch.randn(6, 200, 128, device="cuda", dtype=torch.bfloat16)
    bb = torch.randn(6, 128, 328, device="cuda", dtype=torch.bfloat16)
    assert _rel(gemm_bf16(ab, bb), torch.bmm(ab.float(), bb.float())) < 2e-2
    assert _rel(gemm_bf16(ab, ab.transpose(1, 2)), torch.bmm(ab.float(), ab.float().transpose(1, 2))) < 2e-2
    assert _rel(gemm_bf16(ab, bb[0]), ab.float() @ bb[0].float()) < 2e-2
    # unaligned K (not a multiple of 8) goes through the padding path
    a2 = torch.randn(37, 19, device="cuda", dtype=torch.bfloat16)
    b2 = torch.randn(19, 23, device="cuda", dtype=torch.bfloat16)
    assert _rel(gemm_bf16(a2, b2), a2.float() @ b2.float()) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,D", [(1, 64), (7, 256), (300, 2048), (129, 1024)])
def test_layernorm_fwd_bwd(dtype, rows, D):
    from nabla_b200.native import kernels

    torch.manual_seed(2)
    x = torch.randn(rows, D, device="cuda", dtype=dtype)
    g = torch.randn(D, device="cuda", dtype=dtype)
    b = torch.randn(D, device="cuda", dtype=dtype)
    dy = torch.randn(rows, D, device="cuda", dtype=dtype)
    xr, gr, br = (t.float().requires_grad_(True) for t in (x, g, b))
    ref = torch.nn.functional.layer_norm(xr, (D,), gr, br)
    ref.backward(dy.float())
    y, mean, rstd = kernels.layernorm_fwd(x, g, b, 1e-5)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel(y, ref) < tol
    dx, dg, db = kernels.layernorm_bwd(dy, x, g, mean, rstd)
    assert _rel(dx, xr.grad) < tol and _rel(dg, gr.grad) < tol and _rel(db, br.grad) < tol
    # the same through the dx + dgamma/dbeta kernel pair (the path of rows wider than 8 vectors per lane)
    lib = kernels._L()
    lib.nb_layernorm_bwd_two_kernels(1)
    try:
        dx2, dg2, db2 = kernels.layernorm_bwd(dy, x, g, mean, rstd)
    finally:
        lib.nb_layernorm_bwd_two_kernels(0)
    assert _rel(dx2, xr.grad) < tol and _rel(dg2, gr.grad) < tol and _rel(db2, br.grad) < tol


def test_layernorm_backward_many_rows_and_wide_rows():
    """More rows than the persistent grid of the one-pass kernel holds at once (every warp walks
    several rows), no gamma, and a row too wide for it (4096 bf16 = 16 vectors per lane)."""
    from nabla_b200.native import kernels

    torch.manual_seed(3)
    for rows, D, with_gamma in ((5000, 512, True), (3001, 2048, False), (65, 4096, True)):
        x = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16)
        g = torch.randn(D, device="cuda", dtype=torch.bfloat16) if with_gamma else None
        dy = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16)
        xr = x.float().requires_grad_(True)
        gr = g.float().requires_grad_(True) if with_gamma else None
        torch.nn.functional.layer_norm(xr, (D,), gr, None).backward(dy.float())
        _, mean, rstd = kernels.layernorm_fwd(x, g, None, 1e-5)
        dx, dg, db = kernels.layernorm_bwd(dy, x, g, mean, rstd)
        assert _rel(dx, xr.grad) < 3e-2
        assert _rel(db, dy.float().sum(0)) < 2e-2
        if with_gamma:
            assert _rel(dg, gr.grad) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_softmax_lse_pick_colsum_embedding(dtype):
    from nabla_b200.native import kernels

    torch.manual_seed(3)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    x = torch.randn(37, 1000, device="cuda", dtype=dtype)
    assert _rel(kernels.softmax(x), torch.softmax(x.float(), -1)) < tol
    assert _rel(kernels.softmax(x, log=True), torch.log_softmax(x.float(), -1)) < tol
    t = torch.randint(-5, 1005, (37,), device="cuda")
    lse, picked = kernels.lse_pick_fwd(x, t)
    xf = x.float()
    ref_lse = torch.logsumexp(xf, -1)
    inr = (t >= 0) & (t < 1000)
    ref_pick = torch.where(inr, xf.gather(1, t.clamp(0, 999).unsqueeze(1)).squeeze(1), torch.zeros_like(ref_lse))
    assert _rel(lse, ref_lse) < 1e-4 and _rel(picked, ref_pick) < 1e-4
    gl, gp = torch.randn(37, device="cuda"), torch.randn(37, device="cuda")
    d = kernels.lse_pick_bwd(x, t, lse, gl, gp)
    oh = torch.zeros_like(xf).scatter_(1, t.clamp(0, 999).unsqueeze(1), 1.0) * inr.unsqueeze(1)
    assert _rel(d, torch.exp(xf - ref_lse.unsqueeze(1)) * gl.unsqueeze(1) + oh * gp.unsqueeze(1)) < tol
    y = torch.randn(1234, 264, device="cuda", dtype=dtype)
    assert _rel(kernels.colsum(y), y.float().sum(0)) < tol
    tab = torch.randn(50, 64, device="cuda", dtype=dtype)
    ids = torch.randint(0, 50, (4, 9), device="cuda")
    assert torch.equal(kernels.embedding_gather(tab, ids), tab[ids])
    upd = torch.randn(4, 9, 64, device="cuda", dtype=dtype)
    ref = tab.float().index_add(0, ids.reshape(-1), upd.float().reshape(-1, 64))
    assert _rel(kernels.embedding_scatter_add(tab, ids, upd), ref) < tol


def test_adamw_sgd_activation_rng_dropout_nf4_pool_conv():
    from nabla_b200.native import kernels

    torch.manual_seed(4)
    p = torch.randn(1001, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(1001, device="cuda", dtype=torch.bfloat16)
    m, v = torch.rand(1001, device="cuda"), torch.rand(1001, device="cuda")
    po, mo, vo = kernels.adamw(p, g, m, v, lr=1e-2, b1=0.9, b2=0.99, eps=1e-8, wd=0.1, step=3)
    mn = 0.9 * m + 0.1 * g.float()
    vn = 0.99 * v + 0.01 * g.float() ** 2
    ref = p.float() - 1e-2 * ((mn / (1 - 0.9 ** 3)) / ((vn / (1 - 0.99 ** 3)).sqrt() + 1e-8) + 0.1 * p.float())
    assert _rel(po, ref) < 1e-2 and _rel(mo, mn) < 1e-5 and _rel(vo, vn) < 1e-5
    hyper = torch.tensor([1e-2, 1 - 0.9 ** 3, 1 - 0.99 ** 3, 1.0], device="cuda")
    po2, _, _ = kernels.adamw(p, g, m, v, lr=0.0, b1=0.9, b2=0.99, eps=1e-8, wd=0.1, hyper=hyper)
    assert torch.equal(po, po2)
    ps, bs = kernels.sgd(p.float(), g.float(), m, lr=0.1, momentum=0.9, wd=0.01)
    bref = 0.9 * m + g.float() + 0.01 * p.float()
    assert _rel(bs, bref) < 1e-5 and _rel(ps, p.float() - 0.1 * bref) < 1e-5
    z = torch.randn(777, device="cuda", dtype=torch.bfloat16)
    for mode, fn in (("relu", torch.relu), ("gelu", torch.nn.functional.gelu), ("silu", torch.nn.functional.silu)):
        assert _rel(kernels.activation(z, mode), fn(z.float())) < 2e-2
        zz = z.float().requires_grad_(True)
        fn(zz).backward(g[:777].float())
        assert _rel(kernels.activation_bwd(z, g[:777], mode), zz.grad) < 2e-2
    u = kernels.rng((100000,), torch.float32, "cuda", 1, 0, "uniform", 0.0, 1.0)
    n = kernels.rng((100000,), torch.float32, "cuda", 1, 1, "gaussian", 2.0, 3.0)
    assert 0 <= u.min() and u.max() < 1 and abs(u.mean().item() - 0.5) < 0.01
    assert abs(n.mean().item() - 2.0) < 0.05 and abs(n.std().item() - 3.0) < 0.05
    assert not torch.equal(u, kernels.rng((100000,), torch.float32, "cuda", 1, 5, "uniform", 0.0, 1.0))
    y, mask = kernels.dropout(torch.ones(100000, device="cuda"), 0.3, 7, 0)
    assert abs((mask == 0).float().mean().item() - 0.3) < 0.01 and torch.allclose(y, mask.float() / 0.7)
    from nabla_b200.nn.finetune.qlora import NF4_CODEBOOK

    idx = torch.randint(0, 16, (256,), device="cuda", dtype=torch.uint8)
    packed = (idx[0::2] << 4) | idx[1::2]
    absmax = torch.rand(4, device="cuda") + 0.5
    ref = torch.tensor(NF4_CODEBOOK, device="cuda")[idx.long()] * absmax.repeat_interleave(64)
    assert _rel(kernels.nf4_dequant(packed, absmax, 256, 64, torch.float32), ref) < 1e-3
    x = torch.randn(2, 9, 8, 5, device="cuda")
    for mode, tf in (("avg", torch.nn.functional.avg_pool2d), ("max", torch.nn.functional.max_pool2d)):
        # oracle on the CPU in NCHW-contiguous fp32
        xr = x.cpu().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
        r = tf(xr, (3, 2), (2, 2), padding=(1, 1))
        yk = kernels.pool2d_fwd(x, 3, 2, 2, 2, 1, 1, mode)
        assert _rel(yk.cpu(), r.permute(0, 2, 3, 1)) < 1e-5
        dy = torch.randn_like(yk)
        r.backward(dy.cpu().permute(0, 3, 1, 2).contiguous())
        assert _rel(kernels.pool2d_bwd(x, dy, 3, 2, 2, 2, 1, 1, mode).cpu(), xr.grad.permute(0, 2, 3, 1)) < 1e-5
    # tangent of max pooling: every window picks the tangent at its arg-max
    tan = torch.randn_like(x)
    xc = torch.nn.functional.pad(x.cpu().permute(0, 3, 1, 2), (1, 1, 1, 1), value=float("-inf"))
    tc = torch.nn.functional.pad(tan.cpu().permute(0, 3, 1, 2), (1, 1, 1, 1))
    yy, idx = torch.nn.functional.max_pool2d(xc, (3, 2), (2, 2), return_indices=True)
    sel = tc.flatten(2).gather(2, idx.flatten(2)).view_as(yy).permute(0, 2, 3, 1)
    assert _rel(kernels.pool2d_select(x, tan, 3, 2, 2, 2, 1, 1).cpu(), sel) < 1e-6
    w = torch.randn(3, 3, 5, 4, device="cuda")
    bconv = torch.randn(4, device="cuda")
    ref = torch.nn.functional.conv2d(torch.nn.functional.pad(x.permute(0, 3, 1, 2), (2, 0, 1, 1)), w.permute(3, 2, 0, 1),
                                     bconv, stride=(2, 1)).permute(0, 2, 3, 1)
    assert _rel(kernels.conv2d_direct(x, w, bconv, (2, 1), (1, 1, 2, 0)), ref) < 1e-4


def test_framework_ops_use_native_kernels_on_gpu():
    """Ops on CUDA tensors must run the hand-written kernels (launch counters move) and agree
    with the CPU reference path of the same ops."""
    import nabla_b200 as nb
    from nabla_b200 import nn
    from nabla_b200.native import gemm, kernels
    from nabla_b200.nn import functional as F

    torch.manual_seed(5)
    B, S, D, V = 2, 64, 128, 512
    x = torch.randn(B, S, D)
    g, b = torch.rand(D) + 0.5, torch.randn(D) * 0.1
    w, bias = torch.randn(D, V) * 0.05, torch.randn(1, V) * 0.1
    tg = torch.randint(0, V, (B, S))

    def loss(x, g, b, w, bias, tg):
        return F.cross_entropy_loss(F.linear(F.layer_norm(x, g, b), w, bias, activation="gelu"), tg)

    cpu = [nb.Tensor.from_torch(t) for t in (x, g, b, w, bias, tg)]
    lr, gr = nb.value_and_grad(loss, argnums=(0, 1, 2, 3, 4))(*cpu)
    dev = [nb.Tensor.from_torch(t.cuda().bfloat16() if t.is_floating_point() else t.cuda()) for t in (x, g, b, w, bias, tg)]
    c0, k0 = gemm.launch_count, kernels.launch_count
    lg, gg = nb.value_and_grad(loss, argnums=(0, 1, 2, 3, 4))(*dev)
    assert abs(lg.item() - lr.item()) / abs(lr.item()) < 3e-2
    assert gemm.launch_count > c0 and kernels.launch_count > k0
    for a, r in zip(gg, gr):
        assert _rel(torch.from_numpy(a.to_numpy()), torch.from_numpy(r.to_numpy())) < 8e-2
    # plan-level fusion of matmul + add + relu written with primitives
    c1 = gemm.launch_count
    y = nb.relu(dev[0] @ dev[3] + dev[4])
    y.realize()
    assert gemm.launch_count == c1 + 1
    ref = torch.relu(x.cuda().bfloat16().float() @ w.cuda().bfloat16().float() + bias.cuda().bfloat16().float())
    assert _rel(torch.from_numpy(y.to_numpy()), ref.cpu()) < 3e-2


def test_smoke_entry_and_cuda_graph_compile():
    import __graft_entry__ as ge
    import nabla_b200 as nb

    ge.smoke()
    f = nb.compile(lambda a, b: nb.relu(a @ b) * 2.0, cuda_graph=True)
    a = nb.Tensor.from_torch(torch.randn(256, 128, device="cuda", dtype=torch.bfloat16))
    b = nb.Tensor.from_torch(torch.randn(128, 64, device="cuda", dtype=torch.bfloat16))
    ref = (torch.relu(a.to_torch().float() @ b.to_torch().float()) * 2).cpu()
    for _ in range(3):
        out = f(a, b)
    assert _rel(torch.from_numpy(out.to_numpy()), ref) < 3e-2 and f.stats.fallbacks == 0


@pytest.mark.parametrize("B,H,S,D,causal", [(1, 1, 128, 128, False), (1, 2, 256, 128, True), (2, 2, 200, 128, True),
                                            (2, 3, 384, 64, True), (1, 2, 333, 64, False), (1, 2, 520, 128, True),
                                            (1, 2, 2048, 128, True), (1, 1, 1024, 64, False)])
def test_flash_attention_forward(B, H, S, D, causal):
    from nabla_b200 import native
    from nabla_b200.native import attention as A

    torch.manual_seed(6)
    q = torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16)
    k, v = torch.randn_like(q), torch.randn_like(q)
    assert A.supported(q, k, v, None, 0.0)
    o, lse = A.sdpa_fwd(q, k, v, causal=causal, scale=D ** -0.5)
    native.check_status()
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=causal)
    s = (q.float() @ k.float().transpose(-1, -2)) * D ** -0.5
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    assert (o.float() - ref).abs().max().item() < 3e-2
    assert (lse - torch.logsumexp(s, -1)).abs().max().item() < 1e-2


def test_flash_attention_cross_lengths():
    """seq_q != seq_kv, causal aligned to the last key (row i sees keys <= i + Skv - Sq)."""
    from nabla_b200.native import attention as A

    torch.manual_seed(8)
    B, H, Sq, Skv, D = 1, 2, 130, 300, 128
    q = torch.randn(B, H, Sq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, H, Skv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    for causal in (False, True):
        o, _ = A.sdpa_fwd(q, k, v, causal=causal, scale=D ** -0.5)
        s = (q.float() @ k.float().transpose(-1, -2)) * D ** -0.5
        if causal:
            s = s.masked_fill(~torch.ones(Sq, Skv, dtype=torch.bool, device="cuda").tril(Skv - Sq), float("-inf"))
        ref = torch.softmax(s, -1) @ v.float()
        assert (o.float() - ref).abs().max().item() < 3e-2


@pytest.mark.parametrize("B,H,S,D,causal", [(1, 1, 128, 128, False), (1, 2, 256, 128, True), (2, 2, 200, 128, True),
                                            (1, 2, 320, 128, False), (1, 2, 2048, 128, True), (2, 2, 200, 64, True),
                                            (1, 3, 384, 64, False), (1, 1, 1100, 128, True)])
def test_flash_attention_backward_and_packed(B, H, S, D, causal):
    from nabla_b200 import native
    from nabla_b200.native import attention as A

    torch.manual_seed(7)
    qkv = torch.randn(B, S, H * 3 * D, device="cuda", dtype=torch.bfloat16)
    v5 = qkv.view(B, S, H, 3, D)
    q, k, v = (v5[:, :, :, i, :].permute(0, 2, 1, 3) for i in range(3))      # strided views, no copies
    do = torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16)
    o, lse = A.sdpa_fwd(q, k, v, causal=causal, scale=D ** -0.5)
    dq, dk, dv = A.sdpa_bwd(do, q, k, v, o, lse, causal=causal, scale=D ** -0.5)
    native.check_status()
    qs = [t.float().requires_grad_(True) for t in (q, k, v)]
    torch.nn.functional.scaled_dot_product_attention(*qs, is_causal=causal).backward(do.float())
    for a, b in zip((dq, dk, dv), qs):
        assert _rel(a, b.grad) < 4e-2


@pytest.mark.parametrize("kind", ["float_bh", "bool_rows", "float_2d_causal"])
def test_flash_attention_additive_mask(kind):
    """Forward and backward with an additive / boolean mask against the fp32 composition."""
    from nabla_b200.native import attention as A

    torch.manual_seed(9)
    B, H, S, D = 2, 2, 200, 128
    q = torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16)
    k, v = torch.randn_like(q), torch.randn_like(q)
    do = torch.randn_like(q)
    causal = kind == "float_2d_causal"
    if kind == "float_bh":
        mask = torch.randn(B, H, S, S, device="cuda")
    elif kind == "bool_rows":
        mask = torch.rand(B, 1, 1, S, device="cuda") > 0.3          # key padding mask
        mask[..., 0] = True
    else:
        mask = torch.randn(S, S, device="cuda")
    assert A.supported(q, k, v, mask, 0.0)
    o, lse = A.sdpa_fwd(q, k, v, causal=causal, scale=D ** -0.5, mask=mask)
    dq, dk, dv = A.sdpa_bwd(do, q, k, v, o, lse, causal=causal, scale=D ** -0.5, mask=mask)
    qs = [t.float().requires_grad_(True) for t in (q, k, v)]
    s = (qs[0] @ qs[1].transpose(-1, -2)) * D ** -0.5
    add = torch.zeros_like(s).masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else mask
    s = s + add
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    ref = torch.softmax(s, -1) @ qs[2]
    ref.backward(do.float())
    assert (o.float() - ref).abs().max().item() < 3e-2
    for a, b in zip((dq, dk, dv), qs):
        assert _rel(a, b.grad) < 4e-2


def test_transformer_block_on_gpu_matches_cpu_reference():
    """The packed-attention transformer (all native kernels) against the same model on the CPU."""
    import nabla_b200 as nb
    from nabla_b200.models import transformer as TR
    from nabla_b200.native import attention as A

    cfg = TR.TransformerConfig(n_layers=2, d_model=256, n_heads=2, d_ff=512, vocab=512, max_seq=256)
    nb.seed(11)
    params = TR.init_params(cfg)
    rng = np.random.default_rng(3)
    tok, tgt = rng.integers(0, 512, (2, 256)), rng.integers(0, 512, (2, 256))
    cpu32 = nb.tree_map(lambda t: nb.Tensor.from_torch(t.to_torch().float()), params)
    cfg32 = TR.TransformerConfig(n_layers=2, d_model=256, n_heads=2, d_ff=512, vocab=512, max_seq=256, dtype=nb.DType.float32)
    l_ref, g_ref = nb.value_and_grad(lambda p: TR.loss_fn(p, nb.constant(tok), nb.constant(tgt), cfg32), create_graph=False)(cpu32)
    dev = nb.tree_map(lambda t: nb.Tensor.from_torch(t.to_torch().cuda()), params)
    n0 = A.launch_count
    l_dev, g_dev = nb.value_and_grad(lambda p: TR.loss_fn(p, nb.Tensor.from_torch(torch.from_numpy(tok).cuda()),
                                                          nb.Tensor.from_torch(torch.from_numpy(tgt).cuda()), cfg),
                                     create_graph=False)(dev)
    assert abs(l_dev.item() - l_ref.item()) / l_ref.item() < 2e-2
    assert A.launch_count >= n0 + 2 * (1 + 3)      # forward + backward attention kernels ran for both layers
    for a, b in zip(nb.tree_leaves(g_dev), nb.tree_leaves(g_ref)):
        ga, gb = torch.from_numpy(a.to_numpy()).float(), torch.from_numpy(b.to_numpy()).float()
        assert ((ga - gb).norm() / (gb.norm() + 1e-6)).item() < 0.1


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_status_watchdog_thread_reports_without_synchronising():
    """The C++ watchdog copies a status word to the host on its own stream: a non-zero code written
    on the device shows up in `watchdog_poll` although Python never reads the tensor."""
    import time

    from nabla_b200 import native

    dev = torch.device("cuda", 0)
    word = torch.zeros(4, dtype=torch.int32, device=dev)
    native.watchdog_start(dev, interval_ms=10, word=word)
    try:
        time.sleep(0.2)
        before = native.watchdog_poll(dev)
        assert before["code"] == 0 and before["polls"] > 0
        native.watchdog_check(dev)                      # nothing recorded: no exception
        word[0] = 4                                     # what a timed-out peer wait would store
        torch.cuda.synchronize()
        deadline = time.time() + 5.0
        while native.watchdog_poll(dev)["code"] == 0 and time.time() < deadline:
            time.sleep(0.02)
        assert native.watchdog_poll(dev)["code"] == 4
        with pytest.raises(native.KernelStatusError):
            native.watchdog_check(dev)
    finally:
        native.watchdog_stop(dev)


# ---------------------------------------------------------------- convolution on own kernels
@pytest.mark.parametrize("dtype,N,H,W,C,F,R,S,stride,pad", [
    (torch.float32, 2, 9, 8, 3, 5, 3, 3, (1, 1), (1, 1, 1, 1)),          # narrow channels: direct kernels
    (torch.float32, 3, 11, 7, 1, 4, 3, 2, (2, 2), (1, 0, 0, 1)),
    (torch.float32, 2, 8, 8, 2, 3, 2, 2, (1, 1), (2, 2, 2, 2)),          # padding beyond the filter reach
    (torch.bfloat16, 2, 12, 12, 16, 32, 3, 3, (1, 1), (1, 1, 1, 1)),     # wide channels: im2col + tcgen05 GEMM
    (torch.bfloat16, 2, 13, 10, 8, 16, 3, 3, (2, 1), (1, 1, 0, 0)),
])
def test_conv2d_forward_dgrad_wgrad_and_transpose_without_cudnn(dtype, N, H, W, C, F, R, S, stride, pad):
    """conv2d, its two gradients and conv2d_transpose on GPU against fp32 torch; torch's conv entry
    points are made to raise for the duration, so any library fallback fails the test."""
    import torch.nn.functional as TF
    from unittest import mock

    import nabla_b200 as nb

    torch.manual_seed(3)
    x = torch.randn(N, H, W, C, device="cuda")
    w = torch.randn(R, S, C, F, device="cuda") * 0.3
    if dtype == torch.bfloat16:                       # the reference sees exactly the values the kernels see
        x, w = x.bfloat16().float(), w.bfloat16().float()
    pt, pb, pl, pr = pad
    # reference in float64 on the CPU (GPU library convolutions may run in TF32)
    xp = TF.pad(x.cpu().double().permute(0, 3, 1, 2), (pl, pr, pt, pb)).requires_grad_(True)
    wt = w.cpu().double().permute(3, 2, 0, 1).clone().requires_grad_(True)
    y_ref = TF.conv2d(xp, wt, stride=stride)
    dy = torch.randn_like(y_ref)
    if dtype == torch.bfloat16:
        dy = dy.bfloat16().double()
    gx_ref, gw_ref = torch.autograd.grad(y_ref, (xp, wt), dy)
    gx_ref = gx_ref[:, :, pt:pt + H, pl:pl + W].permute(0, 2, 3, 1)
    gw_ref = gw_ref.permute(2, 3, 1, 0)
    xt_ref = TF.conv_transpose2d(dy, wt.detach(), stride=stride)           # transpose of the same conv
    xt_ref = xt_ref[:, :, pt:xt_ref.shape[2] - pb, pl:xt_ref.shape[3] - pr].permute(0, 2, 3, 1)
    y_ref = y_ref.detach()

    def guard(orig):
        def f(*a, **k):          # shape inference runs these on `meta` tensors; real data must not reach them
            if any(isinstance(t, torch.Tensor) and t.is_cuda for t in list(a) + list(k.values())):
                raise AssertionError("a torch / cuDNN convolution was called on the GPU path")
            return orig(*a, **k)
        return f

    xn, wn = nb.Tensor.from_torch(x.to(dtype)), nb.Tensor.from_torch(w.to(dtype))
    dyn = nb.Tensor.from_torch(dy.permute(0, 2, 3, 1).contiguous().to(device="cuda", dtype=dtype))
    with mock.patch.object(TF, "conv2d", guard(TF.conv2d)), mock.patch.object(TF, "conv_transpose2d", guard(TF.conv_transpose2d)), \
            mock.patch.object(torch.nn.grad, "conv2d_input", guard(torch.nn.grad.conv2d_input)), \
            mock.patch.object(torch.nn.grad, "conv2d_weight", guard(torch.nn.grad.conv2d_weight)):
        y, pull = nb.vjp(lambda a, b: nb.conv2d(a, b, stride=stride, padding=pad), xn, wn)
        gx, gw = pull(dyn)
        # conv2d_transpose with the filter read as (R, S, C_out = C, C_in = F)
        xt = nb.conv2d_transpose(dyn, wn, stride=stride, padding=pad)
        outs = [t.to_torch().double().cpu() for t in (y, gx, gw, xt)]
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    refs = [y_ref.permute(0, 2, 3, 1), gx_ref, gw_ref, xt_ref]
    for name, a, b in zip(("fwd", "dgrad", "wgrad", "transpose"), outs, refs):
        assert a.shape == b.shape, (name, a.shape, b.shape)
        assert _rel(a, b) < tol, (name, _rel(a, b))


def test_qlora_dequant_runs_the_native_kernel():
    import nabla_b200 as nb
    from nabla_b200.native import kernels
    from nabla_b200.nn import finetune

    torch.manual_seed(0)
    w = torch.randn(96, 200, device="cuda")
    q = finetune.quantize_nf4(nb.Tensor.from_torch(w), block_size=64)
    n0 = kernels.launch_count
    for dt in (nb.DType.float32, nb.DType.bfloat16):
        d = finetune.dequantize_nf4(q, dtype=dt).to_torch().float()
        code = torch.tensor(finetune.NF4_CODEBOOK, device="cuda")
        ref = (code[q["indices"].to_torch().long()].reshape(-1, 64) * q["scales"].to_torch().reshape(-1, 1)).reshape(-1)
        ref = ref[: w.numel()].reshape(w.shape)
        assert _rel(d, ref) < (1e-6 if dt is nb.DType.float32 else 1e-2)
    assert kernels.launch_count >= n0 + 2                      # one launch per dequantisation
    assert (finetune.dequantize_nf4(q).to_torch() - w).abs().mean().item() < 0.1


def test_random_ops_use_the_device_stream():
    """uniform / gaussian run the Philox kernel on the device-resident stream position: values are
    in range, consecutive draws differ, re-seeding reproduces them."""
    import nabla_b200 as nb
    from nabla_b200.native import kernels

    dev = nb.Accelerator(0)
    n0 = kernels.launch_count
    nb.seed(77)
    a = nb.uniform((1000, 64), 2.0, 5.0, device=dev).to_torch()
    b = nb.uniform((1000, 64), 2.0, 5.0, device=dev).to_torch()
    g = nb.gaussian((4000, 64), 1.0, 3.0, dtype=nb.DType.bfloat16, device=dev).to_torch().float()
    assert kernels.launch_count >= n0 + 3
    assert a.min() >= 2.0 and a.max() < 5.0 and abs(a.mean().item() - 3.5) < 0.02
    assert (a != b).float().mean().item() > 0.99
    assert abs(g.mean().item() - 1.0) < 0.05 and abs(g.std().item() - 3.0) < 0.05
    nb.seed(77)
    a2 = nb.uniform((1000, 64), 2.0, 5.0, device=dev).to_torch()
    assert torch.equal(a, a2)


def test_dropout_in_a_cuda_graph_draws_new_masks():
    import nabla_b200 as nb

    nb.seed(9)
    x = nb.Tensor.from_torch(torch.ones(256, 256, device="cuda", dtype=torch.bfloat16))
    g = nb.compile(lambda t: nb.nn.functional.dropout(t, p=0.5, training=True) * 1.0, cuda_graph=True)
    outs = [g(x).to_torch().float().clone() for _ in range(4)]
    assert g.stats.cuda_graphs == 1 and g.stats.fallbacks == 0
    for a, b in zip(outs[1:], outs[2:]):                        # replays of the captured graph
        assert (a != b).float().mean().item() > 0.2
    for o in outs:
        assert abs(o.mean().item() - 1.0) < 0.05 and set(o.unique().tolist()) <= {0.0, 2.0}


def test_custom_cuda_kernel_from_source(tmp_path):
    """call_custom_kernel on a .cu file: compiled with nvcc for sm_100a on first use, then launched
    on the current stream (reference: nabla/ops/utils.py:765-824 with a Mojo kernel package)."""
    from nabla_b200.ops import custom

    src = tmp_path / "scale_add.cu"
    src.write_text('''
#include "nabla_custom_kernel.h"
#include <cuda_runtime.h>
__global__ void k(const float* a, const float* b, float* o, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) o[i] = 2.f * a[i] + b[i];
}
extern "C" int scale_add(const NbTensor* in, int n_in, NbTensor* out, int n_out, void* stream) {
  if (n_in != 2 || n_out != 1 || in[0].dtype != NB_F32) return 1;
  long long n = in[0].numel;
  k<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)in[0].data, (const float*)in[1].data,
                                                                 (float*)out[0].data, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
''')
    a = torch.randn(1000, device="cuda")
    b = torch.randn(1000, device="cuda")
    n0 = custom.launch_count
    out = custom.call_custom_kernel("scale_add", str(src), [a, b], ((1000,), torch.float32))
    torch.cuda.synchronize()
    assert custom.launch_count == n0 + 1
    assert torch.allclose(out, 2 * a + b)
    with pytest.raises(KeyError):
        custom.call_custom_kernel("no_such_kernel", str(src), [a, b], ((1000,), torch.float32))


@pytest.mark.parametrize("M,N,K", [(130, 264, 72), (257, 520, 136), (129, 8, 64)])
def test_gemm_tail_tiles_elementwise(M, N, K):
    """Per-element check with an absolute tolerance: a wrong tail tile of small magnitude cannot
    hide behind the maximum of the whole matrix. Small integers make the fp32 reference exact."""
    from nabla_b200.native.gemm import gemm_bf16

    torch.manual_seed(1)
    a = torch.randint(-3, 4, (M, K), device="cuda").to(torch.bfloat16)
    b = torch.randint(-3, 4, (K, N), device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float()
    for layout in ("NN", "NT", "TN"):
        aa = a if layout[0] == "N" else a.t().contiguous().t()
        bb = b if layout[1] == "N" else b.t().contiguous().t()
        out = gemm_bf16(aa, bb, out_dtype=torch.float32)
        bad = (out - ref).abs() > 1e-3
        assert not bad.any(), (layout, bad.nonzero()[:4].tolist())


@pytest.mark.parametrize("M,N,K,layout", [(2048, 2048, 16384, "TN"), (2048, 1536, 65536, "TN"), (512, 2048, 65536, "TN"),
                                          (1024, 1024, 8192, "NN"), (640, 776, 4096, "NT")])
def test_gemm_split_k_matches_fp32(M, N, K, layout):
    """Weight-gradient-shaped GEMMs (few output tiles, long K) run as K slices + one summing pass;
    the result must equal the unsplit kernel's and the fp32 reference."""
    from nabla_b200.native import gemm as G

    torch.manual_seed(2)
    a = (torch.randn(K, M, device="cuda", dtype=torch.bfloat16).t() if layout[0] == "T"
         else torch.randn(M, K, device="cuda", dtype=torch.bfloat16))
    b = (torch.randn(N, K, device="cuda", dtype=torch.bfloat16).t() if layout[1] == "T"
         else torch.randn(K, N, device="cuda", dtype=torch.bfloat16))
    ref = a.float() @ b.float()
    if K == 65536:
        assert G.split_k_factor(M, N, K) > 1           # the tensor-parallel weight-gradient shapes do split
    for sk in (None, 2, 4):
        for od in (torch.bfloat16, torch.float32):
            out = G.gemm_bf16(a, b, out_dtype=od, split_k=sk)
            assert out.dtype == od and _rel(out, ref) < (1e-2 if od == torch.bfloat16 else 1e-4)
    plain = G.gemm_bf16(a, b, out_dtype=torch.float32, split_k=1)
    assert _rel(G.gemm_bf16(a, b, out_dtype=torch.float32), plain) < 1e-4


# ---------------------------------------------------------------- pointwise / reduction families
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pointwise_binary_family(dtype):
    from nabla_b200.native import kernels

    torch.manual_seed(4)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    a = torch.randn(37, 5, 24, device="cuda").to(dtype)
    for bshape in ((37, 5, 24), (1,), (24,), (5, 24), (1, 1, 24)):
        b = (torch.rand(bshape, device="cuda") + 0.5).to(dtype)
        for op, ref in (("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div),
                        ("maximum", torch.maximum), ("minimum", torch.minimum)):
            for x, y in ((a, b), (b, a)):                      # the smaller operand on either side
                out = kernels.binary(x, y, op)
                assert out is not None, (op, bshape)
                want = ref(x.float(), y.float())
                assert out.shape == want.shape and _rel(out, want) < tol, (op, bshape)
    assert kernels.binary(a, torch.randn(5, 1, device="cuda").to(dtype), "add") is None      # general broadcast: not covered
    odd = torch.randn(1003, device="cuda").to(dtype)                                          # tail that is not a whole vector
    assert _rel(kernels.binary(odd, odd, "mul"), odd.float() ** 2) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pointwise_unary_family(dtype):
    from nabla_b200.native import kernels

    torch.manual_seed(5)
    x = (torch.rand(129, 77, device="cuda") * 3 + 0.1).to(dtype)
    refs = {"neg": torch.neg, "abs": torch.abs, "exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt,
            "tanh": torch.tanh, "sigmoid": torch.sigmoid, "sin": torch.sin, "cos": torch.cos, "erf": torch.erf,
            "log1p": torch.log1p, "floor": torch.floor, "trunc": torch.trunc, "round": torch.round,
            "square": torch.square, "reciprocal": torch.reciprocal}
    for op, ref in refs.items():
        for inp in (x, -x if op not in ("log", "sqrt", "rsqrt", "log1p") else x):
            out = kernels.unary(inp, op)
            want = ref(inp.float())
            assert (out.float() - want).abs().max().item() <= (2e-6 if dtype == torch.float32 else 1.6e-2) * (1 + want.abs().max().item()), op


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduction_family(dtype):
    from nabla_b200.native import kernels

    torch.manual_seed(6)
    x = torch.randn(9, 130, 33, device="cuda").to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for axis in (0, 1, 2, -1):
        for keep in (False, True):
            assert _rel(kernels.reduce(x, axis, "sum", keep), x.float().sum(axis, keepdim=keep)) < tol
            assert _rel(kernels.reduce(x, axis, "mean", keep), x.float().mean(axis, keepdim=keep)) < tol
            assert torch.equal(kernels.reduce(x, axis, "max", keep), x.amax(axis, keepdim=keep))
            assert torch.equal(kernels.reduce(x, axis, "min", keep), x.amin(axis, keepdim=keep))
            assert torch.equal(kernels.reduce(x, axis, "argmax", keep), x.float().argmax(axis, keepdim=keep))
            assert torch.equal(kernels.reduce(x, axis, "argmin", keep), x.float().argmin(axis, keepdim=keep))
    wide = torch.randn(7, 5000, device="cuda").to(dtype)                   # block-per-row path, vector loads
    assert _rel(kernels.reduce(wide, 1, "sum"), wide.float().sum(1)) < tol
    assert torch.equal(kernels.reduce(wide, 1, "argmax"), wide.float().argmax(1))
    nan = wide.clone()
    nan[3, 17] = float("nan")
    assert torch.isnan(kernels.reduce(nan, 1, "max")[3]) and not torch.isnan(kernels.reduce(nan, 1, "max")[2])
    tall = torch.randn(6000, 64, device="cuda").to(dtype)                   # few long columns -> slab column sum
    assert _rel(kernels.reduce(tall, 0, "sum"), tall.float().sum(0)) < tol
    for axis in (0, 1, 2):
        for excl in (False, True):
            for rev in (False, True):
                ref = x.float().flip(axis).cumsum(axis).flip(axis) if rev else x.float().cumsum(axis)
                if excl:
                    ref = ref - x.float()
                got = kernels.cumsum(x, axis, excl, rev)
                assert _rel(got, ref) < (1e-5 if dtype == torch.float32 else 5e-2), (axis, excl, rev)


def test_ops_route_through_the_pointwise_and_reduction_kernels():
    """The framework's ops (not only the wrappers) launch these kernels for GPU tensors."""
    import nabla_b200 as nb
    from nabla_b200.native import kernels

    x = nb.Tensor.from_torch(torch.randn(64, 48, device="cuda"))
    n0 = kernels.launch_count
    y = nb.reduce_sum(nb.exp(x) * 2.0 + x, axis=1)
    z = nb.argmax(x, axis=0)
    y.realize(); z.realize()
    assert kernels.launch_count >= n0 + 5
    xt = x.to_torch()
    assert _rel(y.to_torch(), (xt.exp() * 2 + xt).sum(1)) < 1e-5
    assert torch.equal(z.to_torch(), xt.argmax(0))
