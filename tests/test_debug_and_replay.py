"""Substitutes for a race detector / sanitizer: the bounds-checked debug build of the kernels and the
deterministic-replay mode. The CPU cases cover the build plumbing, the record decoding and the replay
comparison; the GPU cases load the checked build in a child process (the choice of build is made at
import time) and run real kernels through it."""
import itertools
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import nabla_b200 as nb
from nabla_b200 import config
from nabla_b200.utils.replay import replay_check

ROOT = Path(__file__).resolve().parent.parent


# ---------------------------------------------------------------- debug build: host side
def test_debug_build_compiles_every_library_with_the_check_macro():
    from nabla_b200.csrc import build

    libs = build.build_all(debug=True)
    names = {p.name for p in libs}
    assert {"libnb_gemm.so", "libnb_kernels.so", "libnb_attention.so", "libnb_comm.so"} <= names
    assert all(p.parent.name == "debug" for p in libs)
    import ctypes

    for lib, units in (("libnb_gemm.so", ("gemm",)), ("libnb_kernels.so", ("fused", "elementwise")),
                       ("libnb_attention.so", ("attention",)), ("libnb_comm.so", ("comm",))):
        dbg = ctypes.CDLL(str(build.LIB / "debug" / lib))
        rel = ctypes.CDLL(str(build.build_all()[0].parent / lib))
        for tu in units:
            assert getattr(dbg, f"nb_debug_enabled_{tu}")() == 1
            assert getattr(rel, f"nb_debug_enabled_{tu}")() == 0


def test_every_kernel_source_includes_the_check_header_and_uses_it():
    csrc = ROOT / "nabla_b200" / "csrc"
    for name in ("gemm_tcgen05.cu", "attention_tcgen05.cu", "peer_collectives.cu", "fused_kernels.cu",
                 "elementwise_kernels.cu"):
        src = (csrc / name).read_text()
        assert '#include "nb_debug.cuh"' in src and "NB_DEBUG_DEFINE(" in src
        assert src.count("NB_IN_BOUNDS(") + src.count("NB_ALIGNED(") >= 3, name
    header = (csrc / "nb_debug.cuh").read_text()
    # the release build turns both macros into the constant `true`
    assert "#define NB_IN_BOUNDS(site, value, limit) true" in header
    assert "#define NB_ALIGNED(site, value, align) true" in header


def test_site_table_matches_the_header():
    from nabla_b200 import native

    header = (ROOT / "nabla_b200" / "csrc" / "nb_debug.cuh").read_text()
    import re

    sites = {int(v) for v in re.findall(r"NB_SITE_\w+ = (\d+),", header)}
    assert sites == set(native._DEBUG_SITES)


def test_release_build_reports_nothing():
    from nabla_b200 import native

    if not native.DEBUG_KERNELS:
        assert native.debug_report() is None
        native.debug_check()


# ---------------------------------------------------------------- deterministic replay: host side
def test_deterministic_flag_is_a_scoped_contextvar():
    assert config.DETERMINISTIC is False and not config.is_deterministic()
    with config.deterministic():
        assert config.DETERMINISTIC is True
        with config.deterministic(False):
            assert not config.is_deterministic()
        assert config.is_deterministic()
    assert not config.is_deterministic()


def _step(p, x):
    loss, g = nb.value_and_grad(lambda q: nb.reduce_sum(nb.tanh(x @ q["w"]) ** 2.0))(p)
    return loss, {"w": p["w"] - 0.1 * g["w"]}


def test_replay_check_passes_for_a_pure_step_eager_and_compiled():
    p = {"w": nb.constant(np.random.randn(8, 4).astype(np.float32))}
    x = nb.constant(np.random.randn(16, 8).astype(np.float32))
    w0 = p["w"].to_numpy().copy()
    rep = replay_check(_step, p, x)
    assert rep.ok and rep.runs == 3 and rep.leaves == 4 and not rep.mismatches
    assert replay_check(nb.compile(_step), p, x, repeats=4)
    assert np.array_equal(p["w"].to_numpy(), w0)            # the caller's arguments are untouched


def test_replay_check_reports_a_run_to_run_difference():
    cnt = itertools.count()
    x = nb.constant(np.ones((4, 4), dtype=np.float32))
    rep = replay_check(lambda t: t + float(next(cnt)), x, check_args=False)
    assert not rep.ok and len(rep.mismatches) == 2
    m = rep.mismatches[0]
    assert (m.run, m.leaf, m.shard, m.n_diff, m.first_index) == (1, "out", 0, 16, 0) and m.max_abs_diff == 1.0
    assert "run 1" in rep.summary()


def test_replay_check_restarts_the_random_stream():
    x = nb.constant(np.zeros((8, 8), dtype=np.float32))
    assert replay_check(lambda t: t + nb.uniform((8, 8)), x)


def test_replay_check_compares_bits_not_values():
    flip = itertools.cycle([0.0, -0.0])
    x = nb.constant(np.zeros((2,), dtype=np.float32))
    rep = replay_check(lambda t: nb.constant(np.full((2,), next(flip), dtype=np.float32)), x, repeats=2, check_args=False)
    assert not rep.ok and rep.mismatches[0].max_abs_diff == 0.0


def test_compile_keeps_separate_entries_for_deterministic_mode():
    c = nb.compile(lambda t: t * 2.0)
    x = nb.constant(np.ones((4,), dtype=np.float32))
    c(x)
    with config.deterministic():
        c(x)
        c(x)
    assert c.stats.misses == 2 and c.stats.hits == 1


# ---------------------------------------------------------------- on a GPU, checked build in a child process
_CHILD = r"""
import json, os, sys
import torch
import nabla_b200 as nb
from nabla_b200 import native, config
from nabla_b200.native import kernels, gemm, attention
assert native.DEBUG_KERNELS
out = {}
torch.manual_seed(0)
dev = "cuda"
# real kernels through the checked build, in-range data only: results match fp32 references, record stays clean
a = torch.randn(333, 136, device=dev, dtype=torch.bfloat16); b = torch.randn(136, 520, device=dev, dtype=torch.bfloat16)
c = gemm.gemm_bf16(a, b)
out["gemm"] = ((c.float() - a.float() @ b.float()).abs().max() / (a.float() @ b.float()).abs().max()).item()
# a shape wide enough for the CTA-pair kernel, with an odd number of 128-row tiles and a ragged last column tile
a2 = torch.randn(4224, 320, device=dev, dtype=torch.bfloat16); b2 = torch.randn(320, 4616, device=dev, dtype=torch.bfloat16)
c2 = gemm.gemm_bf16(a2, b2)
out["gemm_pair"] = ((c2.float() - a2.float() @ b2.float()).abs().max() / (a2.float() @ b2.float()).abs().max()).item()
out["pair_ran"] = native.load("libnb_gemm.so").nb_gemm_pair_max_clusters() > 0
q, k, v = (torch.randn(2, 4, 300, 64, device=dev, dtype=torch.bfloat16) for _ in range(3))
o, lse = attention.sdpa_fwd(q, k, v, causal=True, scale=64 ** -0.5)
ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True)
out["attn"] = (o.float() - ref).abs().max().item()
do = torch.randn_like(o)
dq, dk, dv = attention.sdpa_bwd(do, q, k, v, o, lse, causal=True, scale=64 ** -0.5)
qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True).backward(do.float())
out["attn_bwd"] = max((dq.float() - qf.grad).abs().max().item(), (dk.float() - kf.grad).abs().max().item(),
                      (dv.float() - vf.grad).abs().max().item())
x = torch.randn(37, 200, device=dev)
out["softmax"] = (kernels.softmax(x) - torch.softmax(x, -1)).abs().max().item()
tab = torch.randn(50, 24, device=dev); ids = torch.randint(0, 50, (7, 9), device=dev)
out["gather"] = (kernels.embedding_gather(tab, ids) - tab[ids]).abs().max().item()
xs = torch.randn(3, 70, 33, device=dev)
out["reduce"] = (kernels.reduce(xs, 1, "sum") - xs.sum(1)).abs().max().item()
out["binary"] = (kernels.binary(xs, xs, "mul") - xs * xs).abs().max().item()
img = torch.randn(2, 9, 8, 5, device=dev)
dy = torch.randn(2, 5, 5, 5, device=dev)
ir = img.cpu().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
torch.nn.functional.max_pool2d(ir, (3, 2), (2, 2), padding=(1, 1)).backward(dy.cpu().permute(0, 3, 1, 2).contiguous())
out["pool_bwd"] = (kernels.pool2d_bwd(img, dy, 3, 2, 2, 2, 1, 1, "max").cpu() - ir.grad.permute(0, 2, 3, 1)).abs().max().item()
# deterministic scatter-add: identical bits on every call, equal to the fp32 reference
upd = torch.randn(7, 9, 24, device=dev)
ids[0, :5] = 3                     # a long run of equal ids
with config.deterministic():
    s1 = kernels.embedding_scatter_add(tab, ids, upd)
    s2 = kernels.embedding_scatter_add(tab, ids, upd)
refs = tab.clone().index_add_(0, ids.view(-1), upd.view(-1, 24))
out["scatter_equal"] = bool(torch.equal(s1, s2))
out["scatter"] = (s1 - refs).abs().max().item()
torch.cuda.synchronize()
native.check_status()
out["clean"] = native.debug_report() is None
# a failed check reaches the record: the self-test kernel evaluates the macros on numbers and touches no memory
for lib in ("libnb_gemm.so", "libnb_kernels.so", "libnb_attention.so", "libnb_comm.so"):
    native.debug_selftest(lib, 3, 8, 64, 16)
out["selftest_pass"] = native.debug_report() is None
native.debug_selftest("libnb_kernels.so", 12, 8, 64, 16)
rep = native.debug_report()
out["bounds"] = rep
native.debug_selftest("libnb_gemm.so", 3, 8, 40, 16)
out["align"] = native.debug_report()
native.debug_selftest("libnb_attention.so", -1, 8, 0, 16)
try:
    native.debug_check()
    out["raised"] = False
except native.KernelDebugCheckFailed as e:
    out["raised"] = str(e)
out["after"] = native.debug_report() is None
print("RESULT " + json.dumps(out))
"""


@pytest.mark.gpu
def test_checked_build_runs_the_kernels_and_records_failed_checks():
    from nabla_b200.csrc import build

    build.build_all(debug=True)
    env = dict(os.environ, NABLA_B200_DEBUG_KERNELS="1", PYTHONPATH=str(ROOT))
    res = subprocess.run([sys.executable, "-c", _CHILD], capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert out["gemm"] < 1e-2 and out["attn"] < 3e-2 and out["attn_bwd"] < 8e-2
    assert out["gemm_pair"] < 1e-2 and out["pair_ran"]
    for k in ("softmax", "gather", "reduce", "binary", "pool_bwd", "scatter"):
        assert out[k] < 1e-4, (k, out[k])
    assert out["scatter_equal"] and out["clean"] and out["selftest_pass"]
    assert out["bounds"]["code"] == 5 and out["bounds"]["site"] == 5 and out["bounds"]["value"] == 12
    assert out["bounds"]["limit"] == 8 and out["bounds"]["count"] == 2          # both units of the library
    assert out["align"]["code"] == 6 and out["align"]["value"] == 40 and out["align"]["limit"] == 16
    assert "value -1" in out["raised"] and out["after"]


@pytest.mark.gpu
@pytest.mark.parametrize("cuda_graph", [False, True])
def test_replay_check_of_a_compiled_transformer_step_on_gpu(cuda_graph):
    from nabla_b200 import nn
    from nabla_b200.models import transformer as T

    cfg = T.TransformerConfig(n_layers=2, d_model=256, n_heads=2, d_ff=1024, vocab=1024, max_seq=256)
    with nb.default_device(nb.Accelerator(0)):
        nb.seed(0)
        params = T.init_params(cfg)
        state = nn.adamw_init(params, state_dtype=nb.DType.float32)
        rng = np.random.default_rng(0)
        tok = nb.constant(rng.integers(0, cfg.vocab, (4, 256)), device=nb.Accelerator(0))
        tgt = nb.constant(rng.integers(0, cfg.vocab, (4, 256)), device=nb.Accelerator(0))

        def step(p, st, a, b):
            loss, grads = nb.value_and_grad(lambda q: T.loss_fn(q, a, b, cfg), create_graph=False)(p)
            p2, st2 = nn.adamw_update(p, grads, st, lr=1e-3)
            return loss, p2, st2

        with config.deterministic():
            compiled = nb.compile(step, donate_argnums=(0, 1), cuda_graph=cuda_graph)
            rep = replay_check(compiled, params, state, tok, tgt, repeats=3)
        assert rep.ok, rep.summary()
        assert rep.leaves > 20
