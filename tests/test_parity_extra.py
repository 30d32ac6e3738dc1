"""Extra parity checks modelled on the reference's unit-test areas: Hessians through all four
jacfwd/jacrev compositions, a CNN toy training run, context-variable isolation across threads,
custom pytree nodes, slice assignment, and vmap over collectives."""
import threading

import numpy as np
import pytest
import torch

import nabla_b200 as nb

from common import T, close, rand


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


# ---------------------------------------------------------------- control flow on sharded state
def test_while_loop_with_sharded_state(mesh_2x4):
    """Loop-carried state split over a mesh axis stays sharded through the loop
    (reference: tests/unit/test_control_flow.py:246)."""
    x = np.arange(32, dtype=np.float32).reshape(8, 4)
    xs = nb.shard(nb.constant(x), mesh_2x4, nb.P("dp", None))
    i, out = nb.while_loop(lambda i, v: i < 5.0, lambda i, v: (i + 1.0, v + 1.0), (nb.constant(np.float32(0)), xs))
    assert i.item() == 5.0 and tuple(int(d) for d in out.shape) == (8, 4)
    assert out.is_sharded
    np.testing.assert_allclose(out.to_numpy(), x + 5.0)


def test_cond_and_compiled_while_on_sharded_operands(mesh_2x4):
    x = np.arange(16, dtype=np.float32).reshape(8, 2)
    xs = nb.shard(nb.constant(x), mesh_2x4, nb.P("dp", None))
    r = nb.cond(nb.reduce_sum(xs) > 0.0, lambda a: a * 2.0, lambda a: a - 1.0, xs)
    np.testing.assert_allclose(r.to_numpy(), x * 2.0)
    f = nb.compile(lambda v: nb.while_loop(lambda t: nb.reduce_sum(t) < 500.0, lambda t: t * 2.0 + 1.0, v))
    for scale in (1.0, 0.1, 1.0):
        got = f(nb.shard(nb.constant(x * scale), mesh_2x4, nb.P("dp", None))).to_numpy()
        ref = x * scale
        while ref.sum() < 500.0:
            ref = ref * 2.0 + 1.0
        np.testing.assert_allclose(got, ref, rtol=1e-6)
    assert f.stats.misses == 1


# ---------------------------------------------------------------- introspection, graph walks, debug streams, exports
def test_tensor_impl_introspection_and_graph_walks(capsys):
    from nabla_b200.core.graph import utils

    x = nb.constant(np.ones((2, 3), dtype=np.float32))
    y = nb.relu(x * 2.0) + 1.0
    im = y._impl
    assert im.op_name == "add" and not im.is_leaf and x._impl.is_leaf and x._impl.op is None
    assert [p.op_name for p in im.parents][0] == "relu" and im.ndim == 2
    assert tuple(im.local_shape) == (2, 3) and tuple(im.logical_shape) == (2, 3) and im.global_shape_ints == (2, 3)
    ops = utils.get_operations_topological(y)
    assert [outs[0].op_name for _, outs in ops] == ["mul", "relu", "add"]
    impls = utils.get_all_impls_topological([y])
    assert impls[-1] is im and x._impl in impls
    seen = []
    utils.apply_to_operations(y, lambda op_id, outs: seen.append(outs[0].op_name))
    assert seen == ["add", "relu", "mul"]
    utils.print_trace_graph(y)
    assert "Computation Graph (3 operations)" in capsys.readouterr().out


def test_debug_streams_print_when_switched_on(monkeypatch, capsys):
    for name in ("OP_CALL", "PHYS", "COT_FLOW", "PHYS_VJP", "NESTED_JVP"):
        monkeypatch.setenv("NABLA_DEBUG_" + name, "1")
    x = nb.constant(np.ones((2, 3), dtype=np.float32))
    nb.grad(lambda a: nb.reduce_sum(a * a))(x).realize()
    nb.jvp(lambda a: a * a, (x,), (x,))
    out = capsys.readouterr().out
    for tag in ("[NABLA_DEBUG_OP_CALL] op=mul", "[NABLA_DEBUG_PHYS] mul.infer_outputs", "[NABLA_DEBUG_COT_FLOW] init",
                "[NABLA_DEBUG_PHYS_VJP] reduce_sum.vjp", "[NABLA_DEBUG_NESTED_JVP]"):
        assert tag in out, tag
    for name in ("OP_CALL", "PHYS", "COT_FLOW", "PHYS_VJP", "NESTED_JVP"):
        monkeypatch.delenv("NABLA_DEBUG_" + name)
    nb.grad(lambda a: nb.reduce_sum(a * a))(x).realize()
    assert "NABLA_DEBUG" not in capsys.readouterr().out


def test_reexports_and_path_names():
    from nabla_b200.core.common import pytree
    from nabla_b200.nn import finetune, functional as F
    from nabla_b200.ops import communication as C

    for name in ("relu", "gelu", "sigmoid", "tanh", "softmax", "silu"):
        assert callable(getattr(F, name))
    assert finetune.adamw_init is nb.nn.adamw_init and finetune.adamw_update is nb.nn.adamw_update
    for name in ("shard_op", "all_gather_op", "gather_all_axes_op", "all_reduce_op", "pmean_op", "reduce_scatter_op",
                 "ppermute_op", "all_to_all_op", "distributed_broadcast_op", "axis_index_op", "CollectiveOperation"):
        assert hasattr(C, name), name
    assert C.all_reduce_op.name == "all_reduce" and C.pmean_op.name == "pmean"
    leaves, names, td = pytree.tree_flatten_with_names({"b": [1, (2, 3)], "a": {"x": 4}})
    assert leaves == [4, 1, 2, 3] and names == ["a.x", "b[0]", "b[1][0]", "b[1][1]"]
    assert pytree.leaf_names(td, "lora") == ["lora.a.x", "lora.b[0]", "lora.b[1][0]", "lora.b[1][1]"]


def test_names_the_reference_tests_import_resolve_here():
    """Every name that the reference's unit tests and examples import from `nabla...` resolves under
    `nabla_b200...` (private context variables, op classes, helper functions)."""
    import importlib

    wanted = {
        "": ["metadata"],
        ".config": ["_EAGER_MAX_GRAPH", "_VERIFY_EAGER_SHAPES", "_TRACING", "tracing_context"],
        ".core": ["ComputeGraph", "apply_to_operations", "get_all_impls_topological", "get_operations_topological",
                  "print_trace_graph", "driver_tensor_type", "_in_running_loop"],
        ".core.common": ["_in_running_loop", "tree_flatten_full", "tree_unflatten_full"],
        ".core.graph": ["apply_to_operations", "driver_tensor_type", "get_all_impls_topological",
                        "get_operations_topological"],
        ".core.graph.engine": ["_CURRENT_GRAPH", "_get_current_graph", "_GraphProxy", "ComputeGraph", "GRAPH"],
        ".nn.modules.base": ["_MODULE_CALL_DEPTH"],
        ".ops": ["BinaryOp", "UnaryOp", "ReduceOp", "CreationOp", "CollectiveOp", "_make_hashable", "_get_tensor_hash",
                 "_clear_hashable_cache", "shard", "reshard", "all_reduce", "all_gather", "all_to_all", "reduce_scatter",
                 "ppermute", "cpu", "gpu", "accelerator", "to_device", "transfer_to", "distributed_broadcast", "cond",
                 "scan", "where", "while_loop", "conv2d", "conv2d_transpose", "avg_pool2d", "max_pool2d"],
        ".ops.view": ["SqueezePhysicalOp", "squeeze_physical", "unsqueeze_physical"],
        ".ops.reduction": ["reduce_max_physical", "reduce_min_physical", "reduce_sum_physical", "mean_physical"],
        ".ops.communication": ["AllGatherOp", "AllReduceOp", "ReduceScatterOp", "all_gather", "reshard"],
        ".ops.custom_op": ["call_custom_kernel"],
        ".transforms.utils": ["std_basis", "lift_basis_to_batch_prefix"],
        ".ops.reduction ": ["MeanOp", "MeanPhysicalOp"],
        ".ops.view.axes": ["MoveAxisOp"],
        ".ops.view.batch": ["MoveAxisPhysicalOp"],
        ".core.tensor.api": ["GRAPH", "default_device", "default_dtype", "defaults", "defaults_like"],
        ".ops.communication.all_gather": ["AllGatherOp", "GatherAllAxesOp", "all_gather", "gather_all_axes"],
        ".ops.communication.all_reduce": ["AllReduceOp", "PMeanOp", "all_reduce", "pmean"],
        ".ops.communication.all_to_all": ["AllToAllOp", "all_to_all"],
        ".ops.communication.axis_index": ["AxisIndexOp", "axis_index"],
        ".ops.communication.base": ["CollectiveOperation"],
        ".ops.communication.broadcast": ["DistributedBroadcastOp", "distributed_broadcast"],
        ".ops.communication.p_permute": ["PPermuteOp", "ppermute"],
        ".ops.communication.reduce_scatter": ["ReduceScatterOp", "reduce_scatter"],
        ".ops.communication.reshard": ["reshard", "reshard_tensor", "create_replicated_spec"],
        ".ops.communication.shard": ["ShardOp", "create_replicated_spec", "shard", "broadcast"],
        ".ops.communication.transfer": ["TransferOp", "to_device", "transfer_to", "cpu", "gpu", "accelerator"],
    }
    for mod, names in wanted.items():
        m = importlib.import_module("nabla_b200" + mod.strip())
        for n in names:
            assert hasattr(m, n), f"nabla_b200{mod}.{n}"


def test_physical_extreme_reductions_and_basis_helpers():
    from nabla_b200.ops.reduction import reduce_max_physical, reduce_min_physical
    from nabla_b200.ops.view import broadcast_batch_dims
    from nabla_b200.transforms.utils import lift_basis_to_batch_prefix, std_basis

    x0 = rand(2, 3, 4, seed=91)
    for red, tred, axis in ((reduce_max_physical, torch.amax, 2), (reduce_min_physical, torch.amin, 1)):
        f = lambda t: nb.reduce_sum(red(t * t + 0.1, axis=axis))
        xt = x0.clone().requires_grad_(True)
        tred(xt * xt + 0.1, axis).sum().backward()
        close(nb.grad(f)(T(x0)), xt.grad, rtol=1e-5, atol=1e-5)
        hs = [h(T(x0)).to_numpy() for h in (nb.jacrev(nb.jacrev(f)), nb.jacfwd(nb.jacrev(f)), nb.jacrev(nb.jacfwd(f)),
                                             nb.jacfwd(nb.jacfwd(f)))]
        for h in hs[1:]:
            np.testing.assert_allclose(h, hs[0], rtol=5e-3, atol=5e-3)
    ref = broadcast_batch_dims(T(torch.tensor([1.0, 2.0, 3.0])), (4,))
    sizes, basis = std_basis([ref])
    assert sizes == [3] and basis[0].batch_dims == 0
    lifted = lift_basis_to_batch_prefix(basis, [ref])
    assert lifted[0].batch_dims == ref.batch_dims
    assert tuple(lifted[0]._impl.physical_global_shape[:1]) == tuple(ref._impl.physical_global_shape[:1]) == (4,)
    assert lift_basis_to_batch_prefix(lifted, [ref])[0].batch_dims == 1       # already lifted: left alone
    x = T(torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    for jac in (nb.jacrev, nb.jacfwd):
        j = nb.vmap(jac(lambda v: nb.reduce_sum(v * v * v)))(x)
        assert j.batch_dims == 0 and tuple(int(d) for d in j.shape) == (2, 2)
        close(j, 3.0 * x.to_numpy() ** 2, rtol=1e-5)


def test_small_members_the_reference_exposes_on_its_classes():
    import nabla_b200.ops.binary as B
    from nabla_b200.core.graph.engine import GRAPH, _get_current_graph

    x = T(torch.ones(2, 3))
    y = x * 2.0
    with pytest.raises(TypeError):
        (x * 3.0).driver_tensor                       # a promise has no storage yet
    assert y.hydrate().real and len(y.values) == 1 and tuple(y.driver_tensor.shape) == (2, 3)
    assert y.type[0] == (2, 3)
    g = _get_current_graph()
    assert GRAPH.graph is g.graph and GRAPH.sources is g.sources
    node = (x * 2.0)._impl.output_refs
    assert node.num_outputs == 1 and len(node.get_alive_outputs()) == 1 and len(node.op_args) == 2
    mesh = nb.DeviceMesh("m4", (2, 2), ("a", "b"))
    assert mesh.axis_lookup == {"a": 0, "b": 1} and mesh.phys_strides == [2, 1] and mesh.get_signal_buffers() == []
    spec = nb.ShardingSpec(mesh, [nb.DimSpec(["a"], priority=2), nb.DimSpec([])])
    assert spec.get_max_priority() == 2 and spec.get_min_priority() == 0
    add_op = next(v for v in vars(B).values() if getattr(v, "name", None) == "add")
    assert add_op.allows_partial_passthrough and not add_op.multiple_results
    shapes, dtypes, devices = add_op.compute_physical_shape((x, x), {})
    assert shapes == [(2, 3)] and dtypes == [nb.DType.float32]
    c = nb.compile(lambda t: t * 2.0)
    c(x)
    assert c.stats.cache_size == 1 and c.stats.total_compile_time_ms > 0 and c.stats.total_cached_exec_time_ms >= 0
    # the package's function names survive the import of the like-named reference module paths
    import nabla_b200.ops.communication.shard  # noqa: F401
    import nabla_b200.ops.communication.all_reduce  # noqa: F401
    from nabla_b200.ops.communication import all_reduce, shard

    assert callable(shard) and callable(all_reduce) and callable(nb.shard)


def test_keyword_names_of_the_reference_signatures():
    """Calls written with the reference's parameter names work unchanged."""
    a, b = T(torch.tensor([[1.0, 2.0], [3.0, 4.0]])), T(torch.tensor([[2.0, 2.0], [2.0, 2.0]]))
    close(nb.add(x=a, y=b), a.to_numpy() + 2.0)
    close(nb.matmul(x=a, y=b), a.to_numpy() @ b.to_numpy())
    close(nb.pow(x=a, y=b), a.to_numpy() ** 2)
    assert nb.greater(x=a, y=b).to_numpy().tolist() == [[False, False], [True, True]]
    assert nb.logical_not(x=nb.greater(x=a, y=b)).to_numpy().tolist() == [[True, True], [False, False]]
    close(nb.concatenate(tensors=[a, b], axis=0), np.concatenate([a.to_numpy(), b.to_numpy()], 0))
    close(nb.stack(tensors=[a, b], axis=0), np.stack([a.to_numpy(), b.to_numpy()], 0))
    close(nb.pad(a, paddings=[(1, 0), (0, 1)], mode="constant", value=9.0), np.pad(a.to_numpy(), [(1, 0), (0, 1)], constant_values=9.0))
    close(nb.pad(a, pad_width=[(0, 1), (0, 0)]), np.pad(a.to_numpy(), [(0, 1), (0, 0)]))
    with pytest.raises(NotImplementedError):
        nb.pad(a, paddings=[(1, 0), (0, 1)], mode="reflect")
    p, q = nb.split(a, num_splits=2, axis=1)
    close(p, a.to_numpy()[:, :1])
    z = nb.zeros((2, 2), is_traced=True)
    assert z.is_traced and nb.ones((2,), is_traced=False).to_numpy().tolist() == [1.0, 1.0]
    mesh = nb.DeviceMesh("mk", (2,), ("x",))
    xs = nb.shard(a, mesh, ("x", None))
    close(nb.gather_all_axes(sharded_tensor=xs), a.to_numpy())
    close(nb.pmean(sharded_tensor=xs, axis_name="x"), (a.to_numpy()[:1] + a.to_numpy()[1:]) / 2.0)
    close(nb.ppermute(sharded_tensor=xs, permutation=[(0, 1), (1, 0)]), a.to_numpy()[::-1])
    close(nb.all_to_all(sharded_tensor=xs, split_axis=1, concat_axis=0), a.to_numpy())


def test_defaults_of_the_reference_signatures():
    a = T(rand(1, 3, 1, seed=95))
    assert tuple(int(d) for d in nb.squeeze(a).shape) == (3, 1)                 # default axis 0
    assert tuple(int(d) for d in nb.squeeze(a, axis=None).shape) == (3,)
    assert tuple(int(d) for d in a.squeeze().shape) == (3,)                      # the method squeezes everything
    assert nb.cast(a) is a or nb.cast(a).dtype == a.dtype                        # no dtype: unchanged
    mesh = nb.DeviceMesh("md", (2,), ("x",))
    full = rand(4, 2, seed=96)
    xs = nb.shard(T(full), mesh, ("x", None))
    g = nb.gather(xs)                                                            # no indices: collect the shards
    close(g, full)
    assert g.sharding is None or g.sharding.is_fully_replicated()
    # jacrev / jacfwd differentiate every argument unless told otherwise
    f = lambda u, v: u * v * v
    u, v = T(torch.tensor([1.0, 2.0])), T(torch.tensor([3.0, 4.0]))
    for jac in (nb.jacrev, nb.jacfwd):
        ju, jv = jac(f)(u, v)
        close(ju, np.diag(v.to_numpy() ** 2), rtol=1e-5)
        close(jv, np.diag(2 * u.to_numpy() * v.to_numpy()), rtol=1e-5)
        close(jac(f, argnums=1)(u, v), np.diag(2 * u.to_numpy() * v.to_numpy()), rtol=1e-5)
        close(jac(lambda w: w * w)(u), np.diag(2 * u.to_numpy()), rtol=1e-5)     # one argument: a single Jacobian
        assert isinstance(jac(f, argnums=(0,))(u, v), tuple)


def test_cost_model_and_shape_helpers_of_the_op_base_classes():
    """reference: nabla/ops/communication/base.py:51-66,245-279; nabla/ops/base.py:704-706,881-895."""
    import torch

    from nabla_b200.ops.base import AxisOp, CollectiveOperation, ReduceOperation
    from nabla_b200.ops.communication import AllGatherOp, AllReduceOp, ReduceScatterOp
    from nabla_b200.ops.reduction import ReduceSumOp
    from nabla_b200.ops.view.axes import UnsqueezeOp

    m4 = nb.DeviceMesh("c4", (4,), ("d",))
    m2 = nb.DeviceMesh("c2", (2,), ("d",))
    assert AllReduceOp.estimate_cost(10000, m4, ["d"]) == pytest.approx(10 * AllReduceOp.estimate_cost(1000, m4, ["d"]))
    assert AllReduceOp.estimate_cost(1000, m4, ["d"]) > AllReduceOp.estimate_cost(1000, m2, ["d"])
    assert AllReduceOp.estimate_cost(1000, m4, ["d"]) == pytest.approx(2 * AllGatherOp.estimate_cost(1000, m4, ["d"]))
    assert ReduceScatterOp.estimate_cost(1000, m4, ["d"]) == pytest.approx(750.0)
    assert AllReduceOp.estimate_cost(1000, m4, []) == 0.0 and CollectiveOperation.estimate_cost(1000, m4, ["d"]) == 0.0
    fast = nb.DeviceMesh("f4", (4,), ("d",), bandwidth=10.0)
    assert AllGatherOp.estimate_cost(1000, fast, ["d"]) == pytest.approx(75.0)
    spec = nb.ShardingSpec(m4, [nb.DimSpec(["d"]), nb.DimSpec([])])
    assert AllGatherOp().communication_cost([spec], [spec], [(8, 4)], [(8, 4)], m4) == pytest.approx(0.75 * 8 * 4 * 4)
    assert ReduceSumOp().infer_output_shape([(2, 3, 4)], axis=-2) == (2, 4)
    assert ReduceSumOp().infer_output_shape([(2, 3, 4)], axis=0, keepdims=True) == (1, 3, 4)
    assert isinstance(ReduceSumOp(), ReduceOperation) and ReduceSumOp().axis_arg_names == {"axis"}
    assert UnsqueezeOp.axis_offset_for_insert is True and AxisOp.axis_offset_for_insert is False
    t = nb.Tensor.from_graph_value(torch.ones(2, 3))
    assert tuple(int(d) for d in t.shape) == (2, 3)
    with pytest.raises(TypeError):
        nb.Tensor.from_graph_value([1.0])


def test_shard_level_helpers_and_small_utilities():
    """reference: nabla/core/sharding/spmd.py:44-370, nabla/transforms/utils.py:40-127,
    nabla/config.py:83-99, nabla/core/sharding/spec.py:53-79."""
    import nabla_b200.config as cfg
    from nabla_b200.core.common.context import contextvar_context
    from nabla_b200.core.common.pytree import is_tensor_value
    from nabla_b200.core.graph.engine import driver_tensor_type
    from nabla_b200.core.graph.tracing import GraphPrinter
    from nabla_b200.core.sharding import spmd
    from nabla_b200.core.sharding.spec import check_sub_axes_maximality
    from nabla_b200.transforms.utils import (collect_grads, create_jacobian_helpers, realize_tensors, resolve_argnums,
                                             split_aux)

    mesh = nb.DeviceMesh("sh", (2,), ("x",))
    a = np.arange(12, dtype=np.float32).reshape(4, 3)
    want = nb.ShardingSpec(mesh, [nb.DimSpec(["x"]), nb.DimSpec([])])
    (xs,) = spmd.reshard_inputs((nb.Tensor.from_dlpack(a),), [want], mesh)
    assert xs.sharding == want
    parts = spmd.execute_on_shards(lambda t, k: t * k, (xs,), {"k": 2.0}, mesh)
    assert [tuple(p.shape) for p in parts] == [(2, 3), (2, 3)]
    y = spmd.create_sharded_output(parts, want)
    np.testing.assert_allclose(y.to_numpy(), 2 * a)
    assert tuple(spmd.get_shard_args((xs, 3), 1)[0].shape) == (2, 3) and spmd.get_shard_args((xs, 3), 1)[1] == 3

    assert split_aux((1, 2), True, "f") == (1, 2) and split_aux(5, False, "f") == (5, None)
    with pytest.raises(ValueError):
        split_aux(5, True, "f")
    assert resolve_argnums(None, 3) == (0, 1, 2) and resolve_argnums(-1, 3) == (2,) and resolve_argnums([0, 2], 3) == (0, 2)
    with pytest.raises(ValueError):
        resolve_argnums(3, 3)
    t1, t2 = nb.Tensor.from_dlpack(a), nb.Tensor.from_dlpack(a)
    got = collect_grads({t1: t2}, [t1, t2, 4.0])
    assert got[0] is t2 and got[2] is None and float(got[1].to_numpy().sum()) == 0.0
    lazy = t1 + 1.0
    realize_tensors([lazy, 3])
    assert lazy.is_realized
    diff, part = create_jacobian_helpers(lambda u, v, w: (u, v, w), (0, 2), (1, 2, 3))
    assert diff == (1, 3) and part(10, 30) == (10, 2, 30)

    with cfg.eager_max_graph_context(True), cfg.verify_eager_shapes_context(True):
        assert cfg.EAGER_MAX_GRAPH and cfg.VERIFY_EAGER_SHAPES
    assert not cfg.EAGER_MAX_GRAPH
    with contextvar_context(cfg._TRACING, True):
        assert cfg.TRACING
    assert is_tensor_value(torch.ones(1)) and not is_tensor_value(t1)
    assert driver_tensor_type(torch.ones(2, 3))[0] == (2, 3)
    assert GraphPrinter.__name__ == "GraphPrinter"
    assert len(check_sub_axes_maximality(["x:(1)2", "x:(2)2", "y"])) == 1 and not check_sub_axes_maximality(["x", "y"])


def test_json_auto_sharding_solver_picks_data_or_model_parallel_and_keeps_fixed_layouts():
    """reference: nabla/core/sharding/optimizer/auto_sharding.py:19-330 (same JSON in, same JSON out)."""
    import json

    from nabla_b200.core.sharding.optimizer.auto_sharding import AutoSharding, graph_to_json
    from nabla_b200.core.sharding.propagation import OpShardingRuleTemplate, propagate_sharding

    z = lambda *s: nb.Tensor.from_dlpack(np.zeros(s, np.float32))      # noqa: E731
    g = graph_to_json(lambda x, a, b: nb.relu(x @ a) @ b, (z(64, 32), z(32, 128), z(128, 16)))
    names = [n["op_name"] for n in json.loads(g)["nodes"]]
    assert names == ["matmul", "relu", "matmul"]
    solver = AutoSharding((4,), ("d",))
    sol = solver.solve(g)
    assert solver.seeds["0"]["strategy"] == "dp"
    for node in sol["nodes"].values():                     # rows split everywhere, weights whole
        assert node["outputs"]["0"]["dims"] == [["d"], None]
    assert sol["nodes"]["2"]["inputs"]["1"]["dims"] == [None, None]
    sol = solver.solve(graph_to_json(lambda x, w: nb.exp(x @ w), (z(2, 4096), z(4096, 8))))
    assert solver.seeds["0"]["strategy"] == "mp"           # 2 rows cannot be split over 4 devices
    assert sol["nodes"]["0"]["inputs"]["0"]["dims"] == [None, ["d"]] and sol["nodes"]["0"]["inputs"]["1"]["dims"] == [["d"], None]
    fixed = {"tensors": [{"id": 0, "shape": [64, 32], "fixed_sharding": {"dims": [None, "d"], "replicated": []}},
                         {"id": 1, "shape": [32, 8], "fixed_sharding": None}, {"id": 2, "shape": [64, 8], "fixed_sharding": None}],
             "nodes": [{"id": 0, "op_name": "matmul", "inputs": [0, 1], "outputs": [2],
                        "sharding_rule": {"equation": "m k, k n -> m n", "factor_sizes": {"m": 64, "k": 32, "n": 8}},
                        "compute_stats": {"flops": 2.0 * 64 * 32 * 8}}]}
    sol = solver.solve(json.dumps(fixed))
    assert sol["nodes"]["0"]["inputs"]["0"]["dims"] == [None, ["d"]] and sol["nodes"]["0"]["inputs"]["1"]["dims"] == [["d"], None]

    mesh = nb.DeviceMesh("pr", (4,), ("d",))
    mk = lambda r: nb.ShardingSpec(mesh, [nb.DimSpec([], is_open=True) for _ in range(r)])      # noqa: E731
    a, b, c = mk(2), mk(2), mk(2)
    c.dim_specs[1] = nb.DimSpec(["d"], is_open=False)      # a fact on the output flows back to the weight
    rule = OpShardingRuleTemplate.parse("m k, k n -> m n").instantiate([(8, 16), (16, 32)], [(8, 32)])
    assert propagate_sharding(rule, [a, b], [c]) and b.dim_specs[1].axes == ["d"] and not a.dim_specs[0].axes
    assert not propagate_sharding(rule, [a, b], [c])


def test_op_call_stage_helpers_and_op_class_names():
    """reference: nabla/ops/utils.py:410-762 and the op classes its modules export."""
    import nabla_b200.config as cfg
    from nabla_b200.ops import utils as U
    from nabla_b200.ops.binary import MatmulOp
    from nabla_b200.ops.comparison import ComparisonOp, ComparisonUnaryOp, EqualOp, LogicalNotOp, LogicalXorOp
    from nabla_b200.ops.control_flow import ScanOp, WhileLoopOp
    from nabla_b200.ops.convolution import Conv2DOp, Conv2DTransposeOp
    from nabla_b200.ops.creation import ConstantOp, OnesOp, TriOp, TrilOp, ZerosOp
    from nabla_b200.ops.multi_output import ChunkOp, SplitOp
    from nabla_b200.ops.reduction import PhysicalReduceOp, ReduceSumPhysicalOp
    from nabla_b200.ops.unary import ExpOp, IsNanOp, ReluOp, UnaryOperation

    a = nb.Tensor.from_dlpack(np.ones((4, 3), np.float32))
    assert U.collect_metadata((a, 2)) == (0, False, False, False)
    seen = {}
    nb.vmap(lambda r: seen.setdefault("m", U.collect_metadata((r,))) and r)(a)
    assert seen["m"][0] == 1
    k1 = U.compute_structural_hash("add", (a, a), {"axis": 0})
    assert k1 == U.compute_structural_hash("add", (a * 2.0, a), {"axis": 0}) and k1 != U.compute_structural_hash("add", (a, a), {"axis": 1})
    mesh = nb.DeviceMesh("st", (2,), ("x",))
    y = nb.shard(a, mesh, (None, "x")) @ nb.shard(nb.Tensor.from_dlpack(np.ones((3, 2), np.float32)), mesh, ("x", None))
    assert y.sharding.partial_sum_axes == {"x"}
    r = U.apply_auto_reduction(MatmulOp(), y, mesh, {"x"})
    assert not r.sharding.partial_sum_axes
    np.testing.assert_allclose(r.to_numpy(), np.full((4, 2), 3.0))
    assert U.apply_auto_reduction(MatmulOp(), y, mesh, set()) is y
    with cfg.verify_eager_shapes_context(True):
        U.verify_eager_shapes("op", [[torch.ones(2, 3)]], [[(2, 3)]])
        with pytest.raises(RuntimeError):
            U.verify_eager_shapes("op", [[torch.ones(2, 3)]], [[(2, 4)]])
    assert tuple(U.ensure_tensor(3.0).shape) == ()

    assert issubclass(ExpOp, UnaryOperation) and ExpOp is not ReluOp and IsNanOp().name == "is_nan"
    assert issubclass(EqualOp, ComparisonOp) and issubclass(LogicalXorOp, ComparisonOp) and issubclass(LogicalNotOp, ComparisonUnaryOp)
    assert issubclass(TrilOp, TriOp) and issubclass(ChunkOp, SplitOp) and issubclass(ReduceSumPhysicalOp, PhysicalReduceOp)
    assert Conv2DOp().name == "conv2d" and Conv2DTransposeOp().name == "conv2d_transpose" and WhileLoopOp is not None
    np.testing.assert_allclose(ZerosOp()(shape=(2,), dtype=nb.DType.float32, device=nb.CPU()).to_numpy(), [0.0, 0.0])
    np.testing.assert_allclose(OnesOp()(shape=(2,), dtype=nb.DType.float32, device=nb.CPU()).to_numpy(), [1.0, 1.0])
    np.testing.assert_allclose(ConstantOp()([1.0, 2.0]).to_numpy(), [1.0, 2.0])
    carry, ys = ScanOp()(lambda c, v: (c + v, c), nb.Tensor.from_dlpack(np.zeros(3, np.float32)), a)
    np.testing.assert_allclose(carry.to_numpy(), [4.0, 4.0, 4.0])
    from nabla_b200.nn.modules.linear import Linear
    from nabla_b200.nn.modules.transformer import TransformerDecoderLayer

    assert Linear is nb.nn.Linear and TransformerDecoderLayer is nb.nn.TransformerDecoderLayer


def test_shape_and_layout_inference_entry_points_of_ops():
    """reference: per-op `infer_output_shape` / `infer_sharding_spec`, `OpShardingRule.get_factor_tensors`
    (nabla/ops/base.py, nabla/core/sharding/propagation.py:57-67)."""
    from nabla_b200.core.sharding.propagation import OpShardingRuleTemplate
    from nabla_b200.ops.binary import MatmulOp, OuterOp
    from nabla_b200.ops.multi_output import SplitOp
    from nabla_b200.ops.view.axes import SwapAxesOp

    assert OuterOp().infer_output_shape([(3,), (4,)]) == (3, 4)
    assert MatmulOp().infer_output_shape([(2, 3, 4), (4, 5)]) == (2, 3, 5)
    assert SwapAxesOp().infer_output_shape([(2, 3, 4)], axis1=0, axis2=2) == (4, 3, 2)
    assert SplitOp().infer_output_shape([(6, 2)], sizes=(4, 2), axis=0) == [(4, 2), (2, 2)]
    rule = OpShardingRuleTemplate.parse("m k, k n -> m n").instantiate([(2, 3), (3, 4)])
    assert rule.get_factor_tensors("k") == [("input", 0, 1), ("input", 1, 0)]
    assert rule.get_factor_tensors("m") == [("input", 0, 0), ("output", 0, 0)]
    mesh = nb.DeviceMesh("inf", (2,), ("x",))
    x = nb.shard(nb.Tensor.from_dlpack(np.ones((4, 6), np.float32)), mesh, (None, "x"))
    w = nb.shard(nb.Tensor.from_dlpack(np.ones((6, 2), np.float32)), mesh, ("x", None))
    out, ins, pre = MatmulOp().infer_sharding_spec((x, w), mesh, {})
    assert out.partial_sum_axes == {"x"} and len(ins) == 2 and not pre
