import asyncio
import contextvars

import numpy as np
import pytest
import torch

import nabla_b200 as nb
from nabla_b200 import config
from nabla_b200.core.common import pytree
from common import T, close


def test_tensor_basics_and_repr():
    x = nb.constant(np.array([1.0, 2.0], dtype=np.float32))
    assert repr(x) == "Tensor([1. 2.] : f32[2])"
    y = nb.zeros((2, 3))
    assert repr(y.shape) == "[Dim(2), Dim(3)]"
    assert tuple(int(d) for d in y.shape) == (2, 3)
    assert y.dtype is nb.DType.float32 and repr(y.dtype) == "DType.float32"
    assert repr(y.device) == "Device(type=cpu,id=0)"
    assert not y.is_realized
    y.realize()
    assert y.is_realized and y.numel() == 6


def test_lazy_then_realize_all_batches():
    nb.reset_cache_stats()
    a = nb.ones((4,)) * 2.0
    b = a + 1.0
    c = b * b
    assert not (a.is_realized or b.is_realized or c.is_realized)
    nb.realize_all(a, c)
    assert a.is_realized and c.is_realized
    assert nb.get_cache_stats()["evaluations"] == 1
    close(c, np.full((4,), 9.0))


def test_plan_cache_hits_on_same_structure():
    nb.reset_cache_stats()
    for i in range(3):
        x = nb.constant(np.full((3,), float(i), dtype=np.float32))
        (nb.exp(x) + 1.0).realize()
    s = nb.get_cache_stats()
    assert s["misses"] == 1 and s["hits"] == 2


def test_item_and_scalar_errors():
    assert nb.constant(3.5).item() == 3.5
    with pytest.raises(TypeError):
        nb.ones((2,)).item()


def test_indexing_getitem_setitem_at():
    x = T(np.arange(24, dtype=np.float32).reshape(2, 3, 4))
    close(x[1], np.arange(24).reshape(2, 3, 4)[1])
    close(x[:, 1:3, -1], np.arange(24).reshape(2, 3, 4)[:, 1:3, -1])
    close(x[..., 0], np.arange(24).reshape(2, 3, 4)[..., 0])
    with pytest.raises(NotImplementedError):
        x[::2]
    y = nb.zeros((3, 3))
    y[1] = 5.0
    ref = np.zeros((3, 3), dtype=np.float32)
    ref[1] = 5
    close(y, ref)
    z = nb.zeros((3, 3)).at[0:2, 1].add(2.0)
    ref = np.zeros((3, 3), dtype=np.float32)
    ref[0:2, 1] += 2
    close(z, ref)
    idx = T(np.array([2, 0]))
    close(T(np.arange(6, dtype=np.float32).reshape(3, 2))[idx], np.arange(6).reshape(3, 2)[[2, 0]])


def test_dlpack_numpy_roundtrip():
    a = np.random.rand(3, 4).astype(np.float32)
    t = nb.Tensor.from_dlpack(a)
    np.testing.assert_array_equal(np.asarray(t), a)
    back = torch.from_dlpack(t)
    assert back.shape == (3, 4)


def test_pytree_sorted_dict_and_none():
    tree = {"b": 1, "a": (2, None, [3])}
    leaves, td = pytree.tree_flatten(tree)
    assert leaves == [2, 3, 1]
    assert pytree.tree_unflatten(td, leaves) == tree
    assert hash(td) == hash(pytree.tree_structure({"b": 0, "a": (0, None, [0])}))
    assert pytree.tree_map(lambda x, y: x + y, tree, tree) == {"b": 2, "a": (4, None, [6])}
    with pytest.raises(ValueError):
        pytree.tree_unflatten(td, [1])


def test_pytree_custom_node():
    class Box:
        def __init__(self, a, tag):
            self.a, self.tag = a, tag

    pytree.register_pytree_node(Box, lambda b: ([b.a], b.tag), lambda tag, ch: Box(ch[0], tag))
    out = pytree.tree_map(lambda v: v * 2, [Box(3, "x")])
    assert out[0].a == 6 and out[0].tag == "x"


def test_config_flags_scoped():
    assert config.TRACING is False
    with config.tracing(True):
        assert config.TRACING is True
    assert config.TRACING is False
    with config.eager_max_graph(True):
        x = nb.ones((2,)) + 1.0
        assert x.is_realized
    x = nb.ones((2,)) + 1.0
    assert not x.is_realized


def test_default_dtype_device_context():
    with nb.default_dtype(nb.DType.float64):
        assert nb.zeros((1,)).dtype is nb.DType.float64
    assert nb.zeros((1,)).dtype is nb.DType.float32
    a = nb.ones((2,), dtype=nb.DType.int32)
    with nb.defaults_like(a):
        assert nb.zeros((1,)).dtype is nb.DType.int32


def test_contextvar_isolation_across_tasks():
    async def worker(flag):
        config.set_tracing(flag)
        await asyncio.sleep(0.01)
        return config.TRACING

    async def main():
        t1 = asyncio.create_task(worker(True), context=contextvars.copy_context())
        t2 = asyncio.create_task(worker(False), context=contextvars.copy_context())
        return await asyncio.gather(t1, t2)

    assert asyncio.run(main()) == [True, False]
    assert config.TRACING is False


def test_trace_printing():
    x = T(np.ones((2, 3), dtype=np.float32))
    tr = nb.trace(lambda a: nb.relu(a * 2.0) + 1.0, x)
    s = str(tr)
    assert s.startswith("fn(%a1: f32[2,3])") and "relu(" in s and "return" in s


def test_rng_seed_reproducible_and_fresh():
    nb.seed(7)
    a = nb.uniform((4,)).to_numpy()
    b = nb.uniform((4,)).to_numpy()
    nb.seed(7)
    a2 = nb.uniform((4,)).to_numpy()
    assert np.allclose(a, a2) and not np.allclose(a, b)
    g = nb.gaussian((2000,), mean=1.0, std=2.0).to_numpy()
    assert abs(g.mean() - 1.0) < 0.2 and abs(g.std() - 2.0) < 0.2
