"""Per-context state: the graph proxy, the config flags, the module call depth and the default
device / dtype live in ContextVars, so threads and asyncio tasks that copy their context do not see
each other's settings (the reference's tests/unit/test_contextvar_safety.py, 15 cases)."""
import asyncio
import contextvars
import threading
from contextvars import ContextVar

import numpy as np
import pytest

import nabla_b200 as nb
from nabla_b200 import config as nb_config
from nabla_b200.core.graph import engine
from nabla_b200.core.graph.engine import GRAPH, ComputeGraph
from nabla_b200.nn.modules import base as module_base


async def _gather_isolated(*coros):
    """Run coroutines as tasks, each in its own copy of the current context with its own graph."""
    loop = asyncio.get_running_loop()
    tasks = []
    for coro in coros:
        ctx = contextvars.copy_context()
        ctx.run(engine._GRAPH_VAR.set, ComputeGraph())
        tasks.append(loop.create_task(coro, context=ctx))
    return await asyncio.gather(*tasks)


# ---------------------------------------------------------------- graph proxy
def test_graph_is_a_proxy_over_a_contextvar():
    assert isinstance(GRAPH, engine._GraphProxy)
    assert isinstance(engine._GRAPH_VAR, ContextVar)


def test_graph_proxy_delegates_to_the_current_graph():
    cur = GRAPH._get()
    assert isinstance(cur, ComputeGraph)
    assert GRAPH.epoch == cur.epoch and GRAPH.seed == cur.seed


def test_default_graph_is_shared_until_a_context_installs_its_own():
    assert engine._get_current_graph() is engine._DEFAULT_GRAPH or isinstance(engine._GRAPH_VAR.get(), ComputeGraph)
    g = ComputeGraph()
    tok = GRAPH.use(g)
    try:
        assert GRAPH._get() is g
        GRAPH.set_seed(123)
        assert g.seed == 123
    finally:
        engine._GRAPH_VAR.reset(tok)
    assert GRAPH._get() is not g


def test_setting_attributes_through_the_proxy_hits_the_current_graph():
    g = ComputeGraph()
    tok = GRAPH.use(g)
    try:
        GRAPH.rng_counter = 41
        assert g.rng_counter == 41 and GRAPH.next_rng() == (g.seed, 41)
    finally:
        engine._GRAPH_VAR.reset(tok)


# ---------------------------------------------------------------- config flags
def test_config_reads_via_module_getattr():
    assert nb_config.EAGER_MAX_GRAPH == nb_config._EAGER.get()
    assert nb_config.VERIFY_EAGER_SHAPES == nb_config._VERIFY.get()
    assert nb_config.TRACING == nb_config._TRACING.get()
    with pytest.raises(AttributeError):
        nb_config.NO_SUCH_FLAG


def test_config_token_set_reset():
    original = nb_config._TRACING.get()
    token = nb_config._TRACING.set(not original)
    assert nb_config.TRACING == (not original)
    nb_config._TRACING.reset(token)
    assert nb_config.TRACING == original


def test_config_context_managers_nest():
    base = nb_config.TRACING
    with nb_config.tracing(True):
        assert nb_config.TRACING is True
        with nb_config.tracing(False):
            assert nb_config.TRACING is False
            with nb_config.eager_max_graph(True), nb_config.verify_eager_shapes(True):
                assert nb_config.EAGER_MAX_GRAPH and nb_config.VERIFY_EAGER_SHAPES
        assert nb_config.TRACING is True
    assert nb_config.TRACING == base


def test_config_change_in_a_thread_stays_in_that_thread():
    seen = {}

    def worker():
        nb_config.set_eager_max_graph(True)
        seen["inside"] = nb_config.EAGER_MAX_GRAPH

    before = nb_config.EAGER_MAX_GRAPH
    t = threading.Thread(target=worker)
    t.start()
    t.join()
    assert seen["inside"] is True and nb_config.EAGER_MAX_GRAPH == before


# ---------------------------------------------------------------- module call depth
def test_module_call_depth_is_a_contextvar():
    assert isinstance(module_base._CALL_DEPTH, ContextVar)
    assert module_base._CALL_DEPTH.get() == 0


def test_module_call_depth_tracks_nested_calls():
    depths = []

    class Inner(nb.nn.Module):
        def forward(self, x):
            depths.append(module_base._CALL_DEPTH.get())
            return x * 2.0

    class Outer(nb.nn.Module):
        def __init__(self):
            super().__init__()
            self.inner = Inner()

        def forward(self, x):
            depths.append(module_base._CALL_DEPTH.get())
            return self.inner(x) + 1.0

    y = Outer()(nb.ones((2,)))
    assert depths == [1, 2] and module_base._CALL_DEPTH.get() == 0
    assert np.allclose(y.to_numpy(), 3.0)


# ---------------------------------------------------------------- ops and gradients through the proxy
def test_tensor_ops_through_the_proxy():
    x = nb.constant(np.array([1.0, 2.0, 3.0], dtype=np.float32))
    assert np.allclose((x * x + 1.0).to_numpy(), [2.0, 5.0, 10.0])


def test_gradient_through_the_proxy():
    g = nb.grad(lambda a: nb.reduce_sum(a * a * a))(nb.constant(np.array([1.0, 2.0], dtype=np.float32)))
    assert np.allclose(g.to_numpy(), [3.0, 12.0])


# ---------------------------------------------------------------- asyncio isolation
def test_async_tasks_get_their_own_graphs():
    async def task(seed):
        GRAPH.set_seed(seed)
        await asyncio.sleep(0.01)
        return GRAPH.seed, id(GRAPH._get())

    async def main():
        return await _gather_isolated(task(1), task(2), task(3))

    res = asyncio.run(main())
    assert [r[0] for r in res] == [1, 2, 3]
    assert len({r[1] for r in res}) == 3


def test_async_config_isolation():
    async def task(flag):
        tok = nb_config._TRACING.set(flag)
        await asyncio.sleep(0.01)
        seen = nb_config.TRACING
        nb_config._TRACING.reset(tok)
        return seen

    async def main():
        return await _gather_isolated(task(True), task(False), task(True))

    assert asyncio.run(main()) == [True, False, True]
    assert nb_config.TRACING is False


def test_async_module_depth_isolation():
    class Sleepy(nb.nn.Module):
        def forward(self, x):
            return module_base._CALL_DEPTH.get()

    async def task(n):
        tok = module_base._CALL_DEPTH.set(n)
        await asyncio.sleep(0.01)
        d = Sleepy()(None)
        module_base._CALL_DEPTH.reset(tok)
        return d

    async def main():
        return await _gather_isolated(task(0), task(5), task(9))

    assert asyncio.run(main()) == [1, 6, 10]


def test_async_concurrent_gradients():
    async def task(k):
        x = nb.constant(np.array([1.0, 2.0], dtype=np.float32))
        await asyncio.sleep(0.005)
        g = nb.grad(lambda a: nb.reduce_sum(a * a) * float(k))(x)
        await asyncio.sleep(0.005)
        return g.to_numpy()

    async def main():
        return await _gather_isolated(*(task(k) for k in (1, 2, 3, 4)))

    for k, g in zip((1, 2, 3, 4), asyncio.run(main())):
        assert np.allclose(g, np.array([2.0, 4.0]) * k)


def test_default_dtype_and_device_are_per_context():
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


def test_a_context_that_resets_the_graph_variable_gets_a_fresh_graph_lazily():
    """Reference behaviour (tests/unit/test_contextvar_safety.py, `_gather_isolated`): a copied
    context that sets the variable to None gets its own graph on first use, with a positive epoch."""
    import contextvars

    def inside():
        g = engine._get_current_graph()
        assert g is engine._get_current_graph()      # created once, then kept
        return g

    ctx = contextvars.copy_context()
    ctx.run(engine._CURRENT_GRAPH.set, None)
    g = ctx.run(inside)
    assert isinstance(g, ComputeGraph) and g is not engine._DEFAULT_GRAPH and g.epoch > 0
    assert isinstance(engine._GRAPH_EPOCH, ContextVar)
