"""Random chains of ops for differential tests: the same chain is run on plain inputs and on sharded
(or vmapped) ones, and values and gradients must agree. `step` applies one randomly chosen op that is
valid for the current shape; the choice depends only on the random generator, so a chain can be
replayed by re-seeding it."""
import random

import numpy as np

import nabla_b200 as nb

def rand_spec(rng, shape, mesh):
    axes = list(mesh.axis_names)
    rng.shuffle(axes)
    spec = [None] * len(shape)
    for ax in axes:
        if rng.random() < 0.5:
            d = rng.randrange(len(shape)) if shape else None
            if d is not None and spec[d] is None:
                spec[d] = ax
    return tuple(spec)

UNARY = [nb.exp, nb.tanh, nb.relu, nb.sigmoid, lambda t: t * 0.5 + 1.0, lambda t: -t, nb.abs, lambda t: t * t]

def step(rng, t, others):
    k = rng.choice(["unary", "binary", "reduce", "matmul", "transpose", "reshape", "slice", "concat", "softmax", "mean", "max", "bcast", "where", "cumsum"])
    shp = tuple(int(d) for d in t.shape)
    if rng.random() < 0.6:
        k = "second vocabulary"
    if k == "unary":
        return rng.choice(UNARY)(t), k
    if k == "binary":
        o = rng.choice(others)
        if tuple(int(d) for d in o.shape) == shp:
            return rng.choice([lambda a, b: a + b, lambda a, b: a * b, lambda a, b: a - b])(t, o), k
        return t + 1.0, k
    if k == "reduce" and len(shp) >= 1:
        ax = rng.randrange(len(shp))
        return nb.reduce_sum(t, axis=ax, keepdims=rng.random() < 0.5), k
    if k == "mean" and len(shp) >= 1:
        ax = rng.randrange(len(shp))
        return nb.mean(t, axis=ax, keepdims=rng.random() < 0.5), k
    if k == "max" and len(shp) >= 1:
        ax = rng.randrange(len(shp))
        return nb.reduce_max(t, axis=ax, keepdims=rng.random() < 0.5), k
    if k == "matmul" and len(shp) >= 2:
        return t @ nb.swap_axes(t, -1, -2), k
    if k == "transpose" and len(shp) >= 2:
        a, b = rng.sample(range(len(shp)), 2)
        return nb.swap_axes(t, a, b), k
    if k == "reshape" and len(shp) >= 2:
        return nb.reshape(t, (shp[0] * shp[1],) + shp[2:]), k
    if k == "slice" and len(shp) >= 1 and shp[0] >= 2:
        return t[1:], k
    if k == "concat" and len(shp) >= 1:
        ax = rng.randrange(len(shp))
        return nb.concatenate([t, t * 2.0], axis=ax), k
    if k == "softmax" and len(shp) >= 1:
        return nb.softmax(t, axis=rng.randrange(len(shp))), k
    if k == "bcast" and len(shp) >= 1:
        return nb.broadcast_to(nb.unsqueeze(t, axis=0), (2,) + shp), k
    if k == "where":
        return nb.where(nb.greater(t, 0.0), t, t * 0.1), k
    if k == "cumsum" and len(shp) >= 1:
        return nb.cumsum(t, axis=rng.randrange(len(shp))), k
    k2 = rng.choice(["split", "chunk", "layernorm", "pad", "flip", "permute", "unsq", "stack", "moveaxis", "mm_other",
                     "min", "rowbcast", "reshape_split", "midslice", "intindex", "gather", "argmaxmask", "logsoftmax", "sqrt", "div"])
    if k2 == "split" and len(shp) >= 1 and shp[0] % 2 == 0:
        a, b = nb.split(t, 2, axis=0)
        return a * 2.0 - b, k2
    if k2 == "chunk" and len(shp) >= 1:
        parts = nb.chunk(t, 3, axis=len(shp) - 1)
        return nb.concatenate(list(reversed(parts)), axis=len(shp) - 1), k2
    if k2 == "layernorm" and len(shp) >= 1:
        return nb.nn.functional.layer_norm(t, None, None, eps=1e-5, axis=-1), k2
    if k2 == "pad" and len(shp) >= 1:
        return nb.pad(t, [(1, 0)] + [(0, 1)] * (len(shp) - 1)), k2
    if k2 == "flip" and len(shp) >= 1:
        return nb.flip(t, axis=rng.randrange(len(shp))), k2
    if k2 == "permute" and len(shp) >= 2:
        perm = list(range(len(shp))); rng.shuffle(perm)
        return nb.permute(t, tuple(perm)), k2
    if k2 == "unsq":
        return nb.unsqueeze(t, axis=rng.randrange(len(shp) + 1)), k2
    if k2 == "stack":
        return nb.stack([t, t + 1.0], axis=rng.randrange(len(shp) + 1)), k2
    if k2 == "moveaxis" and len(shp) >= 2:
        return nb.moveaxis(t, 0, -1), k2
    if k2 == "mm_other" and len(shp) >= 2:
        o = rng.choice(others)
        osh = tuple(int(d) for d in o.shape)
        if len(osh) >= 2 and osh[-2] == shp[-1] and osh[:-2] == shp[:-2]:
            return t @ o, k2
        if len(osh) >= 2 and osh[-1] == shp[-1] and osh[:-2] == shp[:-2]:
            return t @ nb.swap_axes(o, -1, -2), k2
        return t * 0.5, k2
    if k2 == "min" and len(shp) >= 1:
        return nb.reduce_min(t, axis=rng.randrange(len(shp)), keepdims=True), k2
    if k2 == "rowbcast" and len(shp) >= 2 and shp[-1] >= 1:
        return t - nb.reduce_max(t, axis=-1, keepdims=True), k2
    if k2 == "reshape_split" and len(shp) >= 1 and shp[0] % 2 == 0:
        return nb.reshape(t, (2, shp[0] // 2) + shp[1:]), k2
    if k2 == "midslice" and len(shp) >= 1 and shp[-1] >= 3:
        idx = (slice(None),) * (len(shp) - 1) + (slice(1, shp[-1] - 1),)
        return t[idx], k2
    if k2 == "intindex" and len(shp) >= 2:
        return t[rng.randrange(shp[0])], k2
    if k2 == "gather" and len(shp) >= 1:
        idx = nb.constant(np.array([shp[0] - 1, 0, shp[0] // 2], dtype=np.int32))
        return nb.gather(t, idx, axis=0), k2
    if k2 == "argmaxmask" and len(shp) >= 1:
        m = nb.reduce_max(t, axis=-1, keepdims=True)
        return nb.where(nb.equal(t, m), t, t * 0.0), k2
    if k2 == "logsoftmax" and len(shp) >= 1:
        return nb.logsoftmax(t, axis=rng.randrange(len(shp))), k2
    if k2 == "sqrt":
        return nb.sqrt(t * t + 1.0), k2
    if k2 == "div":
        return t / 3.0, k2
    return t * 1.5, "scale"


def make_chain(plan_seed: int, nsteps: int):
    """``chain(a, b)`` applying ``nsteps`` random ops to ``a`` (``b`` is available as a second operand);
    ``chain.ops`` lists what the last call applied."""
    def chain(a, b):
        r = random.Random(plan_seed)
        t, ops = a, []
        for _ in range(nsteps):
            t, k = step(r, t, [a, b])
            ops.append(k)
        chain.ops = ops
        return t

    chain.ops = []
    return chain
