"""``jax.tree`` stand-in for lists, tuples and dicts."""


def map(f, tree, *rest, is_leaf=None):
    if is_leaf is not None and is_leaf(tree):
        return f(tree, *rest)
    if isinstance(tree, dict):
        return {k: map(f, v, *[r[k] for r in rest], is_leaf=is_leaf) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)):
        items = [map(f, v, *[r[i] for r in rest], is_leaf=is_leaf) for i, v in enumerate(tree)]
        if hasattr(tree, "_fields"):
            return type(tree)(*items)
        return type(tree)(items)
    if tree is None:
        return None
    return f(tree, *rest)


def leaves(tree, is_leaf=None):
    out = []
    map(lambda x: out.append(x), tree, is_leaf=is_leaf)
    return out


def flatten(tree, is_leaf=None):
    lv = leaves(tree, is_leaf)
    return lv, tree


def unflatten(treedef, leaves_):
    it = iter(leaves_)
    return map(lambda _: next(it), treedef)
