"""jax.lax control flow as Python loops over torch tensors (pytrees: tuples / lists of tensors)."""
import torch


def _map_tree(f, *trees):
    t0 = trees[0]
    if isinstance(t0, (tuple, list)):
        return type(t0)(_map_tree(f, *parts) for parts in zip(*trees))
    return f(*trees)


def _index(tree, i):
    return _map_tree(lambda x: x[i], tree)


def _length(tree):
    while isinstance(tree, (tuple, list)):
        tree = tree[0]
    return tree.shape[0]


def _stack(trees):
    return _map_tree(lambda *xs: torch.stack(xs), *trees)


def scan(f, init, xs, length=None):
    carry, ys = init, []
    for i in range(_length(xs) if xs is not None else length):
        carry, y = f(carry, _index(xs, i) if xs is not None else None)
        ys.append(y)
    return carry, (_stack(ys) if ys and ys[0] is not None else None)


def map(f, xs):   # noqa: A001
    return _stack([f(_index(xs, i)) for i in range(_length(xs))])


def dynamic_slice_in_dim(operand, start_index, slice_size, axis=0):
    """XLA clamps the start so that the slice stays inside the operand."""
    start = int(start_index)
    start = min(max(start, 0), operand.shape[axis] - slice_size)
    return operand.narrow(axis, start, slice_size)


def fori_loop(lower, upper, body_fun, init_val):
    val = init_val
    for i in range(int(lower), int(upper)):
        val = body_fun(i, val)
    return val


def cond(pred, true_fun, false_fun, *operands):
    """With a predicate that is mapped by an enclosing vmap both branches run and are selected, as jax does."""
    try:
        taken = bool(pred)
    except RuntimeError:
        return _map_tree(lambda t, f: torch.where(pred, t, f), true_fun(*operands), false_fun(*operands))
    return true_fun(*operands) if taken else false_fun(*operands)
