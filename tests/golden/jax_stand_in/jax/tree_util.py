"""Present so that ``jaxtyping`` (which the reference imports for annotations) finds ``jax.tree_util``; the attention
path checks no PyTree annotation at run time, so these are never called with anything but tuples and lists."""


def tree_leaves(tree, is_leaf=None):
    if (is_leaf is None or not is_leaf(tree)) and isinstance(tree, (tuple, list)):
        return [leaf for part in tree for leaf in tree_leaves(part, is_leaf)]
    return [tree]


def tree_map(f, tree, *rest):
    if isinstance(tree, (tuple, list)):
        return type(tree)(tree_map(f, *parts) for parts in zip(tree, *rest))
    return f(tree, *rest)
