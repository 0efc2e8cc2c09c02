"""A stand-in for the part of the jax API that the reference's attention path uses, on torch CPU tensors.

TEST INFRASTRUCTURE, used by tests/golden/make_attention_reference_vectors.py only: jax is not installed where this
library is developed, so the reference's own source (jaxmodules/attention.py, imported unmodified from its tree) is
executed on this shim to produce golden vectors.  Arrays are torch tensors; ``vmap`` is ``torch.func.vmap``; ``lax.scan``
and ``lax.map`` are Python loops; ``custom_vjp`` is a ``torch.autograd.Function`` that calls the registered forward /
backward rules; ``vjp`` is ``torch.autograd.grad``.  The arithmetic is therefore torch's float32 on the CPU, not XLA's —
what the vectors pin is the reference's ALGORITHM (block walk, window clamp, running average, padding, head mapping,
the structure of its backward rule), not XLA's rounding."""
import inspect
import threading

import torch

from . import numpy  # noqa: F401  (jax.numpy)
from . import lax    # noqa: F401

Array = torch.Tensor
def _astype(self, dtype):
    if self.dtype.is_floating_point and not dtype.is_floating_point and dtype != torch.bool:
        info = torch.iinfo(dtype)             # XLA saturates a float -> integer conversion (-inf becomes the minimum)
        return torch.nan_to_num(self, nan=0.0, posinf=float(info.max), neginf=float(info.min)).clamp(info.min, info.max).to(dtype)
    return self.to(dtype)


torch.Tensor.astype = _astype   # ndarray methods the reference calls on arrays

_plain_repeat = torch.Tensor.repeat


def _repeat(self, *sizes, axis=None):
    """ndarray.repeat(n, axis=k) repeats elements; torch's own repeat (tiling) is kept for calls without ``axis``."""
    if axis is None:
        return _plain_repeat(self, *sizes)
    return torch.repeat_interleave(self, sizes[0], dim=axis)


torch.Tensor.repeat = _repeat


class _At:
    """``x.at[idx].set(v)`` / ``.add(v)``: functional updates, as copies."""

    def __init__(self, x, idx=None):
        self.x, self.idx = x, idx

    def __getitem__(self, idx):
        return _At(self.x, idx)

    def _in_bounds(self):
        """jax drops a scatter update whose integer index is out of range."""
        items = self.idx if isinstance(self.idx, tuple) else (self.idx,)
        for dim, i in enumerate(items):
            if isinstance(i, (int, torch.Tensor)) and not isinstance(i, bool):
                if isinstance(i, torch.Tensor) and (i.ndim != 0 or i.dtype == torch.bool):
                    continue
                if not -self.x.shape[dim] <= int(i) < self.x.shape[dim]:
                    return False
        return True

    def set(self, v):
        y = self.x.clone()
        if self._in_bounds():
            _plain_setitem(y, self.idx, v)
        return y

    def add(self, v):
        y = self.x.clone()
        if self._in_bounds():
            _plain_setitem(y, self.idx, _plain_getitem(y, self.idx) + v)
        return y


torch.Tensor.at = property(lambda self: _At(self))

_plain_getitem = torch.Tensor.__getitem__
_plain_setitem = torch.Tensor.__setitem__


def _clamping_getitem(self, idx):
    """jax clamps an out-of-range integer array index of a gather (and wraps a negative one); torch raises.  The
    reference relies on the clamp where a select under vmap evaluates the branch that is not taken (list entries
    past a row's count)."""
    items = idx if isinstance(idx, tuple) else (idx,)
    is_index = lambda i: isinstance(i, torch.Tensor) and i.dtype not in (torch.bool, torch.uint8) and not i.dtype.is_floating_point
    plain_int = lambda i: isinstance(i, int) and not isinstance(i, bool)
    if all(plain_int(i) or isinstance(i, slice) or is_index(i) for i in items) and len(items) <= self.ndim:
        fixed = []
        for dim, i in enumerate(items):
            n = self.shape[dim]
            if is_index(i):
                i = torch.where(i < 0, i + n, i).clamp(0, n - 1)
            elif plain_int(i) and n > 0:
                i = min(max(i + n if i < 0 else i, 0), n - 1)
            fixed.append(i)
        idx = tuple(fixed)
    return _plain_getitem(self, idx)


torch.Tensor.__getitem__ = _clamping_getitem


def vmap(fun, in_axes=0, out_axes=0):
    """``torch.func.vmap`` with the mapped axis always produced in front and moved afterwards: torch mishandles
    ``out_dims != 0`` for an output that does not depend on the mapped argument (a mask that ignores b and h)."""
    if isinstance(in_axes, list):
        in_axes = tuple(in_axes)        # jax takes a list of per-argument axes, torch wants a tuple

    def as_arrays(out):                 # jax broadcasts a Python scalar result (a mask function returning True)
        if isinstance(out, (tuple, list)):
            return type(out)(as_arrays(o) for o in out)
        return out if isinstance(out, torch.Tensor) else torch.as_tensor(out)

    mapped = torch.func.vmap(lambda *a: as_arrays(fun(*a)), in_dims=in_axes, out_dims=0)

    def place(out, axis):
        if isinstance(out, (tuple, list)):
            axes = axis if isinstance(axis, (tuple, list)) else [axis] * len(out)
            return type(out)(place(o, a) for o, a in zip(out, axes))
        return out if axis == 0 else torch.movedim(out, 0, axis)

    return lambda *args: place(mapped(*args), out_axes)


def checkpoint(fun, **_):
    return fun


def jit(fun, **_):
    return fun


def vjp(fun, *primals):
    """(fun(*primals), vjp_fn) with vjp_fn(cotangent) -> tuple of cotangents of the primals."""
    with torch.enable_grad():
        leaves = tuple(p.detach().requires_grad_(True) for p in primals)
        out = fun(*leaves)

    def vjp_fn(g):
        grads = torch.autograd.grad(out, leaves, g, allow_unused=True)
        return tuple(torch.zeros_like(p) if gr is None else gr for p, gr in zip(leaves, grads))

    return out.detach(), vjp_fn


_inside_rule = threading.local()


class custom_vjp:
    """``jax.custom_vjp(fun, nondiff_argnames=...)`` with ``defvjp(fwd, bwd)``: differentiable through torch autograd
    by calling ``fwd`` (all arguments, original order) and ``bwd(*nondiff_args, residuals, cotangent)``."""

    def __init__(self, fun, nondiff_argnums=(), nondiff_argnames=()):
        self.fun = fun
        self.sig = inspect.signature(fun)
        names = list(self.sig.parameters)
        self.nondiff = [n for n in names if n in set(nondiff_argnames) or names.index(n) in set(nondiff_argnums)]
        self.fwd = self.bwd = None

    def defvjp(self, fwd, bwd):
        self.fwd, self.bwd = fwd, bwd

    def __call__(self, *args, **kwargs):
        bound = self.sig.bind(*args, **kwargs)
        bound.apply_defaults()
        if getattr(_inside_rule, "depth", 0) > 0 or self.fwd is None:
            return self.fun(*bound.args, **bound.kwargs)      # the primal, e.g. when the forward rule calls the function itself
        values = dict(bound.arguments)
        diff_names = [n for n in values if n not in self.nondiff]
        outer = self

        class Rule(torch.autograd.Function):
            @staticmethod
            def forward(ctx, *diff):
                call = dict(values)
                call.update({n: d.detach() for n, d in zip(diff_names, diff)})
                _inside_rule.depth = getattr(_inside_rule, "depth", 0) + 1
                try:
                    with torch.no_grad():
                        out, res = outer.fwd(**call)
                finally:
                    _inside_rule.depth -= 1
                ctx.res = res
                return out

            @staticmethod
            def backward(ctx, g):
                _inside_rule.depth = getattr(_inside_rule, "depth", 0) + 1
                try:
                    grads = outer.bwd(*[values[n] for n in outer.nondiff], ctx.res, g)
                finally:
                    _inside_rule.depth -= 1
                return tuple(grads)

        return Rule.apply(*[values[n] for n in diff_names])


from . import tree_util  # noqa: E402,F401


class errors:
    class ConcretizationTypeError(Exception):
        pass


class nn:
    @staticmethod
    def softmax(x, axis=-1):
        return torch.softmax(x, dim=axis)


from . import random  # noqa: E402,F401


def _tree_leaves(tree):
    if isinstance(tree, (tuple, list)):
        return [leaf for part in tree for leaf in _tree_leaves(part)]
    if isinstance(tree, dict):
        return [leaf for part in tree.values() for leaf in _tree_leaves(part)]
    return [tree]


def _tree_like(tree, leaves):
    if isinstance(tree, (tuple, list)):
        return type(tree)(_tree_like(part, leaves) for part in tree)
    if isinstance(tree, dict):
        return {k: _tree_like(part, leaves) for k, part in tree.items()}
    return next(leaves)


def value_and_grad(fun, argnums=0, has_aux=False):
    """Reverse-mode derivative through torch autograd (the custom_vjp rules above are honoured); a differentiated
    argument may be a tuple / list / dict of arrays."""
    single = isinstance(argnums, int)
    nums = (argnums,) if single else tuple(argnums)

    def wrapped(*args, **kwargs):
        args = list(args)
        with torch.enable_grad():
            for i in nums:
                args[i] = _tree_like(args[i], iter([x.detach().requires_grad_(True) for x in _tree_leaves(args[i])]))
            out = fun(*args, **kwargs)
            value, aux = out if has_aux else (out, None)
            leaves = [x for i in nums for x in _tree_leaves(args[i])]
            flat = torch.autograd.grad(value, leaves, allow_unused=True)
        flat = iter([torch.zeros_like(x) if g is None else g for x, g in zip(leaves, flat)])
        grads = tuple(_tree_like(args[i], flat) for i in nums)
        value = value.detach()
        result = (value, aux) if has_aux else value
        return result, (grads[0] if single else grads)

    return wrapped


def grad(fun, argnums=0, has_aux=False):
    both = value_and_grad(fun, argnums, has_aux)

    def wrapped(*args, **kwargs):
        value, grads = both(*args, **kwargs)
        return (grads, value[1]) if has_aux else grads

    return wrapped
