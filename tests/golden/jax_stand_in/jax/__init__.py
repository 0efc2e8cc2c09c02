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
torch.Tensor.astype = lambda self, dtype: self.to(dtype)   # ndarray methods the reference calls on arrays


class _At:
    """``x.at[idx].set(v)`` / ``.add(v)``: functional updates, as copies."""

    def __init__(self, x, idx=None):
        self.x, self.idx = x, idx

    def __getitem__(self, idx):
        return _At(self.x, idx)

    def set(self, v):
        y = self.x.clone()
        y[self.idx] = v
        return y

    def add(self, v):
        y = self.x.clone()
        y[self.idx] += v
        return y


torch.Tensor.at = property(lambda self: _At(self))

_plain_getitem = torch.Tensor.__getitem__


def _clamping_getitem(self, idx):
    """jax clamps an out-of-range integer array index of a gather (and wraps a negative one); torch raises.  The
    reference relies on the clamp where a select under vmap evaluates the branch that is not taken (list entries
    past a row's count)."""
    items = idx if isinstance(idx, tuple) else (idx,)
    is_index = lambda i: isinstance(i, torch.Tensor) and i.dtype not in (torch.bool, torch.uint8) and not i.dtype.is_floating_point
    if any(is_index(i) for i in items) and all(isinstance(i, (int, slice)) or is_index(i) for i in items):
        fixed = []
        for dim, i in enumerate(items):
            if is_index(i):
                n = self.shape[dim]
                i = torch.where(i < 0, i + n, i).clamp(0, n - 1)
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
