"""jax.numpy on torch CPU tensors: the functions the reference's attention path calls."""
import builtins as _py
import math as _math

import torch

inf = float("inf")
float32, bfloat16, int32, bool_ = torch.float32, torch.bfloat16, torch.int32, torch.bool
ndarray = torch.Tensor


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def _stack_nested(x):
    """Nested lists / tuples that hold tensors become one tensor (jnp.array([[a, b], [c, d]]))."""
    if isinstance(x, (list, tuple)) and _py.any(isinstance(e, (torch.Tensor, list, tuple)) for e in x):
        parts = [_stack_nested(e) for e in x]
        if _py.any(isinstance(e, torch.Tensor) for e in parts):
            return torch.stack([e if isinstance(e, torch.Tensor) else torch.as_tensor(e) for e in parts])
    return x


def asarray(x, dtype=None):
    t = torch.as_tensor(_stack_nested(x), dtype=dtype)
    if dtype is None and t.dtype == torch.float64:
        t = t.to(torch.float32)               # jax's default float is float32 (x64 is off)
    if dtype is None and t.dtype == torch.int64 and not isinstance(x, torch.Tensor):
        t = t.to(torch.int32)                 # ... and its default integer int32
    return t


array = asarray


def arange(*a, dtype=None):
    return torch.arange(*a, dtype=dtype or torch.int32)


def zeros(shape, dtype=None):
    return torch.zeros(tuple(shape) if not isinstance(shape, int) else (shape,), dtype=dtype or torch.float32)


def ones(shape, dtype=None):
    return torch.ones(tuple(shape) if not isinstance(shape, int) else (shape,), dtype=dtype or torch.float32)


zeros_like, ones_like, full_like = torch.zeros_like, torch.ones_like, torch.full_like


def dot(a, b):
    return torch.dot(a, b) if a.ndim == 1 and b.ndim == 1 else a @ b


def exp(x):
    return torch.exp(_t(x))


def sqrt(x):
    return torch.sqrt(x) if isinstance(x, torch.Tensor) else _math.sqrt(x)


def sum(x, axis=None, keepdims=False):   # noqa: A001
    return torch.sum(x) if axis is None else torch.sum(x, dim=axis, keepdim=keepdims)


def max(x, axis=None, keepdims=False):   # noqa: A001
    return torch.max(x) if axis is None else torch.amax(x, dim=axis, keepdim=keepdims)


def _scalar_like(x, other):
    """A Python scalar next to an array: weak typing — an int stays in the array's dtype, a float makes integers float32."""
    if isinstance(other, torch.Tensor) and (other.dtype.is_floating_point or not isinstance(x, float)):
        return torch.as_tensor(x, dtype=other.dtype)
    return torch.as_tensor(x, dtype=torch.float32 if isinstance(x, float) else None)


def where(c, a, b):
    a = a if isinstance(a, torch.Tensor) else _scalar_like(a, b)
    b = b if isinstance(b, torch.Tensor) else _scalar_like(b, a)
    return torch.where(c if c.dtype == torch.bool else c != 0, a, b)


def maximum(a, b):
    a, b = _t(a), _t(b)
    return torch.maximum(a.to(torch.result_type(a, b)), b.to(torch.result_type(a, b)))


def minimum(a, b):
    a, b = _t(a), _t(b)
    return torch.minimum(a.to(torch.result_type(a, b)), b.to(torch.result_type(a, b)))


def reshape(x, shape):
    return torch.reshape(x, tuple(shape))


def transpose(x, axes=None):
    return x.permute(*axes) if axes is not None else x.T


def pad(x, pad_width, mode="constant"):
    assert mode == "constant"
    flat = []
    for lo, hi in reversed(list(pad_width)):     # torch pads from the last dimension backwards
        flat += [lo, hi]
    return torch.nn.functional.pad(x, flat)


def abs(x):   # noqa: A001
    return torch.abs(x)


bool = torch.bool   # noqa: A001  (jnp.bool)
int64 = torch.int64


def full(shape, fill_value, dtype=None):
    return torch.full(tuple(shape), fill_value, dtype=dtype)


def eye(n, m=None, k=0, dtype=None):
    return tri(n, m, k, dtype=torch.int32).sub(tri(n, m, k - 1, dtype=torch.int32)).to(dtype or torch.float32)


def tri(n, m=None, k=0, dtype=None):
    m = n if m is None else m
    rows, cols = torch.arange(n)[:, None], torch.arange(m)[None, :]
    return (cols <= rows + k).to(dtype or torch.float32)


def broadcast_to(x, shape):
    return torch.broadcast_to(_t(x), tuple(shape))


def argsort(x, axis=-1, stable=True, descending=False):
    """jnp.argsort is stable by default; the order of equal keys is part of what the block lists hold."""
    return torch.argsort(x, dim=axis, stable=True, descending=descending).to(torch.int32)


def flip(x, axis=None):
    return torch.flip(x, dims=tuple(range(x.ndim)) if axis is None else (axis,) if isinstance(axis, int) else tuple(axis))


def any(x, axis=None):   # noqa: A001
    return torch.any(_t(x)) if axis is None else torch.any(x, dim=axis)


def all(x, axis=None):   # noqa: A001
    return torch.all(_t(x)) if axis is None else torch.all(x, dim=axis)


float64, float16, uint32, int8 = torch.float64, torch.float16, torch.int64, torch.int8


def allclose(a, b, rtol=1e-5, atol=1e-8, equal_nan=False):
    a, b = _t(a), _t(b)
    return torch.allclose(a.to(torch.result_type(a, b)), b.to(torch.result_type(a, b)), rtol=rtol, atol=atol, equal_nan=equal_nan)


def array_equal(a, b):
    a, b = _t(a), _t(b)
    return a.shape == b.shape and (a == b).all().item() is True


def isnan(x):
    return torch.isnan(_t(x))


def isinf(x):
    return torch.isinf(_t(x))


def isfinite(x):
    return torch.isfinite(_t(x))


def mean(x, axis=None, keepdims=False):
    return torch.mean(x) if axis is None else torch.mean(x, dim=axis, keepdim=keepdims)


def log(x):
    return torch.log(_t(x))


def stack(xs, axis=0):
    return torch.stack(list(xs), dim=axis)


def concatenate(xs, axis=0):
    return torch.cat(list(xs), dim=axis)


def einsum(pattern, *xs):
    return torch.einsum(pattern, *xs)


class linalg:
    @staticmethod
    def norm(x, ord=None, axis=None):
        return torch.linalg.norm(x) if axis is None and ord is None else torch.linalg.norm(x, ord=ord, dim=axis)


def repeat(x, repeats, axis=None):
    return torch.repeat_interleave(x, repeats) if axis is None else torch.repeat_interleave(x, repeats, dim=axis)


def tile(x, reps):
    return torch.tile(x, (reps,) if isinstance(reps, int) else tuple(reps))


def swapaxes(x, a, b):
    return torch.swapaxes(x, a, b)


def expand_dims(x, axis):
    return torch.unsqueeze(x, axis)


def squeeze(x, axis=None):
    return torch.squeeze(x) if axis is None else torch.squeeze(x, axis)


def tril(x, k=0):
    return torch.tril(x, k)


def triu(x, k=0):
    return torch.triu(x, k)
