"""jax.numpy on torch CPU tensors: the functions the reference's attention path calls."""
import math as _math

import torch

inf = float("inf")
float32, bfloat16, int32, bool_ = torch.float32, torch.bfloat16, torch.int32, torch.bool
ndarray = torch.Tensor


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def asarray(x, dtype=None):
    return torch.as_tensor(x, dtype=dtype)


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


def where(c, a, b):
    a = a if isinstance(a, torch.Tensor) else torch.as_tensor(a, dtype=b.dtype if isinstance(b, torch.Tensor) else None)
    b = b if isinstance(b, torch.Tensor) else torch.as_tensor(b, dtype=a.dtype)
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
