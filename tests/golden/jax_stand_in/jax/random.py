"""jax.random for the reference's tests: keys are pairs of integers, draws come from a torch generator seeded by the key.
The streams differ from jax's; the tests only need seeded normal data."""
import hashlib

import torch


def _mix(*ints):
    digest = hashlib.sha256(",".join(str(int(i)) for i in ints).encode()).digest()
    return int.from_bytes(digest[:4], "little"), int.from_bytes(digest[4:8], "little")


def PRNGKey(seed):
    return torch.tensor(_mix(seed, 0), dtype=torch.int64)


key = PRNGKey


def split(k, num=2):
    return torch.stack([torch.tensor(_mix(k[0], k[1], i + 1), dtype=torch.int64) for i in range(num)])


def _generator(k):
    return torch.Generator().manual_seed((int(k[0]) << 31) ^ int(k[1]))


def normal(k, shape=(), dtype=torch.float32):
    return torch.randn(tuple(shape), generator=_generator(k), dtype=torch.float32).to(dtype)


def uniform(k, shape=(), dtype=torch.float32, minval=0.0, maxval=1.0):
    return (torch.rand(tuple(shape), generator=_generator(k), dtype=torch.float32) * (maxval - minval) + minval).to(dtype)


def randint(k, shape, minval, maxval, dtype=torch.int32):
    return torch.randint(int(minval), int(maxval), tuple(shape), generator=_generator(k)).to(dtype)
