"""Pins the flex_attention oracle the way the reference's tests pin flex_attention itself:
against torch's FlexAttention on the CPU (tests/test_attention.py:17-118, 223-356 of the
reference) and against the dense float64 softmax."""
import math
import types
import warnings

import numpy as np
import pytest
import torch

from oracle import block_mask_oracle as bo
from oracle.flex_oracle import flex_attention_oracle

torch_fa = pytest.importorskip("torch.nn.attention.flex_attention")

B, H, L, E, BLOCK = 2, 4, 8, 16, 4


def qkv(seed=0, hq=H, hkv=H, l=L, e=E, b=B):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(b, hq, l, e, generator=g), torch.randn(b, hkv, l, e, generator=g),
            torch.randn(b, hkv, l, e, generator=g))


def oracle_block_mask(mask_fn, b, h, q_len, kv_len, block):
    d = bo.create_block_mask(mask_fn, b, h, q_len, kv_len, block)
    t = {k: (torch.from_numpy(np.asarray(v)) if isinstance(v, np.ndarray) else v) for k, v in d.items()}
    t["mask_mod"] = mask_fn
    return types.SimpleNamespace(**t)


def torch_flex(q, k, v, **kw):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return torch_fa.flex_attention(q, k, v, **kw)


def dense_softmax(q, k, v, mask=None, scale=None):
    q, k, v = q.double(), k.double(), v.double()
    g = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    s = q @ k.transpose(-1, -2) * (scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))
    if mask is not None:
        s = s.masked_fill(~mask, -math.inf)
    return torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0) @ v


# the reference's mask_mods (tests/test_attention.py:77-91), written for ints and index arrays
def causal(b, h, q, k):
    return q >= k


def sliding(b, h, q, k):
    return (q >= k) & (q - k <= 2)


def alternating(b, h, q, k):
    return (q + k) % 2 == 0


def batch_head_sliding(b, h, q, k):
    return (q >= k) & (q - k <= b + h)


MASKS = [causal, sliding, alternating, batch_head_sliding]


def test_basic_and_gqa():
    q, k, v = qkv()
    out = flex_attention_oracle(q, k, v)
    assert out.shape == (B, H, L, E)
    assert torch.allclose(out.float(), torch_flex(q, k, v), atol=1e-5)
    q, k, v = qkv(1, hq=4, hkv=2)
    out = flex_attention_oracle(q, k, v, enable_gqa=True)
    assert torch.allclose(out.float(), torch_flex(q, k, v, enable_gqa=True), atol=1e-5)
    assert torch.allclose(out, dense_softmax(q, k, v), atol=1e-10)


@pytest.mark.parametrize("mask_fn", MASKS, ids=lambda f: f.__name__)
def test_block_masks_against_torch(mask_fn):
    q, k, v = qkv(2)
    bm = oracle_block_mask(mask_fn, B, H, L, L, BLOCK)
    out = flex_attention_oracle(q, k, v, block_mask=bm)
    tbm = torch_fa.create_block_mask(mask_fn, B, H, L, L, device="cpu", BLOCK_SIZE=BLOCK)
    assert torch.allclose(out.float(), torch_flex(q, k, v, block_mask=tbm), atol=1e-5)
    bi, hi = torch.arange(B)[:, None, None, None], torch.arange(H)[None, :, None, None]
    qi, ki = torch.arange(L)[None, None, :, None], torch.arange(L)[None, None, None, :]
    dense = torch.broadcast_to(mask_fn(bi, hi, qi, ki), (B, H, L, L))
    assert torch.allclose(out, dense_softmax(q, k, v, dense), atol=1e-10)


@pytest.mark.parametrize("scale", [None, 1.0 / math.sqrt(E), 0.5, 2.0, 0.0])
def test_scale(scale):
    q, k, v = qkv(3)
    out = flex_attention_oracle(q, k, v, scale=scale)
    assert torch.allclose(out.float(), torch_flex(q, k, v, scale=scale), atol=1e-5)


def test_broadcast_over_batch_and_head():
    q, k, v = qkv(4, e=2)
    outs = [flex_attention_oracle(q, k, v, block_mask=oracle_block_mask(sliding, b, h, L, L, BLOCK))
            for b, h in ((1, H), (B, 1), (1, 1), (B, H))]
    for o in outs[:-1]:
        assert torch.allclose(o, outs[-1], atol=1e-12)


def test_score_mod_and_edge_values():
    q, k, v = qkv(5)
    mod = lambda score, b, h, qi, ki: score + (qi - ki) * 0.1
    out = flex_attention_oracle(q, k, v, score_mod=mod)
    assert torch.allclose(out.float(), torch_flex(q, k, v, score_mod=mod), atol=1e-5)
    z = torch.zeros_like(q)
    assert torch.allclose(flex_attention_oracle(z, z, z), torch.zeros(B, H, L, E, dtype=torch.float64))
    big = [t * 1e3 for t in (q, k, v)]
    assert torch.allclose(flex_attention_oracle(*big).float(), torch_flex(*big), rtol=1e-4, atol=1e-2)


def test_rows_without_keys_return_zero():
    q, k, v = qkv(6)
    none_below_4 = lambda b, h, qi, ki: (qi >= 4) & (ki <= qi)
    out = flex_attention_oracle(q, k, v, block_mask=oracle_block_mask(none_below_4, 1, 1, L, L, BLOCK))
    assert torch.all(out[:, :, :4] == 0) and torch.isfinite(out).all()
