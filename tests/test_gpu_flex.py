"""flex_attention on the GPU against the flex oracle (the reference's block walk in float64) —
the cases of the reference's tests/test_attention.py:17-425 plus the three BlockMask routes.
Tolerances: float32 inputs 1e-4 max-abs; bfloat16 inputs 2e-2 max-abs and 2e-3 mean-abs,
relative to max(1, |ref|)."""
import math

import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200 import masks as M
from jaxmodules_b200 import _native as nat
from jaxmodules_b200.flex import flex_attention, flex_route
from jaxmodules_b200 import attention as A
from oracle.flex_oracle import flex_attention_oracle

pytestmark = pytest.mark.gpu

B, H, L, E, BLOCK = 2, 4, 8, 16, 4


def qkv(seed=0, hq=H, hkv=H, l=L, e=E, b=B, dtype=torch.float32, s=None):
    g = torch.Generator().manual_seed(seed)
    mk = lambda h, n: torch.randn(b, h, n, e, generator=g).to(dtype).cuda()
    return mk(hq, l), mk(hkv, s or l), mk(hkv, s or l)


def close(got, ref, dtype=torch.float32):
    err = (got.double().cpu() - ref).abs() / ref.abs().clamp(min=1.0)
    if dtype == torch.float32:
        assert err.max() <= 1e-4, err.max()
    else:
        assert err.max() <= 2e-2 and err.mean() <= 2e-3, (err.max(), err.mean())


def causal(b, h, q, k):
    return q >= k


def sliding(b, h, q, k):
    return (q >= k) & (q - k <= 2)


def alternating(b, h, q, k):
    return (q + k) % 2 == 0


def batch_head_sliding(b, h, q, k):
    return (q >= k) & (q - k <= b + h)


def test_basic_gqa_scale():
    q, k, v = qkv()
    out = flex_attention(q, k, v)
    assert out.shape == (B, H, L, E) and out.dtype == torch.float32
    close(out, flex_attention_oracle(q, k, v))
    q, k, v = qkv(1, hq=4, hkv=2)
    close(flex_attention(q, k, v, enable_gqa=True), flex_attention_oracle(q, k, v, enable_gqa=True))
    with pytest.raises(AssertionError):
        flex_attention(q, k, v)
    q, k, v = qkv(2)
    for scale in (1.0 / math.sqrt(E), 0.5, 2.0, 0.0, torch.tensor(0.25)):
        close(flex_attention(q, k, v, scale=scale), flex_attention_oracle(q, k, v, scale=float(scale)))


@pytest.mark.parametrize("mask_fn", [causal, sliding, alternating, batch_head_sliding], ids=lambda f: f.__name__)
def test_block_mask_from_callable(mask_fn):
    q, k, v = qkv(3)
    bm = jm.create_block_mask(mask_fn, B, H, L, L, BLOCK)
    close(flex_attention(q, k, v, block_mask=bm), flex_attention_oracle(q, k, v, block_mask=bm))


def test_broadcasting_and_edge_values():
    q, k, v = qkv(4, e=2)
    ref = flex_attention_oracle(q, k, v, block_mask=jm.create_block_mask(sliding, B, H, L, L, BLOCK))
    for b, h in ((1, H), (B, 1), (1, 1), (B, H)):
        close(flex_attention(q, k, v, block_mask=jm.create_block_mask(sliding, b, h, L, L, BLOCK)), ref)
    z = torch.zeros_like(q)
    assert torch.all(flex_attention(z, z, z) == 0)
    q, k, v = qkv(5)
    big = [t * 1e3 for t in (q, k, v)]
    ref = flex_attention_oracle(*big)
    assert torch.allclose(flex_attention(*big).double().cpu(), ref, rtol=1e-4, atol=1e-2)


def test_error_cases():
    q, k, v = qkv(6)
    with pytest.raises(AssertionError):
        flex_attention(q, k[:, :, : L - 1], v)
    bad = jm.BlockMask.full_mask(B, H, L, L, 4, device="cuda")
    bad.Q_BLOCK_SIZE = 3
    with pytest.raises(AssertionError):
        flex_attention(q, k, v, block_mask=bad)
    with pytest.raises(NotImplementedError):
        flex_attention(q, k, v, return_lse=True)
    with pytest.raises(NotImplementedError):
        flex_attention(q, k, v, score_mod=lambda s, b, h, qi, ki: s * s)


def test_score_mod_affine():
    """The reference's score_mod test (tests/test_attention.py:120-147) and ALiBi with a causal BlockMask:
    forward against the flex oracle (which applies score_mod element by element), gradients against dense
    float64 autograd with the same bias."""
    q, k, v = qkv(11)
    rel = lambda score, b, h, qi, ki: score + 0.1 * (qi - ki)
    close(flex_attention(q, k, v, score_mod=rel), flex_attention_oracle(q, k, v, score_mod=rel))
    for dtype, e, l, block in ((torch.float32, 32, 128, 64), (torch.bfloat16, 128, 384, 128), (torch.bfloat16, 64, 384, 128)):
        b, h = 2, 4
        q, k, v = qkv(12, hq=h, hkv=h, l=l, e=e, b=b, dtype=dtype)
        slopes = [2.0 ** -(i + 3) for i in range(h)]
        alibi = lambda score, b_, h_, qi, ki: score + slopes[h_] * (ki - qi)
        bm = jm.create_block_mask(M.causal_mask(), 1, 1, l, l, block)
        d_out = torch.randn(b, h, l, e, generator=torch.Generator().manual_seed(3)).cuda()
        got = run_with_grads(q, k, v, d_out, block_mask=bm, score_mod=alibi)
        qd, kd, vd = (t.double().cpu().requires_grad_(True) for t in (q, k, v))
        idx = torch.arange(l, dtype=torch.float64)
        bias = torch.tensor(slopes, dtype=torch.float64)[None, :, None, None] * (idx[None, None, None, :] - idx[None, None, :, None])
        s = qd @ kd.transpose(-1, -2) / math.sqrt(e) + bias
        s = s.masked_fill(~torch.tril(torch.ones(l, l, dtype=torch.bool)), -math.inf)
        ref = torch.softmax(s, dim=-1) @ vd
        ref.backward(d_out.double().cpu())
        for x, r in zip(got, (ref.detach(), qd.grad, kd.grad, vd.grad)):
            close(x, r, dtype)


def test_score_mod_sees_the_kv_head_under_gqa():
    """enable_gqa with a head-dependent score_mod: the reference calls score_mod with the KV-head index
    (jaxmodules/attention.py:543-554), so ``slopes`` has one entry per kv head and every query head of a
    group gets its group's slope.  Checked against the flex oracle, which applies score_mod per element."""
    for dtype, e, l in ((torch.float32, 32, 64), (torch.bfloat16, 128, 256)):
        hq, hkv = 4, 2
        q, k, v = qkv(21, hq=hq, hkv=hkv, l=l, e=e, b=2, dtype=dtype)
        slopes = [0.25, 0.03125]                       # len == Hkv: indexing it with a query head would raise
        alibi = lambda score, b_, h_, qi, ki: score + slopes[h_] * (ki - qi)
        bm = jm.create_block_mask(M.causal_mask(), 1, 1, l, l, 64 if l == 64 else 128)
        got = flex_attention(q, k, v, score_mod=alibi, block_mask=bm, enable_gqa=True)
        want = flex_attention_oracle(q, k, v, score_mod=alibi, block_mask=bm, enable_gqa=True)
        close(got, want, dtype)


def dense_reference_grads(q, k, v, dense, d_out, scale=None):
    """float64 autograd through the dense softmax with the element mask ``dense`` [B,Hq,L,S]."""
    q, k, v = (t.double().cpu().requires_grad_(True) for t in (q, k, v))
    g = q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    s = q @ kk.transpose(-1, -2) * (scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))
    s = s.masked_fill(~dense, -math.inf)
    out = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0) @ vv
    out.backward(d_out.double().cpu())
    return out.detach(), q.grad, k.grad, v.grad


def run_with_grads(q, k, v, d_out, **kw):
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = flex_attention(q, k, v, **kw)
    out.backward(d_out.to(out.dtype))
    return out.detach(), q.grad, k.grad, v.grad


def test_grad_reference_shapes():
    """tests/test_attention.py:359-425 of the reference: grads through a causal BlockMask."""
    q, k, v = qkv(7)
    bm = jm.create_block_mask(causal, B, H, L, L, BLOCK)
    d_out = torch.randn(B, H, L, E, generator=torch.Generator().manual_seed(1)).cuda()
    dense = torch.tril(torch.ones(L, L, dtype=torch.bool)).expand(B, H, L, L)
    for got, ref in zip(run_with_grads(q, k, v, d_out, block_mask=bm), dense_reference_grads(q, k, v, dense, d_out)):
        assert got.shape == ref.shape
        close(got, ref)


def routes_for(q, k, v, bm, grads=True):
    Q, K, V = (t.transpose(1, 2) for t in (q, k, v))
    tiles = [A.plan(Q, K, V)[1:]] + ([A.plan(Q, K, V, backward=True)[1:]] if grads else [])
    return flex_route(bm, q.shape[0], q.shape[1], tiles, q.device)


@pytest.mark.parametrize("dtype,e,block", [(torch.bfloat16, 128, 128), (torch.float32, 32, 64)], ids=["tcgen05", "simt"])
def test_route_lists(dtype, e, block):
    """Block size == kernel tile: the BlockMask's own lists drive the kernels, [B,H,L,E] strides
    are read in place.  A BlockMask that drops blocks the mask would allow must be honoured."""
    b, hq, hkv, l = 2, 4, 2, 4 * block
    q, k, v = qkv(8, hq=hq, hkv=hkv, l=l, e=e, b=b, dtype=dtype)
    d_out = torch.randn(b, hq, l, e, generator=torch.Generator().manual_seed(2)).cuda()
    bm = jm.create_block_mask(M.causal_mask(), 1, 1, l, l, block)
    assert routes_for(q, k, v, bm) == "lists"
    dense = torch.tril(torch.ones(l, l, dtype=torch.bool)).expand(b, hq, l, l)
    got = run_with_grads(q, k, v, d_out, block_mask=bm, enable_gqa=True)
    for x, ref in zip(got, dense_reference_grads(q, k, v, dense, d_out)):
        close(x, ref, dtype)
    close(got[0], flex_attention_oracle(q, k, v, block_mask=bm, enable_gqa=True), dtype)
    # kv-side lists only, per-head, with the full block (row 3, column 0) removed for head 1
    full = bm.get_full_blocks().expand(1, hq, 4, 4).clone()
    full[0, 1, 3, 0] = False
    sparse = jm.BlockMask.from_blocks(bm.get_partial_blocks().expand(1, hq, 4, 4), full, block, M.causal_mask())
    kv_only = jm.BlockMask.from_kv_blocks(sparse.kv_num_blocks, sparse.kv_indices, sparse.full_kv_num_blocks,
                                          sparse.full_kv_indices, block, M.causal_mask(), seq_lengths=(l, l))
    assert kv_only.q_indices is None and routes_for(q, k, v, kv_only) == "lists"
    dense = dense.clone()
    dense[:, 1, 3 * block:, :block] = False
    got = run_with_grads(q, k, v, d_out, block_mask=kv_only, enable_gqa=True)
    for x, ref in zip(got, dense_reference_grads(q, k, v, dense, d_out)):
        close(x, ref, dtype)
    close(got[0], flex_attention_oracle(q, k, v, block_mask=kv_only, enable_gqa=True), dtype)


def test_route_terms_and_table():
    """Block size != kernel tile: lists that are exactly the mask's blocks recompile from the
    structured terms; lists that differ go through the bit table."""
    b, h, l, e, block = 1, 2, 512, 128, 64
    q, k, v = qkv(9, hq=h, hkv=h, l=l, e=e, b=b, dtype=torch.bfloat16)
    mask = M.sliding_window_mask(100, 0)
    bm = jm.create_block_mask(mask, 1, 1, l, l, block)
    assert routes_for(q, k, v, bm) == "terms"
    close(flex_attention(q, k, v, block_mask=bm), flex_attention_oracle(q, k, v, block_mask=bm), torch.bfloat16)
    full = bm.get_full_blocks().clone()
    part = bm.get_partial_blocks().clone()
    part[0, 0, 5, 4] = False          # drop a partial block the mask allows
    cut = jm.BlockMask.from_blocks(part, full, block, mask)
    assert routes_for(q, k, v, cut) == "table"
    ref = flex_attention_oracle(q, k, v, block_mask=cut)
    got = flex_attention(q, k, v, block_mask=cut)
    close(got, ref, torch.bfloat16)
    assert not torch.allclose(ref, flex_attention_oracle(q, k, v, block_mask=bm))
    # a document mask under a batch-broadcast BlockMask reads segment ids of batch 0 only
    seg = torch.tensor([[0] * 200 + [1] * 312, [0] * 64 + [1] * 448])
    q, k, v = qkv(10, hq=h, hkv=h, l=l, e=e, b=2, dtype=torch.bfloat16)
    doc = M.document_mask(seg, causal=True)
    bm = jm.create_block_mask(doc, 2, 1, l, l, 128)
    assert routes_for(q, k, v, bm) == "lists"
    close(flex_attention(q, k, v, block_mask=bm), flex_attention_oracle(q, k, v, block_mask=bm), torch.bfloat16)
    first = jm.BlockMask.from_blocks(bm.get_partial_blocks()[:1], bm.get_full_blocks()[:1], 128, doc)
    assert first.B == 1 and routes_for(q, k, v, first) == "table"
    close(flex_attention(q, k, v, block_mask=first), flex_attention_oracle(q, k, v, block_mask=first), torch.bfloat16)
