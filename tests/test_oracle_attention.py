"""Pins the attention oracle the way the reference's own tests pin masked_attention_via_map:
against torch.nn.functional.scaled_dot_product_attention on CPU, with the shapes, masks and
closeness rule of the reference's tests/test_mapped_attention.py."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import attention_oracle as ao


def close(a, b, rtol=1e-3, atol=1e-4):
    """Closeness rule of tests/test_mapped_attention.py:275-300 (norm based)."""
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    diff = np.linalg.norm(a - b)
    return diff < atol or diff / min(np.linalg.norm(a), np.linalg.norm(b)) < rtol


def sdpa(Q, K, V, mask):
    """Q [B,N,Hq,d], K,V [B,L,Hkv,d], mask [B,Hq,N,L] bool -> [B,N,Hq,d] (GQA by repeating kv heads)."""
    G = Q.shape[2] // K.shape[2]
    q = Q.permute(0, 2, 1, 3)
    k = K.permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    v = V.permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    out = F.scaled_dot_product_attention(q, k, v, attn_mask=torch.as_tensor(mask))
    return out.permute(0, 2, 1, 3)


def rand(*shape, seed):
    return torch.from_numpy(np.random.default_rng(seed).standard_normal(shape).astype(np.float32))


MASKS_8 = {
    # tests/test_mapped_attention.py:303-430 — N=L=8, H=4, d=16
    "causal": lambda h, q, k: q >= k,
    "sliding": lambda h, q, k: (q - 2 <= k) & (k <= q + 2),
    "alternating": lambda h, q, k: (q + k) % 2 == 0,
    "head_specific": lambda h, q, k: np.where(h % 2 == 0, q >= k, (q + k) % 2 == 0),
}


@pytest.mark.parametrize("name", list(MASKS_8))
@pytest.mark.parametrize("block_size", [None, 4])
def test_small_masks_match_sdpa(name, block_size):
    N = L = 8
    H, d = 4, 16
    Q, K, V = rand(N, H, d, seed=1), rand(L, H, d, seed=2), rand(L, H, d, seed=3)
    fn = MASKS_8[name]
    mask = ao.eval_mask_grid(lambda b, h, q, k: fn(h, q, k), 1, H, np.arange(N), np.arange(L))
    ref = sdpa(Q[None], K[None], V[None], mask)[0]
    port = ao.masked_attention_via_map(Q, K, V, mask_fn=fn, block_size=block_size)
    truth = ao.masked_attention_dense(Q, K, V, mask_fn=fn, block_size=block_size)["O"]
    assert close(port.numpy(), ref.numpy()) and close(truth, ref.numpy())


def test_block_size_invariance():
    # tests/test_mapped_attention.py:433-452
    N = L = 16
    Q, K, V = rand(N, 4, 16, seed=4), rand(L, 4, 16, seed=5), rand(L, 4, 16, seed=6)
    outs = [ao.masked_attention_via_map(Q, K, V, is_causal=True, block_size=bs).numpy() for bs in (4, 8, 16)]
    assert close(outs[0], outs[1]) and close(outs[1], outs[2])


def test_gqa_and_grads_match_sdpa():
    # tests/test_mapped_attention.py:564-605 — N=32, L=64, Hq=8, Hkv=4, d=64, causal, gradients
    N, L, Hq, Hkv, d = 32, 64, 8, 4, 64
    Q, K, V, g = rand(N, Hq, d, seed=7), rand(L, Hkv, d, seed=8), rand(L, Hkv, d, seed=9), rand(N, Hq, d, seed=10)
    mask = ao.eval_mask_grid(lambda b, h, q, k: q >= k, 1, Hq, np.arange(N), np.arange(L))
    Qt, Kt, Vt = (x.clone().requires_grad_(True) for x in (Q, K, V))
    out = sdpa(Qt[None], Kt[None], Vt[None], mask)[0]
    out.backward(g)
    O, dQ, dK, dV = ao.masked_attention_via_map(Q, K, V, is_causal=True, dO=g)
    truth = ao.masked_attention_dense(Q, K, V, is_causal=True, dO=g)
    for got, tr, ref in ((O, truth["O"], out), (dQ, truth["dQ"], Qt.grad), (dK, truth["dK"], Kt.grad), (dV, truth["dV"], Vt.grad)):
        assert close(got.numpy(), ref.detach().numpy()) and close(tr, ref.detach().numpy())


def test_padding_and_batch_dependent_mask():
    # tests/test_mapped_attention.py:1076-1112 (N=10, L=13, block 4) and :1249-1307 (batch-dependent mask)
    B, N, L, H, d = 2, 10, 13, 4, 16
    Q, K, V, g = rand(B, N, H, d, seed=11), rand(B, L, H, d, seed=12), rand(B, L, H, d, seed=13), rand(B, N, H, d, seed=14)
    fn = lambda b, h, q, k: (q + b >= k)
    mask = ao.eval_mask_grid(fn, B, H, np.arange(N), np.arange(L))
    Qt, Kt, Vt = (x.clone().requires_grad_(True) for x in (Q, K, V))
    out = sdpa(Qt, Kt, Vt, mask)
    out.backward(g)
    O, dQ, dK, dV = ao.masked_attention_via_map(Q, K, V, mask_fn=fn, block_size=4, dO=g)
    assert O.shape == (B, N, H, d) and dK.shape == (B, L, H, d)
    for got, ref in ((O, out), (dQ, Qt.grad), (dK, Kt.grad), (dV, Vt.grad)):
        assert close(got.numpy(), ref.detach().numpy())


def test_window_semantics():
    # tests/test_mapped_attention.py:1552-1648: block counts left=ceil(l/bs), right=1+ceil(r/bs), clamped start
    assert ao.window_blocks((1, 1), 16) == (1, 2)
    assert ao.window_blocks((16, 1), 16) == (1, 2)
    assert ao.window_blocks((17, 1), 16) == (2, 2)
    assert [ao.window_start(i, 1, 2, 4) for i in range(4)] == [0, 0, 1, 1]
    N = L = 64
    Q, K, V = rand(N, 4, 16, seed=15), rand(L, 4, 16, seed=16), rand(L, 4, 16, seed=17)
    no_win = ao.masked_attention_via_map(Q, K, V, block_size=16).numpy()
    w11 = ao.masked_attention_via_map(Q, K, V, block_size=16, window_size=(1, 1)).numpy()
    w161 = ao.masked_attention_via_map(Q, K, V, block_size=16, window_size=(16, 1)).numpy()
    w171 = ao.masked_attention_via_map(Q, K, V, block_size=16, window_size=(17, 1)).numpy()
    assert np.abs(no_win - w11).max() > 1e-3
    assert np.abs(w161 - w11).max() < 1e-3
    assert np.abs(w161 - w171).max() > 1e-3
    # the window applied on top of an exact sliding mask changes nothing (:1552-1590)
    N = L = 32
    Q, K, V = rand(N, 4, 16, seed=18), rand(L, 4, 16, seed=19), rand(L, 4, 16, seed=20)
    fn = lambda h, q, k: (q - 3 <= k) & (k <= q + 2)
    a = ao.masked_attention_via_map(Q, K, V, mask_fn=fn, block_size=8).numpy()
    b = ao.masked_attention_via_map(Q, K, V, mask_fn=fn, block_size=8, window_size=(3, 2)).numpy()
    assert close(a, b, rtol=1e-4)
    # and the dense truth applies the same window
    t = ao.masked_attention_dense(Q, K, V, block_size=8, window_size=(3, 2))["O"]
    p = ao.masked_attention_via_map(Q, K, V, block_size=8, window_size=(3, 2)).numpy()
    assert close(p, t)
    with pytest.raises(ValueError):
        ao.masked_attention_via_map(Q, K, V, block_size=8, window_size=(30, 30))


def test_zero_inputs_and_empty_rows():
    # tests/test_mapped_attention.py:1032-1039: all-zero inputs give zeros; rows without keys give 0, not NaN
    z = torch.zeros(8, 2, 16)
    assert torch.count_nonzero(ao.masked_attention_via_map(z, z, z, is_causal=True)) == 0
    Q, K, V, g = rand(8, 2, 16, seed=21), rand(8, 2, 16, seed=22), rand(8, 2, 16, seed=23), rand(8, 2, 16, seed=24)
    fn = lambda h, q, k: (k < q)   # row 0 has no key
    O, dQ, dK, dV = ao.masked_attention_via_map(Q, K, V, mask_fn=fn, dO=g)
    assert torch.isfinite(O).all() and torch.count_nonzero(O[0]) == 0 and torch.count_nonzero(dQ[0]) == 0
    t = ao.masked_attention_dense(Q, K, V, mask_fn=fn, dO=g)
    assert np.isneginf(t["lse"][:, 0]).all()
    for got, tr in ((O, t["O"]), (dQ, t["dQ"]), (dK, t["dK"]), (dV, t["dV"])):
        assert close(got.numpy(), tr)


def test_errors():
    # tests/test_mapped_attention.py:1051-1073
    Q, K, V = rand(8, 2, 16, seed=1), rand(8, 2, 16, seed=2), rand(8, 2, 16, seed=3)
    with pytest.raises(ValueError):
        ao.masked_attention_via_map(Q, K, V, is_causal=True, mask_fn=lambda h, q, k: True)
    with pytest.raises(AssertionError):
        ao.masked_attention_via_map(Q, rand(8, 2, 32, seed=4), V)


def test_bf16_inputs_return_float32():
    # the carry is float32 (jaxmodules/attention.py:173), so O is float32 for bf16 inputs
    Q, K, V = (rand(16, 2, 16, seed=s).to(torch.bfloat16) for s in (1, 2, 3))
    O = ao.masked_attention_via_map(Q, K, V, is_causal=True, block_size=8)
    assert O.dtype == torch.float32
    t = ao.masked_attention_dense(Q.float(), K.float(), V.float(), is_causal=True)["O"]
    assert np.abs(O.numpy() - t).max() < 2e-2
