"""CPU restatement of jaxmodules' masked_attention_via_map.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline / reference legs of the benchmark may
import this file; the product package never does.

Two restatements live here:

* ``blockwise_*`` — a faithful port of the reference's algorithm (q-block map, kv-block
  scan, running *normalised average* carry, zero guard, block-window slicing with XLA's
  start clamping, padding quirk, recompute-style backward) written with torch CPU
  tensors so that it can use every host core.  It is what the benchmark times as the
  CPU baseline.
* ``dense_*`` — float64 dense masked softmax attention with analytic gradients, the
  ground truth that both the port above and the CUDA kernels are compared against.

Parity status: PINNED against the reference's own source, executed on a torch-backed stand-in for the jax API
(jax/jaxlib are not installed on these machines): tests/golden/make_reference_vectors.py imports the unmodified
jaxmodules/attention.py and writes O, dQ, dK, dV for fifteen cases to tests/golden/reference_vectors.npz, and
tests/test_reference_vectors.py holds both restatements below to them (float32: 1e-4, measured below 1e-6).  The float
primitives under the stand-in are torch's, not XLA's, so this pins the algorithm to rounding, not XLA to the bit.
It is also pinned relationally, the way the reference's own tests pin it: against
torch.nn.functional.scaled_dot_product_attention on the shapes/masks of tests/test_mapped_attention.py
(tests/test_oracle_attention.py).

Citations are paths inside acutkosky/jaxmodules.
"""
from __future__ import annotations

import math

import numpy as np
import torch


# --------------------------------------------------------------------------------------
# mask helpers
# --------------------------------------------------------------------------------------

def canonical_mask_fn(mask_fn, is_causal: bool):
    """Mask canonicalisation of the public wrapper (jaxmodules/attention.py:404-419)."""
    if mask_fn is not None and _argcount(mask_fn) == 3:
        three = mask_fn
        mask_fn = lambda b, h, q, k: three(h, q, k)
    if is_causal and mask_fn is not None:
        raise ValueError("cannot specify both 'is_causal' and 'mask_fn'!")
    if is_causal:
        mask_fn = lambda b, h, q, k: q >= k
    if mask_fn is None:
        mask_fn = lambda b, h, q, k: True
    return mask_fn


def _argcount(fn):
    code = getattr(fn, "__code__", None)
    if code is None:
        code = fn.__call__.__code__
        return code.co_argcount - 1
    return code.co_argcount


def eval_mask_grid(mask_fn, B, H, q_idx, k_idx):
    """mask[b, h, q, k] for all b < B, h < H and the given index vectors -> bool ndarray.

    The reference evaluates the same grid with fancy_vmap (jaxmodules/attention.py:70-73).
    """
    b = np.arange(B, dtype=np.int64)[:, None, None, None]
    h = np.arange(H, dtype=np.int64)[None, :, None, None]
    q = np.asarray(q_idx, dtype=np.int64)[None, None, :, None]
    k = np.asarray(k_idx, dtype=np.int64)[None, None, None, :]
    shape = (B, H, q.shape[2], k.shape[3])
    try:
        out = mask_fn(b, h, q, k)
        return np.broadcast_to(np.asarray(out), shape).astype(bool)
    except Exception:
        out = np.zeros(shape, dtype=bool)
        for bi in range(B):
            for hi in range(H):
                for i, qq in enumerate(q.ravel()):
                    for j, kk in enumerate(k.ravel()):
                        out[bi, hi, i, j] = bool(mask_fn(bi, hi, int(qq), int(kk)))
        return out


def window_blocks(window_size, block_size):
    """Block counts of the key window (jaxmodules/attention.py:199-204)."""
    if window_size is None:
        return None, None
    left, right = window_size
    return (left + block_size - 1) // block_size, 1 + (right + block_size - 1) // block_size


def window_start(block_idx, left_blocks, right_blocks, num_kv_blocks):
    """First kv block of q-block ``block_idx`` (jaxmodules/attention.py:161-167).

    ``dynamic_slice_in_dim`` clamps the start so that the slice stays inside the array,
    which slides the window inward at the right edge."""
    total = left_blocks + right_blocks
    if total > num_kv_blocks:
        raise ValueError("window covers more blocks than there are key blocks")
    start = max(0, block_idx - left_blocks)
    return min(start, num_kv_blocks - total)


def effective_dense_mask(mask_fn, B, Hq, N, L, block_size=None, window_size=None):
    """The [B, Hq, N, L] boolean mask that masked_attention_via_map effectively applies:
    mask_fn AND the block window (jaxmodules/attention.py:161-167), in unpadded coordinates.

    The padding of jaxmodules/attention.py:426-437 changes the block counts that the window
    clamp sees, so they are reproduced here too."""
    mask = eval_mask_grid(mask_fn, B, Hq, np.arange(N), np.arange(L)).copy()
    if block_size is None:
        block_size = N
    if window_size is not None:
        Np, Lp = padded_lengths(N, L, block_size)
        lb, rb = window_blocks(window_size, block_size)
        nkb = Lp // block_size
        for i in range(Np // block_size):
            s = window_start(i, lb, rb, nkb)
            q0, q1 = i * block_size, min((i + 1) * block_size, N)
            if q0 >= N:
                break
            k0, k1 = s * block_size, (s + lb + rb) * block_size
            mask[:, :, q0:q1, :min(k0, L)] = False
            mask[:, :, q0:q1, min(k1, L):] = False
    return mask


def padded_lengths(N, L, block_size):
    """Lengths after the wrapper's padding (jaxmodules/attention.py:426-434): only when
    N is not a multiple of block_size; K/V then get block_size - (L % block_size) extra rows,
    a whole extra block when L is already a multiple."""
    if block_size is not None and N % block_size != 0:
        return N + block_size - (N % block_size), L + block_size - (L % block_size)
    return N, L


# --------------------------------------------------------------------------------------
# float64 ground truth
# --------------------------------------------------------------------------------------

def dense_attention(Q, K, V, mask, dO=None, kernel=None):
    """Dense masked softmax attention in float64 (NumPy) with analytic gradients.

    Q [B,N,Hq,d], K,V [B,L,Hkv,d], mask [B,Hq,N,L] bool.  Scores are exp(q.k/sqrt(d))
    (default_kernel, jaxmodules/attention.py:39-50); masked scores are multiplied by zero
    (line 81); rows without any allowed key return 0 (lines 99-100) and get zero gradient.
    Query head hq reads kv head hq // (Hq/Hkv) (rearrange at lines 68, 80).

    ``kernel=(a, b)`` replaces the score by exp(a*q.k + b) — threshold_kernel (lines 18-36) is
    (1, -threshold/sqrt(d)); b only shifts the log-sum-exp.

    Returns dict(O [B,N,Hq,d], lse [B,Hq,N]) and, when dO is given, dQ, dK, dV.
    """
    Q = np.asarray(Q, dtype=np.float64)
    K = np.asarray(K, dtype=np.float64)
    V = np.asarray(V, dtype=np.float64)
    B, N, Hq, d = Q.shape
    _, L, Hkv, _ = K.shape
    G = Hq // Hkv
    scale, shift = (1.0 / math.sqrt(d), 0.0) if kernel is None else kernel
    O = np.zeros((B, N, Hq, d))
    lse = np.full((B, Hq, N), -np.inf)
    out = {}
    if dO is not None:
        dO = np.asarray(dO, dtype=np.float64)
        dQ = np.zeros_like(Q)
        dK = np.zeros_like(K)
        dV = np.zeros_like(V)
    for b in range(B):
        for h in range(Hq):
            hk = h // G
            s = (Q[b, :, h, :] @ K[b, :, hk, :].T) * scale           # [N, L]
            m = mask[b, h]
            s_m = np.where(m, s, -np.inf)
            row_max = s_m.max(axis=1, keepdims=True)
            row_max = np.where(np.isfinite(row_max), row_max, 0.0)
            p = np.where(m, np.exp(s - row_max), 0.0)
            denom = p.sum(axis=1, keepdims=True)
            valid = denom > 0
            safe = np.where(valid, denom, 1.0)
            P = p / safe
            O[b, :, h, :] = P @ V[b, :, hk, :]
            with np.errstate(divide="ignore"):
                lse[b, h] = np.where(valid[:, 0], np.log(safe[:, 0]) + row_max[:, 0] + shift, -np.inf)
            if dO is not None:
                g = dO[b, :, h, :]
                dV[b, :, hk, :] += P.T @ g
                dP = g @ V[b, :, hk, :].T
                delta = (g * O[b, :, h, :]).sum(axis=1, keepdims=True)
                dS = P * (dP - delta)
                dQ[b, :, h, :] = (dS @ K[b, :, hk, :]) * scale
                dK[b, :, hk, :] += (dS.T @ Q[b, :, h, :]) * scale
    out["O"] = O
    out["lse"] = lse
    if dO is not None:
        out.update(dQ=dQ, dK=dK, dV=dV)
    return out


def masked_attention_dense(Q, K, V, *, is_causal=False, mask_fn=None, block_size=None, window_size=None, dO=None,
                           kernel=None):
    """Ground truth for the whole public call (jaxmodules/attention.py:347-455) in float64,
    including 3-D inputs, mask canonicalisation, padding and the block window."""
    Q, K, V = (np.asarray(x) for x in (Q, K, V))
    added = Q.ndim == 3
    if added:
        Q, K, V = Q[None], K[None], V[None]
        if dO is not None:
            dO = np.asarray(dO)[None]
    mask_fn = canonical_mask_fn(mask_fn, is_causal)
    B, N, Hq, d = Q.shape
    L = K.shape[1]
    mask = effective_dense_mask(mask_fn, B, Hq, N, L, block_size, window_size)
    out = dense_attention(Q, K, V, mask, dO, kernel)
    if added:
        out = {k: v[0] for k, v in out.items()}
    return out


# --------------------------------------------------------------------------------------
# faithful blockwise port (torch CPU) — the timed CPU baseline
# --------------------------------------------------------------------------------------

def _kq_block(normalizer, running, q_idx, k_idx, q_block, k_block, v_block, mask_fn):
    """One (q-block, kv-block) update — jaxmodules/attention.py:52-105.

    normalizer [B,Lq,Hq] f32, running [B,Lq,Hq,dv] f32, q_block [B,Lq,Hq,d],
    k_block/v_block [B,Lk,Hkv,d].  Scores and their sums stay in the input dtype, the
    carry is float32, exactly where the reference's dtypes fall."""
    B, Lq, Hq, d = q_block.shape
    Lk, Hkv = k_block.shape[1], k_block.shape[2]
    G = Hq // Hkv
    mask = torch.from_numpy(eval_mask_grid(mask_fn, B, Hq, q_idx, k_idx))      # [B,Hq,Lq,Lk]
    mask = mask.permute(0, 2, 1, 3).reshape(B, Lq, Hkv, G, Lk)
    qb = q_block.reshape(B, Lq, Hkv, G, d)
    # default_kernel: exp(q.k / sqrt(d)) with d = k.shape[-1]  (lines 39-50); no max subtraction
    scores = torch.exp(torch.einsum("bqhmd,bkhd->bqhmk", qb, k_block) / math.sqrt(d))
    scores = scores * mask.to(scores.dtype)                                       # line 81
    local = scores.sum(dim=-1, keepdim=True)                                      # line 83
    n = normalizer.reshape(B, Lq, Hkv, G, 1)
    r = running.reshape(B, Lq, Hkv, G, -1)
    unnorm = torch.einsum("bqhmk,bkhd->bqhmd", scores, v_block)                   # line 89
    new_n = n + local                                                             # line 91
    safe = torch.where(new_n > 0, new_n, torch.ones_like(new_n))                  # line 99
    r = torch.where(new_n > 0, r + (unnorm - r * local) / safe, torch.zeros_like(r))  # line 100
    return new_n.reshape(B, Lq, Hq), r.reshape(B, Lq, Hq, -1)


def _attn_block(block_idx, q_idx, q_block, K, V, mask_fn, left_blocks, right_blocks):
    """All kv blocks for one q-block — jaxmodules/attention.py:133-177."""
    B, Lq, Hq, d = q_block.shape
    L = K.shape[1]
    if L % Lq != 0:
        raise ValueError("key length must be a multiple of the query block size")
    nkb = L // Lq                                      # kv block size == q block size (155-158)
    first, count = 0, nkb
    if left_blocks is not None:
        first = window_start(block_idx, left_blocks, right_blocks, nkb)
        count = left_blocks + right_blocks
    normalizer = torch.zeros((B, Lq, Hq), dtype=torch.float32)                 # carry is f32 (173)
    running = torch.zeros((B, Lq, Hq, V.shape[-1]), dtype=torch.float32)
    for j in range(first, first + count):                                        # lax.scan (171)
        k_idx = np.arange(j * Lq, (j + 1) * Lq)
        normalizer, running = _kq_block(
            normalizer, running, q_idx, k_idx, q_block,
            K[:, j * Lq:(j + 1) * Lq], V[:, j * Lq:(j + 1) * Lq], mask_fn)
    return running


def blockwise_forward(Q, K, V, mask_fn, block_size=None, window_size=None):
    """_masked_attention_via_map primal (jaxmodules/attention.py:180-241): sequential map
    over q-blocks.  Inputs are 4-D torch CPU tensors, already padded; returns float32."""
    B, N, Hq, d = Q.shape
    if block_size is None:
        block_size = N
    lb, rb = window_blocks(window_size, block_size)
    assert K.shape[-1] == d and V.shape[1] == K.shape[1] and V.shape[-1] == d
    assert Hq % K.shape[2] == 0 and V.shape[2] == K.shape[2]
    assert N % block_size == 0, "block_size must divide number of queries!"
    outs = []
    for i in range(N // block_size):
        q_idx = np.arange(i * block_size, (i + 1) * block_size)
        outs.append(_attn_block(i, q_idx, Q[:, i * block_size:(i + 1) * block_size], K, V, mask_fn, lb, rb))
    return torch.cat(outs, dim=1)


def blockwise_backward(Q, K, V, g, mask_fn, block_size=None, window_size=None):
    """_masked_attention_via_map_bwd (jaxmodules/attention.py:266-342): scan over q-blocks,
    each step re-runs the forward of that block under autodiff and adds full-size dK, dV
    into a carry held in the input dtype (lines 323-324, 339)."""
    B, N, Hq, d = Q.shape
    if block_size is None:
        block_size = N
    lb, rb = window_blocks(window_size, block_size)
    dK = torch.zeros_like(K)
    dV = torch.zeros_like(V)
    dQ = []
    for i in range(N // block_size):
        q_idx = np.arange(i * block_size, (i + 1) * block_size)
        q = Q[:, i * block_size:(i + 1) * block_size].detach().clone().requires_grad_(True)
        Kc = K.detach().clone().requires_grad_(True)
        Vc = V.detach().clone().requires_grad_(True)
        out = _attn_block(i, q_idx, q, Kc, Vc, mask_fn, lb, rb)
        gq, gk, gv = torch.autograd.grad(out, (q, Kc, Vc), g[:, i * block_size:(i + 1) * block_size].to(out.dtype))
        dK = dK + gk
        dV = dV + gv
        dQ.append(gq)
    return torch.cat(dQ, dim=1), dK, dV


def masked_attention_via_map(Q, K, V, *, is_causal=False, mask_fn=None, block_size=None,
                             window_size=None, dO=None):
    """Faithful port of the public wrapper (jaxmodules/attention.py:347-455) on torch CPU
    tensors / ndarrays.  Returns O (float32, as the reference does for every input dtype),
    or (O, dQ, dK, dV) when a cotangent dO is given."""
    to_t = lambda x: x if isinstance(x, torch.Tensor) else torch.from_numpy(np.asarray(x))
    Q, K, V = to_t(Q), to_t(K), to_t(V)
    for name, x in (("K", K), ("Q", Q), ("V", V)):
        if x.ndim not in (3, 4):
            raise ValueError(f"{name} must have 3 or 4 dimensions")
    assert K.ndim == Q.ndim and V.ndim == Q.ndim
    added = Q.ndim == 3
    if added:
        Q, K, V = Q[None], K[None], V[None]
        if dO is not None:
            dO = to_t(dO)[None]
    elif dO is not None:
        dO = to_t(dO)
    mask_fn = canonical_mask_fn(mask_fn, is_causal)
    assert K.shape[0] == Q.shape[0] == V.shape[0]
    B, N, Hq, d = Q.shape
    L = K.shape[1]
    padded = block_size is not None and N % block_size != 0
    if padded:                                                          # lines 426-437
        pq = block_size - (N % block_size)
        pk = block_size - (L % block_size)
        Q = torch.nn.functional.pad(Q, (0, 0, 0, 0, 0, pq))
        K = torch.nn.functional.pad(K, (0, 0, 0, 0, 0, pk))
        V = torch.nn.functional.pad(V, (0, 0, 0, 0, 0, pk))
        inner = mask_fn
        mask_fn = lambda b, h, q, k: inner(b, h, q, k) & (q < N) & (k < L)
        if dO is not None:
            dO = torch.nn.functional.pad(dO, (0, 0, 0, 0, 0, pq))
    O = blockwise_forward(Q, K, V, mask_fn, block_size, window_size)
    grads = None
    if dO is not None:
        grads = blockwise_backward(Q, K, V, dO, mask_fn, block_size, window_size)
    if padded:
        O = O[:, :N]
        if grads is not None:
            grads = (grads[0][:, :N], grads[1][:, :L], grads[2][:, :L])
    if added:
        O = O[0]
        if grads is not None:
            grads = tuple(x[0] for x in grads)
    if grads is None:
        return O
    return (O,) + tuple(grads)
