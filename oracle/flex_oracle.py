"""TEST INFRASTRUCTURE ONLY — CPU restatement of ``_flex_attention``
(jaxmodules/attention.py:458-687).  Nothing in the product imports this module.

The walk is the reference's: per (b, kv head h, group member g, query block l) first the FULL
kv blocks listed for the query head, then the PARTIAL ones with ``mask_mod`` applied, carrying
(normalised result, sum of exponentials, running maximum) with the same guards against
``-inf`` (:598-627).  List reads clamp out-of-range indices like JAX gathers do.  Arithmetic is
float64, so the result is the reference's up to its float32 rounding.

Pinned by tests/test_oracle_flex.py against ``torch.nn.attention.flex_attention`` — the same
cross-check the reference's own tests use (tests/test_attention.py:17-118, 223-356) — and
against the dense float64 softmax; and by tests/test_reference_vectors.py against outputs of the reference's own
flex_attention source, run on a stand-in for jax by tests/golden/make_reference_vectors.py.
"""
from __future__ import annotations

import math

import numpy as np
import torch


def _clamped(t: torch.Tensor, *ix):
    return t[tuple(min(max(int(i), 0), n - 1) for i, n in zip(ix, t.shape))]


def _mask_block(mask_mod, b, h, q0, QB, k0, KVB) -> torch.Tensor:
    q = np.arange(q0, q0 + QB, dtype=np.int64)[:, None]
    k = np.arange(k0, k0 + KVB, dtype=np.int64)[None, :]
    try:
        out = np.broadcast_to(np.asarray(mask_mod(b, h, q, k)), (QB, KVB)).astype(bool)
    except Exception:
        out = np.array([[bool(mask_mod(b, h, int(qq), int(kk))) for kk in k[0]] for qq in q[:, 0]])
    return torch.from_numpy(out.copy())


def flex_attention_oracle(query, key, value, block_mask=None, scale=None, enable_gqa=False, score_mod=None):
    """query [B,Hq,L,E], key/value [B,Hkv,S,E] -> [B,Hq,L,Ev] float64.  ``block_mask`` is any
    object with the BlockMask fields (CPU tensors)."""
    query, key, value = query.double().cpu(), key.double().cpu(), value.double().cpu()
    B, Hq, L, E = query.shape
    _, Hkv, S, _ = key.shape
    Ev = value.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(E)
    if not enable_gqa:
        assert Hq == Hkv
    G = Hq // Hkv
    if block_mask is None:
        QB, KVB = L, S
        lists = None
    else:
        QB, KVB = block_mask.Q_BLOCK_SIZE, block_mask.KV_BLOCK_SIZE
        assert L == block_mask.Q_LEN and S == block_mask.KV_LEN and L % QB == 0 and S % KVB == 0
        lists = tuple(t.cpu() for t in (block_mask.full_kv_num_blocks, block_mask.full_kv_indices,
                                        block_mask.kv_num_blocks, block_mask.kv_indices))
    out = torch.zeros((B, Hq, L, Ev), dtype=torch.float64)
    for b in range(B):
        for h in range(Hkv):
            for g in range(G):
                hq = h * G + g
                for l in range(L // QB):
                    q = query[b, hq, l * QB:(l + 1) * QB]
                    acc = torch.zeros((QB, Ev), dtype=torch.float64)
                    ssum = torch.zeros((QB, 1), dtype=torch.float64)
                    smax = torch.full((QB, 1), -math.inf, dtype=torch.float64)
                    if lists is None:
                        visits = [(0, False)]
                        bb = hh_list = hh_mask = 0
                    else:
                        f_num, f_idx, p_num, p_idx = lists
                        bb = 0 if block_mask.B == 1 else b
                        hh_list = 0 if block_mask.H == 1 else hq     # lists: query head (:630-643)
                        hh_mask = 0 if block_mask.H == 1 else h      # mask_mod: kv head (:582-592)
                        nf = min(int(_clamped(f_num, bb, hh_list, l)), f_idx.shape[-1])
                        npart = min(int(_clamped(p_num, bb, hh_list, l)), p_idx.shape[-1])
                        visits = [(int(_clamped(f_idx, bb, hh_list, l, j)), False) for j in range(nf)]
                        visits += [(int(_clamped(p_idx, bb, hh_list, l, j)), True) for j in range(npart)]
                    for s, do_mask in visits:
                        s = min(max(s, 0), S // KVB - 1)
                        score = q @ key[b, h, s * KVB:(s + 1) * KVB].T * scale
                        if score_mod is not None:
                            for i in range(QB):
                                for j in range(KVB):
                                    score[i, j] = float(score_mod(score[i, j], b, h, l * QB + i, s * KVB + j))
                        if do_mask:
                            mask = _mask_block(block_mask.mask_mod, bb, hh_mask, l * QB, QB, s * KVB, KVB)
                        else:
                            mask = torch.ones_like(score, dtype=torch.bool)
                        masked = torch.where(mask, score, torch.full_like(score, -math.inf))
                        nmax = torch.maximum(smax, masked.max(dim=-1, keepdim=True).values)
                        p = torch.where(mask, torch.exp(score - nmax), torch.zeros_like(score))
                        p = torch.nan_to_num(p, nan=0.0)
                        delta = smax - torch.where(nmax == -math.inf, torch.zeros_like(nmax), nmax)
                        nsum = ssum * torch.exp(delta) + p.sum(dim=-1, keepdim=True)
                        carry = torch.where(nsum == 0, torch.zeros_like(nsum), torch.exp(delta) * (ssum / nsum))
                        vmul = torch.where(nsum == 0, torch.zeros_like(nsum), 1.0 / nsum)
                        carry = torch.nan_to_num(carry, nan=0.0)
                        acc = acc * carry + (p @ value[b, h, s * KVB:(s + 1) * KVB]) * vmul
                        ssum, smax = nsum, nmax
                    out[b, hq, l * QB:(l + 1) * QB] = acc
    return out
