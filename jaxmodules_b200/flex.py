"""``flex_attention`` of jaxmodules/attention.py:458-692 on the block-list attention kernels.

The reference walks, per query block, first the FULL kv blocks of the BlockMask (no element
mask) and then its PARTIAL blocks (``mask_mod`` applied), with an online softmax.  The CUDA
kernels do the same walk, so a BlockMask whose block size equals the kernel tile is handed to
them as it is (route "lists").  Other block sizes take one of two routes:

* "terms"  — ``mask_mod`` is a structured mask and the BlockMask's lists are exactly the blocks
  of that mask (checked on the device): the element mask alone defines the result and the
  lists are recompiled at the kernel's tile size;
* "table"  — anything else: the element mask the reference would apply
  (``full_block | partial_block & mask_mod``) is evaluated once on the host into a bit table.

Differences from the reference, all deliberate: ``score_mod`` is limited to the affine family
``a * score + w[h] * k`` plus terms constant along k (ALiBi and relative-position biases); a block
that appears twice in a row's lists is visited once.  Like the reference (:615-622), a row whose listed blocks allow no key returns 0.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import numpy as np
import torch

from . import _native as nat
from . import masks as _masks
from . import attention as _att
from .block_mask import BlockMask, compile_block_lists, get_dense_from_kv_blocks, get_sparse_q_data_from_blocks

__all__ = ["flex_attention", "flex_route"]


def _structured_terms(mask_mod) -> Optional[_masks.MaskTerms]:
    """Device terms of ``mask_mod`` when the kernels can evaluate it without a table."""
    if isinstance(mask_mod, _masks.StructuredMask) and mask_mod.terms.bitmap is None:
        return mask_mod.terms
    return None


def _dense_blocks(bm: BlockMask, device):
    """(full, partial) bool [B, H, NQ, NKV] from the kv-side lists."""
    NQ, NKV = bm.Q_LEN // bm.Q_BLOCK_SIZE, bm.KV_LEN // bm.KV_BLOCK_SIZE
    dev = lambda t: t.to(device)
    full = get_dense_from_kv_blocks(bm.B, bm.H, NQ, NKV, dev(bm.full_kv_num_blocks), dev(bm.full_kv_indices))
    part = get_dense_from_kv_blocks(bm.B, bm.H, NQ, NKV, dev(bm.kv_num_blocks), dev(bm.kv_indices))
    return full, part & ~full


class _ReadyLists:
    """Block lists of a user BlockMask in the layout ``bma_block_lists`` wants: int32, row
    width equal to the number of blocks on the other side, counts and indices clamped into
    range (out-of-range reads clamp under JAX, jaxmodules/attention.py:642-666)."""

    def __init__(self, bm: BlockMask, device):
        self.bm, self.device = bm, device
        self.NQ, self.NKV = bm.Q_LEN // bm.Q_BLOCK_SIZE, bm.KV_LEN // bm.KV_BLOCK_SIZE
        self._kv = self._q = self._consistent = None

    def _fit(self, num, idx, width):
        num = num.to(device=self.device, dtype=torch.int32)
        idx = idx.to(device=self.device, dtype=torch.int32)
        num = num.clamp(0, min(idx.shape[-1], width)).contiguous()
        idx = idx[..., :width].clamp(0, width - 1)
        if idx.shape[-1] < width:
            idx = torch.nn.functional.pad(idx, (0, width - idx.shape[-1]))
        return num, idx.contiguous()

    def _kv_side(self):
        if self._kv is None:
            bm = self.bm
            self._kv = (*self._fit(bm.kv_num_blocks, bm.kv_indices, self.NKV),
                        *self._fit(bm.full_kv_num_blocks, bm.full_kv_indices, self.NKV))
        return self._kv

    def _q_side(self):
        if self._q is None:
            bm = self.bm
            if bm.q_indices is not None and bm.full_q_indices is not None:
                self._q = (*self._fit(bm.q_num_blocks, bm.q_indices, self.NQ),
                           *self._fit(bm.full_q_num_blocks, bm.full_q_indices, self.NQ))
            else:  # kv-side only (from_kv_blocks without generate_q_blocks): transpose on the device
                full, part = _dense_blocks(bm, self.device)
                self._q = (*get_sparse_q_data_from_blocks(part), *get_sparse_q_data_from_blocks(full))
                self._q = tuple(t.contiguous() for t in self._q)
        return self._q

    @property
    def consistent(self) -> bool:
        """True when the q-side and the kv-side arrays name the same blocks (checked once, on the device);
        the backward then may hand dS tiles from the kv-major kernel to the query-major one."""
        if self._consistent is None:
            bm = self.bm
            kv_num, kv_idx, fkv_num, fkv_idx = self._kv_side()
            q_num, q_idx, fq_num, fq_idx = self._q_side()
            kv = (get_dense_from_kv_blocks(bm.B, bm.H, self.NQ, self.NKV, kv_num, kv_idx)
                  | get_dense_from_kv_blocks(bm.B, bm.H, self.NQ, self.NKV, fkv_num, fkv_idx))
            q = (get_dense_from_kv_blocks(bm.B, bm.H, self.NKV, self.NQ, q_num, q_idx)
                 | get_dense_from_kv_blocks(bm.B, bm.H, self.NKV, self.NQ, fq_num, fq_idx))
            self._consistent = bool(torch.equal(kv, q.transpose(-1, -2)))
        return self._consistent

    def visited_counts(self, lists, device):
        """Host array of visited (full + partial) blocks per list head (sizes the backward scratch); the lists of a
        BlockMask do not change, so the counts are fetched from the device once."""
        if getattr(self, "_visited", None) is None:
            kv_num, _, fkv_num, _ = self._kv_side()
            self._visited = (kv_num.sum(dim=-1, dtype=torch.int64) + fkv_num.sum(dim=-1, dtype=torch.int64)).reshape(-1).cpu().numpy()
        return self._visited

    def __call__(self, q_tile: int, kv_tile: int, q_side: bool):
        bm = self.bm
        if q_tile != bm.Q_BLOCK_SIZE or kv_tile != bm.KV_BLOCK_SIZE:
            return None
        kv_num, kv_idx, fkv_num, fkv_idx = self._kv_side()
        t = dict(kv_num_blocks=kv_num, kv_indices=kv_idx, full_kv_num_blocks=fkv_num, full_kv_indices=fkv_idx)
        lists = nat.BlockLists()
        lists.B, lists.H, lists.NQ, lists.NKV = bm.B, bm.H, self.NQ, self.NKV
        lists.q_block, lists.kv_block = q_tile, kv_tile
        lists.kv_num, lists.kv_idx = kv_num.data_ptr(), kv_idx.data_ptr()
        lists.full_kv_num, lists.full_kv_idx = fkv_num.data_ptr(), fkv_idx.data_ptr()
        if q_side:
            q_num, q_idx, fq_num, fq_idx = self._q_side()
            t.update(q_num_blocks=q_num, q_indices=q_idx, full_q_num_blocks=fq_num, full_q_indices=fq_idx)
            lists.q_num, lists.q_idx = q_num.data_ptr(), q_idx.data_ptr()
            lists.full_q_num, lists.full_q_idx = fq_num.data_ptr(), fq_idx.data_ptr()
        return lists, t


def _lists_match_terms(bm: BlockMask, terms: _masks.MaskTerms, B: int, Hq: int, device) -> bool:
    """True when the BlockMask's full / partial blocks are exactly the blocks of ``terms`` at
    the BlockMask's own block size (one mask compile and one comparison on the device)."""
    dmask = _masks.to_device_mask(terms, bm.Q_LEN, bm.KV_LEN, device)
    _, t = compile_block_lists(dmask, B, Hq, bm.Q_LEN, bm.KV_LEN, bm.Q_BLOCK_SIZE, bm.KV_BLOCK_SIZE, device,
                               out_B=bm.B, out_H=bm.H, q_side=False, floor_blocks=True)
    NQ, NKV = bm.Q_LEN // bm.Q_BLOCK_SIZE, bm.KV_LEN // bm.KV_BLOCK_SIZE
    want_full = get_dense_from_kv_blocks(bm.B, bm.H, NQ, NKV, t["full_kv_num_blocks"], t["full_kv_indices"])
    want_part = get_dense_from_kv_blocks(bm.B, bm.H, NQ, NKV, t["kv_num_blocks"], t["kv_indices"])
    full, part = _dense_blocks(bm, device)
    return bool((torch.equal(full, want_full) and torch.equal(part, want_part)))


def _effective_table(bm: BlockMask, G: int, Hq: int) -> torch.Tensor:
    """Bit table [Bm, Hm, Q_LEN, words] of the element mask the reference applies:
    ``full_block | (partial_block & mask_mod(block_b, block_h, q, k))`` where the block lists
    are read with the query head and ``mask_mod`` is called with the kv-head index
    (jaxmodules/attention.py:577-593, 630-666)."""
    full, part = _dense_blocks(bm, "cpu")
    full, part = full.numpy(), part.numpy()
    QB, KVB = bm.Q_BLOCK_SIZE, bm.KV_BLOCK_SIZE
    Hm = 1 if bm.H == 1 else Hq
    mask_mod = bm.mask_mod

    def eff(b, h, q, k):
        hh = h if bm.H > 1 else np.zeros_like(h)
        blk_full = full[b, hh, q // QB, k // KVB]
        blk_part = part[b, hh, q // QB, k // KVB]
        allowed = np.asarray(mask_mod(b, hh // G, q, k)).astype(bool)
        return blk_full | (blk_part & allowed)

    def eff_scalar(b, h, q, k):
        hh = h if bm.H > 1 else 0
        if full[b, hh, q // QB, k // KVB]:
            return True
        return bool(part[b, hh, q // QB, k // KVB]) and bool(mask_mod(b, hh // G, q, k))

    try:
        return _masks.bitmap_from_callable(_Strict(eff), bm.B, Hm, bm.Q_LEN, bm.KV_LEN, batch_dependent=bm.B > 1)
    except _NotVectorisable:
        return _masks.bitmap_from_callable(eff_scalar, bm.B, Hm, bm.Q_LEN, bm.KV_LEN, batch_dependent=bm.B > 1)


class _NotVectorisable(Exception):
    pass


class _Strict:
    """Calls ``fn`` on index arrays and refuses scalars, so that a ``mask_mod`` that cannot
    broadcast is retried element by element with the scalar form instead."""

    def __init__(self, fn):
        self.fn = fn

    def __call__(self, b, h, q, k):
        if np.ndim(q) == 0:
            raise _NotVectorisable()
        return self.fn(b, h, q, k)


def flex_route(block_mask: Optional[BlockMask], B: int, Hq: int, tiles, device) -> str:
    """Which of "lists" / "terms" / "table" a BlockMask takes; ``tiles`` are the (q, kv) tile
    pairs of the passes that will run."""
    if block_mask is None:
        return "terms"
    terms = _structured_terms(block_mask.mask_mod)
    if terms is None or (terms.seg_q is not None and block_mask.B != B):
        return "table"
    if all(t == (block_mask.Q_BLOCK_SIZE, block_mask.KV_BLOCK_SIZE) for t in tiles):
        return "lists"
    return "terms" if _lists_match_terms(block_mask, terms, B, Hq, device) else "table"


def score_mod_affine(score_mod: Callable, B: int, H: int, L: int, S: int):
    """(a, w) with ``score_mod(score, b, h, q, k) == a * score + w[h] * k + (terms constant along k)``
    for ``h`` in ``range(H)``.  The reference calls score_mod with the KV-head index
    (jaxmodules/attention.py:543-554: ``score_mod(score, b, h, ...)`` inside the loop over kv heads),
    so ``flex_attention`` probes ``H = Hkv`` heads and repeats ``w`` over each query-head group.

    Terms that do not vary with the key index cancel in the softmax, so such a score_mod — ALiBi
    ``score + slope[h] * (k - q)``, the relative-position bias of the reference's
    tests/test_attention.py:131-132 — is a logit scale ``a`` plus a per-head key bias ``w``,
    which the kernels apply (``bma_attn_args.key_bias``).  The function is probed with Python
    numbers on a few scores and index pairs per head; anything that is not of this form (not
    affine in the score, not linear in k, or a key slope that depends on the batch index or the
    query index) raises NotImplementedError."""
    def f(s, b, h, q, k):
        return float(score_mod(np.float64(s), b, h, q, k))
    qs = sorted({0, L // 3, L - 1})
    ks = sorted({0, S // 2, S - 1}) if S > 2 else list(range(S))
    a_ref, w = None, np.zeros(H, dtype=np.float64)
    for b in sorted({0, B - 1}):
        for h in range(H):
            base = f(0.0, b, h, qs[0], ks[0])
            a = f(1.0, b, h, qs[0], ks[0]) - base
            slope = (f(0.0, b, h, qs[0], ks[-1]) - base) / (ks[-1] - ks[0]) if len(ks) > 1 else 0.0
            a_ref = a if a_ref is None else a_ref
            for q in qs:
                row0 = f(0.0, b, h, q, ks[0])
                for k in ks:
                    for sc in (-1.5, 0.0, 2.0):
                        want = a_ref * sc + row0 + slope * (k - ks[0])
                        if abs(f(sc, b, h, q, k) - want) > 1e-6 * (1.0 + abs(want)):
                            raise NotImplementedError(
                                "score_mod must be a * score + w[h] * k + (terms constant along k); other score "
                                "modifications are not implemented on the CUDA path")
            if b == 0:
                w[h] = slope
            elif abs(w[h] - slope) > 1e-6 * (1.0 + abs(slope)):
                raise NotImplementedError("score_mod: the key slope must not depend on the batch index")
    return float(a_ref), w


def flex_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, score_mod: Optional[Callable] = None,
                   block_mask: Optional[BlockMask] = None, scale: Optional[float] = None, enable_gqa: bool = False,
                   return_lse: bool = False, *, out_dtype: Optional[torch.dtype] = None,
                   backend: int = nat.BMA_BACKEND_AUTO) -> torch.Tensor:
    """Drop-in for ``flex_attention`` of jaxmodules/attention.py:458-692.

    query ``[B, Hq, L, E]``, key / value ``[B, Hkv, S, E]`` (any strides with a contiguous
    last dimension; nothing is copied).  Returns ``[B, Hq, L, E]`` float32 like the reference
    (``out_dtype=torch.bfloat16`` halves the output traffic).  Differentiable in query, key and
    value.  Shape checks and their messages follow jaxmodules/attention.py:501-531;
    ``return_lse`` raises NotImplementedError as there (:491-492).  ``score_mod``: functions of the form
    ``a * score + w[h] * k_idx + (terms constant along k_idx)`` (see ``score_mod_affine``; ``h`` is the kv-head
    index, as in the reference) run on the same kernels as a logit scale plus a per-head key bias — a
    compile-time variant of the tcgen05 kernels for bf16, the SIMT kernels for float32; others raise
    NotImplementedError."""
    if return_lse:
        raise NotImplementedError("return_lse is not supported yet")
    if query.ndim != 4 or key.ndim != 4 or value.ndim != 4:
        raise ValueError("query, key and value must be [B, H, L, E]")
    B, Hq, L, E = query.shape
    Bk, Hkv, S, Ek = key.shape
    Bv, Hv, Sv, Ev = value.shape
    assert E == Ek, "query and key must have the same embedding dimension"
    assert B == Bk, "query and key must have the same batch dimension"
    assert Sv == S, "value and key must have the same sequence length"
    assert Bv == B, "value and query must have the same batch dimension"
    assert Hv == Hkv, "value and key must have the same head count"
    if Ev != E:
        raise NotImplementedError("value head dimension must equal the query / key head dimension")
    if block_mask is not None:
        assert L == block_mask.Q_LEN, "query length must match block mask"
        assert S == block_mask.KV_LEN, "key length must match block mask"
        assert L % block_mask.Q_BLOCK_SIZE == 0, "query length must be divisible by Q_BLOCK_SIZE"
        assert S % block_mask.KV_BLOCK_SIZE == 0, "key length must be divisible by KV_BLOCK_SIZE"
    if not enable_gqa:
        assert Hq == Hkv, "query and key must have the same head count, unless enable_gqa is True"
    assert Hq % Hkv == 0, "kv head count must divide query head count"
    if block_mask is not None:
        if block_mask.B not in (1, B) or block_mask.H not in (1, Hq):
            raise ValueError("block_mask batch / head extents must be 1 or match the query")
    # score_mod sees the kv-head index, like the reference (:543-554); raises for other forms
    affine = None if score_mod is None else score_mod_affine(score_mod, B, Hkv, L, S)
    if not (query.is_cuda and key.is_cuda and value.is_cuda):
        raise RuntimeError("flex_attention needs CUDA tensors; there is no CPU path")
    if query.dtype not in (torch.float32, torch.bfloat16) or key.dtype != query.dtype or value.dtype != query.dtype:
        raise TypeError("query, key, value must share dtype float32 or bfloat16")

    fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
    Q, K, V = fix(query).transpose(1, 2), fix(key).transpose(1, 2), fix(value).transpose(1, 2)
    dev = Q.device
    lists_fn = None
    key_bias = None
    if affine is not None:
        scale = affine[0] * (1.0 / math.sqrt(E) if scale is None else float(scale))
        if np.any(affine[1] != 0.0):   # the kernels index the bias with the query head: hq = hkv * G + g
            key_bias = torch.from_numpy(np.repeat(affine[1], Hq // Hkv).astype(np.float32)).to(dev)
    with torch.cuda.device(dev):
        if block_mask is None:
            terms = _masks.MaskTerms()
        else:
            tiles = [_att.plan(Q, K, V, backend, key_bias=key_bias)[1:]]
            if torch.is_grad_enabled() and (query.requires_grad or key.requires_grad or value.requires_grad):
                tiles.append(_att.plan(Q, K, V, backend, backward=True, key_bias=key_bias)[1:])
            route = flex_route(block_mask, B, Hq, tiles, dev)
            if route == "table":
                terms = _masks.MaskTerms(bitmap=_effective_table(block_mask, Hq // Hkv, Hq))
            else:
                terms = _structured_terms(block_mask.mask_mod)
                if route == "lists":
                    # fitted once per BlockMask and device (the reference's BlockMask is immutable as well)
                    cached = getattr(block_mask, "_ready_lists", None)
                    if cached is None or cached.device != dev:
                        cached = _ReadyLists(block_mask, dev)
                        try:
                            block_mask._ready_lists = cached
                        except AttributeError:
                            pass
                    lists_fn = cached
        O, _ = _att._MaskedAttention.apply(Q, K, V, terms, out_dtype or torch.float32, backend,
                                           None if scale is None else float(scale), lists_fn, key_bias)
    return O.transpose(1, 2)
