"""Device-evaluable mask descriptions for ``mask_fn(b, h, q, k)``.

The reference accepts an arbitrary Python callable (jaxmodules/attention.py:354, 368-372)
and traces it with vmap.  A CUDA kernel cannot call Python, so a mask reaches the device in
one of two forms:

* a *structured* mask built by the factories below (``causal_mask``, ``sliding_window_mask``,
  ``document_mask``, ``and_masks``).  They are ordinary callables with the reference's
  ``(b, h, q, k)`` signature — usable anywhere a ``mask_fn`` is — that also carry the terms
  the kernels evaluate in registers;
* any other callable is evaluated once on the host over the full index grid and shipped as a
  bit-packed table (1 bit per (b, h, q, k); a 3-argument ``(h, q, k)`` callable gives a
  batch-independent table).  Only sensible up to a few thousand positions.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass, field
from typing import Callable, Optional, Tuple

import numpy as np
import torch

from . import _native as nat

_BIG = 1 << 30
MAX_BITMAP_BITS = 1 << 34  # 2 GiB of table; beyond this a structured mask is required


@dataclass(frozen=True)
class MaskTerms:
    """AND of the enabled terms; see ``bma_mask_spec`` in include/bma.h."""
    causal: bool = False
    band: Optional[Tuple[int, int]] = None           # (left, right): q-left <= k <= q+right
    seg_q: Optional[torch.Tensor] = None             # [B, >=N] int32
    seg_k: Optional[torch.Tensor] = None             # [B, >=L] int32
    window: Optional[Tuple[int, int, int, int]] = None   # (block, left_blocks, right_blocks, num_kv_blocks)
    bitmap: Optional[torch.Tensor] = None            # [Bm, Hm, Q, words] int32 (bit pattern of uint32)
    tiles: Optional[tuple] = None                    # (tile_class uint8 [Bm,Hm,TQ,TK], tile_slot int32, tile_bits int32 [cut,2,128,4])
    q_offset: int = 0
    k_offset: int = 0

    def merged(self, other: "MaskTerms") -> "MaskTerms":
        band = self.band
        if other.band is not None:
            band = other.band if band is None else (min(band[0], other.band[0]), min(band[1], other.band[1]))
        if self.seg_q is not None and other.seg_q is not None:
            raise NotImplementedError("and_masks: only one document_mask term is supported")
        if (self.bitmap is not None and other.bitmap is not None) or (self.tiles is not None and other.tiles is not None):
            raise NotImplementedError("and_masks: only one table-backed term is supported")
        return MaskTerms(
            causal=self.causal or other.causal, band=band,
            seg_q=self.seg_q if self.seg_q is not None else other.seg_q,
            seg_k=self.seg_k if self.seg_k is not None else other.seg_k,
            window=self.window or other.window,
            bitmap=self.bitmap if self.bitmap is not None else other.bitmap,
            tiles=self.tiles if self.tiles is not None else other.tiles,
            q_offset=self.q_offset or other.q_offset, k_offset=self.k_offset or other.k_offset)


class StructuredMask:
    """A ``mask_fn`` that the kernels can evaluate: callable as ``m(b, h, q, k)`` on ints or
    broadcastable NumPy arrays, with the device terms in ``m.terms``."""

    def __init__(self, terms: MaskTerms, fn: Callable, name: str):
        self.terms = terms
        self._fn = fn
        self.__name__ = name

    def __call__(self, b, h, q, k):
        return self._fn(b, h, q, k)

    def __repr__(self):
        return f"StructuredMask({self.__name__})"


def causal_mask() -> StructuredMask:
    """``q >= k`` — what ``is_causal=True`` installs (jaxmodules/attention.py:412-415)."""
    return StructuredMask(MaskTerms(causal=True), lambda b, h, q, k: q >= k, "causal")


def full_mask() -> StructuredMask:
    """Everything allowed — the default when no mask is given (jaxmodules/attention.py:417-419)."""
    return StructuredMask(MaskTerms(), lambda b, h, q, k: (q == q) & (k == k), "full")


def sliding_window_mask(left: int, right: int) -> StructuredMask:
    """``q - left <= k <= q + right`` (the explicit-window mask the reference's docstring
    recommends, jaxmodules/attention.py:378-382)."""
    left, right = int(left), int(right)
    if left < 0 or right < 0:
        raise ValueError("window extents must be non-negative")
    return StructuredMask(MaskTerms(band=(min(left, _BIG), min(right, _BIG))),
                          lambda b, h, q, k: (k >= q - left) & (k <= q + right), f"sliding({left},{right})")


def document_mask(seg_q, seg_k=None, causal: bool = False) -> StructuredMask:
    """``seg_q[b, q] == seg_k[b, k]`` (packed documents), optionally AND ``k <= q``.

    ``seg_q``/``seg_k``: integer arrays [B, N] / [B, L] (tensor or ndarray); ``seg_k``
    defaults to ``seg_q``."""
    sq = torch.as_tensor(np.asarray(seg_q.cpu()) if isinstance(seg_q, torch.Tensor) else np.asarray(seg_q))
    sk = sq if seg_k is None else torch.as_tensor(np.asarray(seg_k.cpu()) if isinstance(seg_k, torch.Tensor) else np.asarray(seg_k))
    if sq.ndim != 2 or sk.ndim != 2 or sq.shape[0] != sk.shape[0]:
        raise ValueError("segment ids must be [B, N] and [B, L]")
    sq = sq.to(torch.int32).contiguous()
    sk = sk.to(torch.int32).contiguous()
    sq_np, sk_np = sq.numpy(), sk.numpy()

    def fn(b, h, q, k):
        same = sq_np[b, q] == sk_np[b, k]
        return (same & (k <= q)) if causal else same

    return StructuredMask(MaskTerms(causal=causal, seg_q=sq, seg_k=sk), fn,
                          "document_causal" if causal else "document")


def and_masks(*masks) -> StructuredMask:
    """Conjunction of structured masks."""
    if not masks or not all(isinstance(m, StructuredMask) for m in masks):
        raise TypeError("and_masks takes StructuredMask arguments")
    terms = masks[0].terms
    for m in masks[1:]:
        terms = terms.merged(m.terms)

    def fn(b, h, q, k):
        out = masks[0](b, h, q, k)
        for m in masks[1:]:
            out = out & m(b, h, q, k)
        return out

    return StructuredMask(terms, fn, "&".join(m.__name__ for m in masks))


def argcount(fn) -> int:
    """Positional-argument count the way the reference reads it
    (``mask_fn.__code__.co_argcount``, jaxmodules/attention.py:405)."""
    if isinstance(fn, StructuredMask):
        return 4
    code = getattr(fn, "__code__", None)
    if code is not None:
        return code.co_argcount
    return fn.__call__.__code__.co_argcount - 1


def bitmap_from_callable(mask_fn, B: int, H: int, N: int, L: int, batch_dependent: bool) -> torch.Tensor:
    """Evaluate ``mask_fn(b, h, q, k)`` over the whole grid on the host and bit-pack it along k
    (bit k%32 of word k//32).  Returns an int32 CPU tensor [Bm, H, N, ceil(L/32)]."""
    Bm = B if batch_dependent else 1
    if Bm * H * N * L > MAX_BITMAP_BITS:
        raise NotImplementedError(
            "mask_fn is an arbitrary callable and its table would exceed 2 GiB; build the mask with "
            "jaxmodules_b200.masks (causal_mask, sliding_window_mask, document_mask, and_masks)")
    b = np.arange(Bm, dtype=np.int64)[:, None, None, None]
    h = np.arange(H, dtype=np.int64)[None, :, None, None]
    q = np.arange(N, dtype=np.int64)[None, None, :, None]
    k = np.arange(L, dtype=np.int64)[None, None, None, :]
    try:
        dense = np.broadcast_to(np.asarray(mask_fn(b, h, q, k)), (Bm, H, N, L)).astype(bool)
    except Exception:
        dense = np.zeros((Bm, H, N, L), dtype=bool)
        for bi in range(Bm):
            for hi in range(H):
                for qi in range(N):
                    for ki in range(L):
                        dense[bi, hi, qi, ki] = bool(mask_fn(bi, hi, qi, ki))
    words = (L + 31) // 32
    padded = np.zeros((Bm, H, N, words * 32), dtype=bool)
    padded[..., :L] = dense
    packed = np.packbits(padded, axis=-1, bitorder="little")        # uint8, little bit order
    packed = packed.reshape(Bm, H, N, words, 4).copy().view("<u4").reshape(Bm, H, N, words)
    return torch.from_numpy(packed.view(np.int32).copy())


@dataclass
class DeviceMask:
    """A MaskTerms resolved for one call: owns the device copies that the C struct points at."""
    spec: nat.MaskSpec
    keep: tuple = field(default_factory=tuple)
    depends_b: bool = False
    depends_h: bool = False


# Device copies of host-side mask arrays (segment ids, bit tables), kept for as long as the source tensor lives and
# has not been written to: a mask object built once is shipped to the GPU once, not at every attention call, and the
# per-mask caches further down (visited-block counts) can recognise it by its device tensor.
_device_copies = {}   # id(source) -> (weakref to source, {(device, dtype): (source version, copy)})


def _on_device(t: torch.Tensor, device, dtype=None) -> torch.Tensor:
    device = torch.device(device)
    dtype = dtype or t.dtype
    if t.device == device and t.dtype == dtype and t.is_contiguous():
        return t
    entry = _device_copies.get(id(t))
    if entry is None or entry[0]() is not t:
        entry = (weakref.ref(t), {})
        _device_copies[id(t)] = entry
        weakref.finalize(t, _device_copies.pop, id(t), None)
    hit = entry[1].get((device, dtype))
    if hit is not None and hit[0] == t._version:
        return hit[1]
    copy = t.to(device=device, dtype=dtype).contiguous()
    entry[1][(device, dtype)] = (t._version, copy)
    return copy


def to_device_mask(terms: MaskTerms, N: int, L: int, device) -> DeviceMask:
    s = nat.MaskSpec()
    keep = []
    flags = 0
    s.q_valid, s.k_valid = N, L
    s.q_offset, s.k_offset = terms.q_offset, terms.k_offset
    if terms.causal:
        flags |= nat.BMA_MASK_CAUSAL
    if terms.band is not None:
        flags |= nat.BMA_MASK_BAND
        s.band_left, s.band_right = min(terms.band[0], _BIG), min(terms.band[1], _BIG)
    if terms.window is not None:
        flags |= nat.BMA_MASK_BLOCK_WINDOW
        s.win_block, s.win_left, s.win_right, s.win_nblk = terms.window
    depends_b = depends_h = False
    if terms.seg_q is not None:
        flags |= nat.BMA_MASK_SEGMENT
        sq = _on_device(terms.seg_q, device, torch.int32)
        sk = sq if terms.seg_k is terms.seg_q else _on_device(terms.seg_k, device, torch.int32)
        if sq.shape[1] < N + terms.q_offset or sk.shape[1] < L + terms.k_offset:
            raise ValueError("segment id arrays are shorter than the sequences")
        keep += [sq, sk]
        s.seg_q, s.seg_k = sq.data_ptr(), sk.data_ptr()
        s.seg_q_stride, s.seg_k_stride = sq.stride(0), sk.stride(0)
        depends_b = True
    if terms.bitmap is not None:
        flags |= nat.BMA_MASK_BITMAP
        bm = _on_device(terms.bitmap, device)
        keep.append(bm)
        s.bitmap = bm.data_ptr()
        s.bitmap_B, s.bitmap_H, s.bitmap_q, s.bitmap_words = bm.shape
        depends_b = depends_b or bm.shape[0] > 1
        depends_h = bm.shape[1] > 1
    if terms.tiles is not None:
        flags |= nat.BMA_MASK_TILES
        cls, slot, bits = (_on_device(t, device) for t in terms.tiles)
        if cls.shape[2] * 128 < N + terms.q_offset or cls.shape[3] * 128 < L + terms.k_offset:
            raise ValueError("the mask's tile grid is smaller than the sequences")
        keep += [cls, slot, bits]
        s.tile_class, s.tile_slot, s.tile_bits = cls.data_ptr(), slot.data_ptr(), bits.data_ptr()
        s.tiles_B, s.tiles_H, s.tiles_q, s.tiles_k = cls.shape
        depends_b = depends_b or cls.shape[0] > 1
        depends_h = depends_h or cls.shape[1] > 1
    s.flags = flags
    return DeviceMask(spec=s, keep=tuple(keep), depends_b=depends_b, depends_h=depends_h)


# A traced mask_fn whose dense table would be larger than this many bits is stored in the TILES form instead (4 KB per
# 128 x 128 tile that the mask cuts; whole and empty tiles cost a byte): 2^26 bits = 8 MiB of table.
TILES_ABOVE_BITS = 1 << 26


def _table_from_program(mask_fn, nargs: int, B: int, Hq: int, N: int, L: int, device):
    """``mask_fn`` evaluated on the GPU from its traced program: MaskTerms with the dense bit table (small masks) or
    with the tile form (large ones), or None when the function cannot be traced (it is then evaluated on the host)."""
    from . import mask_program as mp
    try:
        prog = mp.trace(mask_fn, nargs)
    except mp.TraceError:
        return None
    Bm, Hm = (B if prog.uses_b else 1), (Hq if prog.uses_h else 1)
    if Bm * Hm * N * L >= TILES_ABOVE_BITS:
        return MaskTerms(tiles=mp.build_tiles(prog, B, Hq, N, L, device))
    if Bm * Hm * N * L > MAX_BITMAP_BITS:
        raise NotImplementedError(
            "the bit table of this mask_fn would exceed 2 GiB; build the mask with "
            "jaxmodules_b200.masks (causal_mask, sliding_window_mask, document_mask, and_masks)")
    return MaskTerms(bitmap=mp.build_table(prog, B, Hq, N, L, device))


# Bit tables already built for a callable: function object -> {(B, Hq, N, L, device): MaskTerms}.  The reference
# re-traces mask_fn at every call (jaxmodules/attention.py:70-73); here the table of a given function object is built
# once per shape and device.  A function whose result depends on state it captured and that state changes must be
# passed as a new function object (or the cache cleared with clear_mask_cache()).
_terms_of_callable = weakref.WeakKeyDictionary()


def clear_mask_cache() -> None:
    """Forgets every cached bit table, device copy and per-mask count."""
    _terms_of_callable.clear()
    _device_copies.clear()
    _visited_counts.clear()


def terms_from_mask_fn(mask_fn, B: int, Hq: int, N: int, L: int, device=None) -> MaskTerms:
    """Structured masks pass through; any other callable becomes a bit table — built on the GPU
    from the traced mask program when ``device`` is a CUDA device and the function can be traced
    (arithmetic, comparisons, ``& | ~``, ``mask_program.where`` / ``Table``), evaluated on the host
    over index grids otherwise.  The table is cached on the function object (see ``clear_mask_cache``)."""
    if mask_fn is None:
        return MaskTerms()
    if isinstance(mask_fn, StructuredMask):
        t = mask_fn.terms
        if t.seg_q is not None and t.seg_q.shape[0] != B:
            raise ValueError("document_mask batch size differs from the batch size of Q")
        return t
    key = (B, Hq, N, L, None if device is None else str(torch.device(device)))
    try:
        cached = _terms_of_callable.get(mask_fn)
    except TypeError:          # not weak-referenceable (a callable object without __weakref__): never cached
        cached = None
    if cached is not None and key in cached:
        return cached[key]
    terms = _build_terms_from_callable(mask_fn, B, Hq, N, L, device)
    try:
        _terms_of_callable.setdefault(mask_fn, {})[key] = terms
    except TypeError:
        pass
    return terms


def _build_terms_from_callable(mask_fn, B: int, Hq: int, N: int, L: int, device=None) -> MaskTerms:
    n = argcount(mask_fn)
    if n in (3, 4) and device is not None and torch.device(device).type == "cuda":
        terms = _table_from_program(mask_fn, n, B, Hq, N, L, device)
        if terms is not None:
            return terms
    if n == 3:
        fn = lambda b, h, q, k: mask_fn(h, q, k)
        return MaskTerms(bitmap=bitmap_from_callable(fn, B, Hq, N, L, batch_dependent=False))
    if n == 4:
        return MaskTerms(bitmap=bitmap_from_callable(mask_fn, B, Hq, N, L, batch_dependent=True))
    raise TypeError("mask_fn must take (b, h, q, k) or (h, q, k)")


# ---- visited-block counts per mask ---------------------------------------------------------------
# The backward scratch is sized by the number of visited blocks, which lives on the device.  It is fetched once per
# distinct mask (a host synchronisation) and remembered: masks without arrays by their parameters, masks with arrays
# by the identity and version of their device tensors.
_visited_counts = {}   # key -> (weakrefs of the mask's device tensors, numpy int64 [LB * LH])


def visited_counts(dmask: DeviceMask, lists: "nat.BlockLists", device, extra_key=()):
    """Host int64 array [lists.B * lists.H] of visited (full + partial) blocks per list head for the lists just
    compiled from ``dmask``; cached per mask, shape and tile size."""
    import ctypes as C
    s = dmask.spec
    key = (s.flags, s.q_valid, s.k_valid, s.q_offset, s.k_offset, s.band_left, s.band_right, s.win_block, s.win_left,
           s.win_right, s.win_nblk, tuple((id(t), t._version, tuple(t.shape)) for t in dmask.keep),
           lists.B, lists.H, lists.NQ, lists.NKV, lists.q_block, lists.kv_block, str(torch.device(device))) + tuple(extra_key)
    hit = _visited_counts.get(key)
    if hit is not None and all(r() is t for r, t in zip(hit[0], dmask.keep)):
        return hit[1]
    out = torch.empty((lists.B * lists.H,), dtype=torch.int64, device=device)
    nat.check(nat.lib().bma_block_lists_visited(C.byref(lists), out.data_ptr(), torch.cuda.current_stream(device).cuda_stream),
              "bma_block_lists_visited")
    counts = out.cpu().numpy().copy()          # synchronises once per distinct mask
    if len(_visited_counts) > 256:
        _visited_counts.clear()
    _visited_counts[key] = (tuple(weakref.ref(t) for t in dmask.keep), counts)
    return counts
