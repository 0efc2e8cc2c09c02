"""Multi-GPU execution of the attention path: one process per GPU.

Attention is independent per (batch, kv-head group) — the reference has no cross-(b, h) term
(jaxmodules/attention.py:70-105 is batched over B and H only element-wise) — so the default
partition deals contiguous ranges of the ``B * Hkv`` units to the ranks and needs no collective
(``shard_units`` / ``sharded_attention``).

For sequences too long for one device the sequence axis can be split instead
(``ring_attention_forward``): every rank keeps its query chunk, the K/V chunks rotate around the
ring with point-to-point sends (``torch.distributed`` over NCCL on GPUs) into local buffers, every
step attends one chunk with global query/key offsets in the mask, and the partial results are
merged with their log-sum-exps.  The reference itself is single-device; this mode has no
counterpart there.
"""
from __future__ import annotations

import ctypes as C
import os
from datetime import timedelta
from typing import Callable, List, Optional, Tuple

import torch

from . import _native as nat
from . import masks as _masks


def shard_range(units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) of ``units`` items for ``rank``: sizes differ by at most one."""
    if not (0 <= rank < world):
        raise ValueError("rank outside the world")
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_units(B: int, Hkv: int, rank: int, world: int) -> List[Tuple[int, int, int]]:
    """The (batch, kv_head_lo, kv_head_hi) slices that make up this rank's range of the
    flattened ``B * Hkv`` units; a kv head's query-head group always stays together."""
    lo, hi = shard_range(B * Hkv, rank, world)
    out = []
    u = lo
    while u < hi:
        b, h0 = divmod(u, Hkv)
        h1 = min(Hkv, h0 + (hi - u))
        out.append((b, h0, h1))
        u += h1 - h0
    return out


def _offset_mask(mask_fn, b0: int, h0: int):
    """The same mask seen from a shard whose batch / query-head indices start at (b0, h0)."""
    if mask_fn is None:
        return None
    if isinstance(mask_fn, _masks.StructuredMask):
        t = mask_fn.terms
        if t.bitmap is not None:
            raise NotImplementedError("table-backed masks cannot be re-indexed for a shard; use a callable")
        if t.seg_q is None:
            return mask_fn
        terms = _masks.MaskTerms(causal=t.causal, band=t.band, seg_q=t.seg_q[b0:b0 + 1], seg_k=t.seg_k[b0:b0 + 1],
                                 window=t.window, q_offset=t.q_offset, k_offset=t.k_offset)
        return _masks.StructuredMask(terms, lambda b, h, q, k: mask_fn(b + b0, h + h0, q, k), mask_fn.__name__)
    if _masks.argcount(mask_fn) == 3:
        return lambda h, q, k: mask_fn(h + h0, q, k)
    return lambda b, h, q, k: mask_fn(b + b0, h + h0, q, k)


def sharded_attention(Q, K, V, *, rank: int, world: int, attend: Optional[Callable] = None, **kwargs):
    """Runs this rank's share of ``masked_attention_via_map(Q, K, V, **kwargs)``.

    Q, K, V are the full tensors (or views of them) visible to this process; the result is a
    list of ``((b, hq_lo, hq_hi), O_slice)`` for the slices of ``shard_units``.  No communication
    happens here; gather the slices only if one array is wanted.  ``attend`` replaces the CUDA
    call (tests inject a CPU stand-in)."""
    if attend is None:
        from .attention import masked_attention_via_map as attend
    B, N, Hq, d = Q.shape
    Hkv = K.shape[2]
    G = Hq // Hkv
    out = []
    mask_fn = kwargs.pop("mask_fn", None)
    for b, h0, h1 in shard_units(B, Hkv, rank, world):
        q = Q[b:b + 1, :, h0 * G:h1 * G]
        k = K[b:b + 1, :, h0:h1]
        v = V[b:b + 1, :, h0:h1]
        o = attend(q, k, v, mask_fn=_offset_mask(mask_fn, b, h0 * G), **kwargs)
        out.append(((b, h0 * G, h1 * G), o))
    return out


# ---------------------------------------------------------------------------------------------
# ring sequence partition (forward)
# ---------------------------------------------------------------------------------------------

def cuda_attend(Q, K, V, terms: _masks.MaskTerms):
    """One partial attention on the CUDA kernels: (O float32, lse)."""
    from .attention import attention_forward
    O, lse, _ = attention_forward(Q, K, V, terms, out_dtype=torch.float32)
    return O, lse


def cuda_merge(O, lse, O2, lse2):
    """In-place merge of (O2, lse2) into (O, lse) with ``bma_attn_merge``."""
    from .attention import _tensor
    a = nat.AttnArgs()
    a.B, a.N, a.Hq, a.d = O.shape
    a.L, a.Hkv = 1, a.Hq
    a.o, a.d_o = _tensor(O), _tensor(O2)
    a.lse, a.delta = lse.data_ptr(), lse2.data_ptr()
    with torch.cuda.device(O.device):
        nat.check(nat.lib().bma_attn_merge(C.byref(a), torch.cuda.current_stream(O.device).cuda_stream), "bma_attn_merge")
    return O, lse


def ring_schedule(rank: int, world: int) -> List[int]:
    """Owner of the K/V chunk a rank holds at each ring step: its own first, then the chunks of
    its predecessors as they arrive from rank-1."""
    return [(rank - s) % world for s in range(world)]


def _step_terms(terms: _masks.MaskTerms, q_offset: int, k_offset: int) -> _masks.MaskTerms:
    return _masks.MaskTerms(causal=terms.causal, band=terms.band, seg_q=terms.seg_q, seg_k=terms.seg_k,
                            window=terms.window, bitmap=terms.bitmap, tiles=terms.tiles, q_offset=terms.q_offset + q_offset,
                            k_offset=terms.k_offset + k_offset)


def contiguous_layout(n_local: int) -> Callable[[int, int], List[Tuple[int, int]]]:
    """Rank r holds tokens [r*n, (r+1)*n)."""
    return lambda rank, world: [(rank * n_local, n_local)]


def zigzag_layout(n_local: int) -> Callable[[int, int], List[Tuple[int, int]]]:
    """The sequence is cut into 2*world chunks and rank r holds chunks r and 2*world-1-r (its local
    tensors are the two chunks back to back).  Under a causal mask every rank then has the same
    number of allowed (query, key) pairs at every ring step, where the contiguous layout leaves
    rank 0 idle for world-1 steps."""
    if n_local % 2:
        raise ValueError("zig-zag layout needs an even local length")
    c = n_local // 2
    return lambda rank, world: [(rank * c, c), ((2 * world - 1 - rank) * c, c)]


def _segments(layout, rank: int, world: int):
    """[(local start, global start, length)] of a rank's local sequence."""
    out, pos = [], 0
    for g0, n in layout(rank, world):
        out.append((pos, g0, n))
        pos += n
    return out


def _pair_is_empty(terms: _masks.MaskTerms, q0: int, qn: int, k0: int, kn: int) -> bool:
    """True when the interval terms alone rule out every (q, k) of the pair (no launch needed)."""
    q_lo, q_hi = terms.q_offset + q0, terms.q_offset + q0 + qn - 1
    k_lo, k_hi = terms.k_offset + k0, terms.k_offset + k0 + kn - 1
    if terms.causal and k_lo > q_hi:
        return True
    if terms.band is not None and (k_hi < q_lo - terms.band[0] or k_lo > q_hi + terms.band[1]):
        return True
    return False


def _pair_is_full(terms: _masks.MaskTerms, q0: int, qn: int, k0: int, kn: int) -> bool:
    """True when the mask consists of interval terms only and they allow every (q, k) of the pair."""
    if terms.seg_q is not None or terms.bitmap is not None or terms.tiles is not None or terms.window is not None:
        return False
    q_lo, q_hi = terms.q_offset + q0, terms.q_offset + q0 + qn - 1
    k_lo, k_hi = terms.k_offset + k0, terms.k_offset + k0 + kn - 1
    if terms.causal and k_hi > q_lo:
        return False
    if terms.band is not None and (k_lo < q_hi - terms.band[0] or k_hi > q_lo + terms.band[1]):
        return False
    return True


def _step_calls(terms: _masks.MaskTerms, q_segs, k_segs):
    """The attention calls of one ring step: [(q local start, q length, k local start, k length, terms)].

    One call per (query segment, key segment) pair that the mask does not empty, except that pairs the mask leaves
    untouched are joined along the segment axis they share — segments lie back to back in the local buffers — into one
    unmasked call: under a causal mask with the zig-zag layout every step but the first is then ONE call (both query
    segments against the older visiting segment, or the later query segment against both visiting segments) instead
    of two, with half the mask compiles, merges and accumulations."""
    join = os.environ.get("BMA_RING_JOIN", "1") != "0"      # 0: one call per pair (for measurements)
    state = [["empty" if _pair_is_empty(terms, qg, qn, kg, kn) else "full" if join and _pair_is_full(terms, qg, qn, kg, kn) else "cut"
              for (_, kg, kn) in k_segs] for (_, qg, qn) in q_segs]
    done = [[st == "empty" for st in row] for row in state]
    calls, free = [], _masks.MaskTerms()
    q_all = (q_segs[0][0], sum(n for _, _, n in q_segs))
    for j, (kl, kg, kn) in enumerate(k_segs):            # every query segment sees this key segment whole
        if len(q_segs) > 1 and all(state[i][j] == "full" for i in range(len(q_segs))):
            calls.append((q_all[0], q_all[1], kl, kn, free))
            for i in range(len(q_segs)):
                done[i][j] = True
    for i, (ql, qg, qn) in enumerate(q_segs):
        rest = [j for j in range(len(k_segs)) if not done[i][j]]
        if len(rest) > 1 and rest == list(range(rest[0], rest[-1] + 1)) and all(state[i][j] == "full" for j in rest):
            calls.append((ql, qn, k_segs[rest[0]][0], sum(k_segs[j][2] for j in rest), free))
            continue
        for j in rest:
            kl, kg, kn = k_segs[j]
            calls.append((ql, qn, kl, kn, free if state[i][j] == "full" else _step_terms(terms, qg, kg)))
    return calls


class RingTransferError(RuntimeError):
    """A ring step could not complete: a neighbour holds a chunk of another shape, or a transfer did not finish
    within the deadline (a rank that died, left, or never entered the call)."""


def _wait_all(reqs, timeout_s: Optional[float], what: str) -> None:
    """Waits for point-to-point requests, turning a time-out or a transport error into RingTransferError.  The
    deadline is enforced on the host by backends whose wait blocks the host (gloo; NCCL with blocking wait);
    otherwise the process group's own timeout ends a transfer whose peer is gone."""
    for r in reqs:
        try:
            if timeout_s is None:
                r.wait()
            else:
                r.wait(timedelta(seconds=timeout_s))
        except Exception as e:   # gloo raises RuntimeError, NCCL DistBackendError
            raise RingTransferError(f"{what}: transfer did not complete ({type(e).__name__}: {e})") from e


def _check_neighbours(K: torch.Tensor, rank: int, world: int, group, timeout_s: Optional[float]) -> None:
    """Exchanges the chunk geometry with both ring neighbours before any K/V moves: every rank must hold chunks of the
    same shape and dtype (a receive buffer of the wrong size would corrupt or stall the ring).  Costs one tiny
    message each way and a host synchronisation per call."""
    import torch.distributed as dist
    if world == 1:
        return
    mine = tuple(int(x) for x in K.shape) + (K.element_size(),)
    send = torch.tensor(mine, dtype=torch.int64, device=K.device)
    recv = torch.empty_like(send)
    dst, src = (rank + 1) % world, (rank - 1) % world
    reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, send, dst, group), dist.P2POp(dist.irecv, recv, src, group)])
    _wait_all(reqs, timeout_s, f"rank {rank}: geometry exchange with ranks {src} / {dst}")
    theirs = tuple(int(x) for x in recv.cpu())
    if theirs != mine:
        raise RingTransferError(f"rank {rank}: rank {src} holds K/V chunks of shape {theirs[:-1]} ({theirs[-1]} bytes per "
                                f"element), this rank {mine[:-1]} ({mine[-1]}): every rank must hold an equal share")


def ring_attention_forward(Q, K, V, *, rank: int, world: int, is_causal: bool = False,
                           terms: Optional[_masks.MaskTerms] = None, group=None,
                           attend: Callable = cuda_attend, merge: Callable = cuda_merge, layout=None,
                           timeout_s: Optional[float] = None, validate: bool = True, exchange: Optional[Callable] = None):
    """Forward attention over a sequence split across ``world`` ranks.

    Q ``[B, n, Hq, d]`` and K, V ``[B, n, Hkv, d]`` are this rank's tokens (equal sizes on every
    rank); ``layout(rank, world)`` says which global token ranges they are — ``contiguous_layout``
    (default) or ``zigzag_layout``.  Returns (O float32, lse) for the local queries.  Each step
    posts the send of the K/V it holds to rank+1 and the receive of the next from rank-1 before it
    computes, so the transfer runs under the kernels; received data always lands in this device's
    own memory before a kernel reads it.  Within a step every (local query range, visiting key
    range) pair is one attention call with the global offsets in the mask description; pairs the
    interval terms rule out entirely are skipped.

    Failure handling: with ``validate`` the ranks first compare chunk shapes with their neighbours; every wait takes
    ``timeout_s`` (None = the process group's own timeout).  Either check raises ``RingTransferError`` instead of
    hanging or reading a half-filled buffer.  ``exchange(tensors, dst, src)`` replaces the point-to-point transfer
    and returns the received tensors (measurements of the compute alone pass a stub)."""
    import torch.distributed as dist
    terms = terms or _masks.MaskTerms(causal=is_causal)
    layout = layout or contiguous_layout(Q.shape[1])
    q_segs = _segments(layout, rank, world)
    k_cur, v_cur = K.contiguous(), V.contiguous()
    if validate and exchange is None:
        _check_neighbours(k_cur, rank, world, group, timeout_s)
    parts = [None] * len(q_segs)          # (O, lse) per local query range
    # two receive pairs used in turn: the pair received at step s is sent at step s+1 and free again at step s+2
    kv_bufs = [[torch.empty_like(k_cur), torch.empty_like(v_cur)] for _ in range(2)] if exchange is None and world > 1 else None
    for s, owner in enumerate(ring_schedule(rank, world)):
        reqs = []
        if s + 1 < world:
            dst, src = (rank + 1) % world, (rank - 1) % world
            if exchange is not None:
                k_nxt, v_nxt = exchange([k_cur, v_cur], dst, src)
            else:
                k_nxt, v_nxt = kv_bufs[s & 1]
                ops = [dist.P2POp(dist.isend, k_cur, dst, group), dist.P2POp(dist.isend, v_cur, dst, group),
                       dist.P2POp(dist.irecv, k_nxt, src, group), dist.P2POp(dist.irecv, v_nxt, src, group)]
                reqs = dist.batch_isend_irecv(ops)
        for ql, qn, kl, kn, call_terms in _step_calls(terms, q_segs, _segments(layout, owner, world)):
            O_s, lse_s = attend(Q[:, ql:ql + qn], k_cur[:, kl:kl + kn], v_cur[:, kl:kl + kn], call_terms)
            for i, (sl, _, sn) in enumerate(q_segs):     # a call may cover several local query segments
                if not ql <= sl < ql + qn:
                    continue
                whole = (sl, sn) == (ql, qn)
                O_i = O_s if whole else O_s[:, sl - ql:sl - ql + sn]
                lse_i = lse_s if whole else lse_s[:, :, sl - ql:sl - ql + sn].contiguous()
                parts[i] = (O_i, lse_i) if parts[i] is None else merge(parts[i][0], parts[i][1], O_i, lse_i)
        _wait_all(reqs, timeout_s, f"rank {rank}: K/V rotation, ring step {s}")
        if s + 1 < world:
            k_cur, v_cur = k_nxt, v_nxt
    for i, (ql, qg, qn) in enumerate(q_segs):
        if parts[i] is None:   # a query range without any allowed key anywhere
            parts[i] = (torch.zeros((Q.shape[0], qn, Q.shape[2], Q.shape[3]), dtype=torch.float32, device=Q.device),
                        torch.full((Q.shape[0], Q.shape[2], qn), float("-inf"), dtype=torch.float32, device=Q.device))
    if len(parts) == 1:
        return parts[0]
    return torch.cat([p[0] for p in parts], dim=1), torch.cat([p[1] for p in parts], dim=2)


# ---------------------------------------------------------------------------------------------
# ring sequence partition (backward)
# ---------------------------------------------------------------------------------------------

def cuda_backward(Q, K, V, O, lse, dO, terms: _masks.MaskTerms, reuse: Optional[dict] = None):
    """Gradients of one (query chunk, key chunk) pair on the CUDA kernels.  ``O`` and ``lse`` are
    the FINAL output and log-sum-exp of the local queries over the whole sequence, so that
    ``P = exp(s - lse)`` and ``delta = rowsum(dO * O)`` are the global quantities and the three
    partial gradients simply add up over the key chunks.  ``reuse``: a dict kept by the caller per
    query chunk — ``delta`` and the bf16 copy of ``dO`` depend on the queries only, so the first call
    stores them there and the calls against the other key chunks skip the preprocess kernel."""
    from .attention import attention_backward
    dmask = _masks.to_device_mask(terms, Q.shape[1], K.shape[1], Q.device)
    return attention_backward(Q, K, V, O, lse, dO, dict(dmask=dmask, reuse=reuse))


def ring_attention_backward(Q, K, V, O, lse, dO, *, rank: int, world: int, is_causal: bool = False,
                            terms: Optional[_masks.MaskTerms] = None, group=None,
                            backward: Callable = cuda_backward, exchange: Optional[Callable] = None, layout=None,
                            timeout_s: Optional[float] = None):
    """dQ, dK, dV for a sequence split across ``world`` ranks (the counterpart of
    ``ring_attention_forward`` with the same ``layout``; ``O`` / ``lse`` are its results for the
    local queries).

    K and V travel round the ring as in the forward pass, and the float32 accumulators of dK and
    dV travel with them, one step behind: at step s this rank computes the contribution of its
    queries to the tokens it holds into a buffer of its own, and only then takes the accumulator
    that the previous rank sent at the end of ITS step s-1 — a transfer that has run under this
    step's kernels — adds the two and posts the sum to rank+1.  So neither the K/V transfer (posted
    before the step's kernels) nor the accumulator transfer (posted after them, awaited a step
    later) sits on the critical path.  After the last step one more wait brings every accumulator
    home to the rank that owns the tokens.  dQ stays local (float32 accumulation over the steps).
    Receive buffers are two fixed pairs used in turn; nothing is allocated per step.

    ``exchange(tensors, dst, src)`` replaces the point-to-point transfer (it returns the received
    tensors); the default uses ``torch.distributed.batch_isend_irecv`` on ``group``."""
    import torch.distributed as dist
    terms = terms or _masks.MaskTerms(causal=is_causal)
    layout = layout or contiguous_layout(Q.shape[1])
    q_segs = _segments(layout, rank, world)
    dst, src = (rank + 1) % world, (rank - 1) % world

    def start(tensors, recv):
        """Posts send(tensors) -> dst and recv -> src; returns (received tensors, requests to wait for)."""
        if exchange is not None:
            return exchange(tensors, dst, src), []
        ops = [dist.P2POp(dist.isend, t, dst, group) for t in tensors] + [dist.P2POp(dist.irecv, t, src, group) for t in recv]
        return recv, dist.batch_isend_irecv(ops)

    if world == 1 and exchange is None:
        exchange = lambda tensors, dst_, src_: tensors      # a ring of one: the hop to oneself
    f32 = dict(dtype=torch.float32, device=K.device)
    own = exchange is None                        # the default transfer receives into buffers kept here
    k_cur, v_cur = K.contiguous(), V.contiguous()
    # K/V: two receive pairs used in turn (the pair received at step s is sent at step s+1 and free again at s+2)
    kv_bufs = [[torch.empty_like(k_cur), torch.empty_like(v_cur)] for _ in range(2)] if own else None
    # accumulators: two pairs for the sums built here (one may still be in flight to rank+1 while the next is built)
    # and two pairs for the sums arriving from rank-1
    part_bufs = [[torch.empty(K.shape, **f32), torch.empty(V.shape, **f32)] for _ in range(2)]
    recv_bufs = [[torch.empty(K.shape, **f32), torch.empty(V.shape, **f32)] for _ in range(2)] if own else None
    dq_acc = torch.zeros(Q.shape, dtype=torch.float32, device=Q.device)
    O, dO = O.contiguous(), dO.contiguous()
    incoming, acc_reqs = None, []
    per_query_chunk, lse_chunks = {}, {}      # what depends on the local queries only is taken once, not once per step
    for s, owner in enumerate(ring_schedule(rank, world)):
        kv_next, kv_reqs = (None, [])
        if s + 1 < world:
            kv_next, kv_reqs = start([k_cur, v_cur], kv_bufs[s & 1] if own else None)
        dk_part, dv_part = part_bufs[s % len(part_bufs)]
        written = set()
        k_segs = _segments(layout, owner, world)
        for ql, qn, kl, kn, call_terms in _step_calls(terms, q_segs, k_segs):
            qs, ks = slice(ql, ql + qn), slice(kl, kl + kn)
            key = (ql, qn)
            extra = dict(reuse=per_query_chunk.setdefault(key, {})) if backward is cuda_backward else {}
            if key not in lse_chunks:
                lse_chunks[key] = lse[:, :, qs].contiguous()
            dq_s, dk_s, dv_s = backward(Q[:, qs], k_cur[:, ks], v_cur[:, ks], O[:, qs], lse_chunks[key],
                                        dO[:, qs], call_terms, **extra)
            dq_acc[:, qs] += dq_s
            for sl, _, sn in k_segs:                     # a call may cover several visiting key segments
                if not kl <= sl < kl + kn:
                    continue
                sub = slice(sl - kl, sl - kl + sn)
                if sl in written:
                    dk_part[:, sl:sl + sn] += dk_s[:, sub]
                    dv_part[:, sl:sl + sn] += dv_s[:, sub]
                else:          # the first contribution to these tokens in this step: no zero-fill, no read
                    dk_part[:, sl:sl + sn].copy_(dk_s[:, sub])
                    dv_part[:, sl:sl + sn].copy_(dv_s[:, sub])
                    written.add(sl)
        for kl, kg, kn in k_segs:
            if kl not in written:
                dk_part[:, kl:kl + kn].zero_()
                dv_part[:, kl:kl + kn].zero_()
        if incoming is not None:
            # sent by rank-1 at the end of its previous step; the transfer ran under this step's kernels
            _wait_all(acc_reqs, timeout_s, f"rank {rank}: dK/dV rotation, backward ring step {s - 1}")
            dk_part += incoming[0]
            dv_part += incoming[1]
        incoming, acc_reqs = start([dk_part, dv_part], recv_bufs[s & 1] if own else None)
        _wait_all(kv_reqs, timeout_s, f"rank {rank}: K/V rotation, backward ring step {s}")
        if kv_next is not None:
            k_cur, v_cur = kv_next
    # the last hop brings every accumulator back to the rank that owns the tokens
    _wait_all(acc_reqs, timeout_s, f"rank {rank}: dK/dV rotation, last hop")
    dk_acc, dv_acc = incoming
    return dq_acc.to(Q.dtype), dk_acc.to(K.dtype), dv_acc.to(V.dtype)
