"""``masked_attention_via_map`` with the reference's signature and error behaviour
(jaxmodules/attention.py:347-455), executing on sm_100a CUDA kernels through the C ABI.

Inputs are CUDA torch tensors ``[B, L, H, d]`` (or 3-D without the batch axis).  The result is
differentiable (torch autograd) — the counterpart of the reference's ``jax.custom_vjp``
(jaxmodules/attention.py:180, 244-345); the backward saves ``(Q, K, V, O, lse)`` instead of
recomputing the forward.  There is no CPU or eager-PyTorch path.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Callable, Optional, Tuple

import torch

from . import _native as nat
from . import masks as _masks
from .block_mask import compile_block_lists


def default_kernel(q, k):
    """Marker for the reference's default score ``exp(q.k / sqrt(d))``
    (jaxmodules/attention.py:39-50).  The CUDA kernels implement exactly this kernel; the
    function itself also evaluates it for host-side use."""
    q, k = torch.as_tensor(q), torch.as_tensor(k)
    return torch.exp(torch.dot(q, k) / math.sqrt(k.shape[-1]))


def threshold_kernel(threshold: Optional[float] = None):
    """jaxmodules/attention.py:18-36: ``exp(q.k - threshold / sqrt(d))`` — note that the dot
    product is NOT divided by sqrt(d).  The constant factor cancels in the normalised output,
    so on the CUDA path this is the softmax with scale 1 (the log-sum-exp is shifted by
    ``-threshold / sqrt(d)``)."""
    def kernel_fn(q, k):
        q, k = torch.as_tensor(q), torch.as_tensor(k)
        dotp = torch.dot(q, k)
        if threshold is not None:
            dotp = dotp - threshold / math.sqrt(q.shape[0])
        return torch.exp(dotp)
    kernel_fn.log_affine = lambda d: (1.0, 0.0 if threshold is None else -float(threshold) / math.sqrt(d))
    return kernel_fn


def kernel_log_affine(kernel_fn: Callable, d: int) -> Tuple[float, float]:
    """(a, b) with ``kernel_fn(q, k) == exp(a * q.k + b)`` for vectors of length ``d``.

    The CUDA kernels implement exactly this family (``a`` is their logit scale, ``b`` only
    shifts the log-sum-exp).  ``default_kernel`` and ``threshold_kernel`` carry the pair; any
    other callable is probed on random vectors (NumPy float64, then torch) and accepted when
    ``log kernel_fn`` is an affine function of the dot product to 1e-6, e.g. the custom kernel
    of the reference's tests/test_mapped_attention.py:1122-1142.  Everything else — kernels
    that are not exponentials of the dot product — raises NotImplementedError."""
    if kernel_fn is default_kernel:
        return 1.0 / math.sqrt(d), 0.0
    if hasattr(kernel_fn, "log_affine"):
        a, b = kernel_fn.log_affine(d)
        return float(a), float(b)
    import numpy as np
    rng = np.random.default_rng(0)
    xs, ys = [], []
    for i in range(12):
        # different norms and angles, dot products spread over roughly [-4, 4]
        q = rng.standard_normal(d) * (0.25 + 0.25 * (i % 4)) / math.sqrt(math.sqrt(d))
        k = rng.standard_normal(d) * (1.5 - 0.25 * (i % 5)) / math.sqrt(math.sqrt(d))
        if i % 3 == 0:
            k = k + q * (1.0 + i / 6.0)
        try:
            w = kernel_fn(q, k)
        except Exception:
            w = kernel_fn(torch.from_numpy(q), torch.from_numpy(k))
        w = float(w)
        if not (w > 0.0 and math.isfinite(w)):
            raise NotImplementedError("kernel_fn must be positive and finite; only exp(a*q.k + b) kernels run on the CUDA path")
        xs.append(float(q @ k))
        ys.append(math.log(w))
    A = np.stack([np.asarray(xs), np.ones(len(xs))], axis=1)
    (a, b), *_ = np.linalg.lstsq(A, np.asarray(ys), rcond=None)
    if np.abs(A @ np.array([a, b]) - np.asarray(ys)).max() > 1e-6 * (1.0 + np.abs(ys).max()):
        raise NotImplementedError("kernel_fn is not of the form exp(a*q.k + b); only such kernels run on the CUDA path")
    return float(a), float(b)


_DTYPES = {torch.float32: nat.BMA_DTYPE_F32, torch.bfloat16: nat.BMA_DTYPE_BF16}


def block_window(N: int, L: int, block_size: Optional[int], window_size: Optional[Tuple[int, int]]):
    """Block geometry exactly as the reference derives it, and its errors: padding only when N is not a multiple of
    ``block_size`` (jaxmodules/attention.py:426-434; then any L is accepted), otherwise L must be a whole number of
    blocks because the keys are cut into blocks of the QUERY block size (:155-158); ``block_size=None`` means one block
    of N queries (:195-196).  Returns None without ``window_size``, else ``(block, left_blocks, right_blocks, key_blocks)``
    with ``left = ceil(l / block)``, ``right = 1 + ceil(r / block)`` (:199-204); a window of more blocks than there are
    key blocks is an error (a shape error inside the reference's slice).  Nothing is physically padded on the CUDA
    path; the kernels bound-check instead."""
    bs = N if block_size is None else int(block_size)
    if bs <= 0:
        raise ValueError("block_size must be positive")
    if N % bs != 0:
        Lp = L + bs - (L % bs)
    else:
        Lp = L
        if L % bs != 0:
            raise ValueError("number of keys must be a multiple of block_size when the number of queries is")
    if window_size is None:
        return None
    left, right = window_size
    lb = (left + bs - 1) // bs
    rb = 1 + (right + bs - 1) // bs
    nkb = Lp // bs
    if lb + rb > nkb:
        raise ValueError("window_size covers more blocks than there are key blocks")
    return bs, lb, rb, nkb


def _tensor(t: Optional[torch.Tensor]) -> nat.Tensor:
    out = nat.Tensor()
    if t is None:
        return out
    if t.stride(-1) != 1:
        raise ValueError("innermost dimension must be contiguous")
    out.ptr = t.data_ptr()
    out.stride_b, out.stride_l, out.stride_h = t.stride(0), t.stride(1), t.stride(2)
    out.dtype = _DTYPES[t.dtype]
    return out


def _make_args(Q, K, V, backend=nat.BMA_BACKEND_AUTO, scale=None, key_bias=None) -> nat.AttnArgs:
    a = nat.AttnArgs()
    a.B, a.N, a.Hq, a.d = Q.shape
    a.L, a.Hkv = K.shape[1], K.shape[2]
    a.scale = 1.0 / math.sqrt(K.shape[-1]) if scale is None else float(scale)
    a.backend = backend
    a.q, a.k, a.v = _tensor(Q), _tensor(K), _tensor(V)
    if key_bias is not None:   # [Hq] float32 on the device, kept alive by the caller
        a.key_bias = key_bias.data_ptr()
    return a


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def plan(Q, K, V, backend=nat.BMA_BACKEND_AUTO, backward: bool = False, key_bias=None, scale=None):
    """(backend, q_tile, kv_tile) the library will use for the forward (or backward) pass."""
    a = _make_args(Q, K, V, backend, scale, key_bias)
    be, tq, tk = C.c_int32(), C.c_int32(), C.c_int32()
    fn = nat.lib().bma_attn_bwd_plan if backward else nat.lib().bma_attn_plan
    nat.check(fn(C.byref(a), C.byref(be), C.byref(tq), C.byref(tk)), "bma_attn_plan")
    return be.value, tq.value, tk.value


class _Span:
    """One launch group: an NVTX range named after it (visible in a timeline profiler, free otherwise) and,
    when ``sink`` is a dict, a CUDA-event bracket on the launching stream (the benchmark times single
    kernels with it)."""

    def __init__(self, sink, key, device):
        self.sink, self.key, self.device = sink, key, device

    def __enter__(self):
        torch.cuda.nvtx.range_push("bma." + self.key)
        if self.sink is not None:
            self.t0 = torch.cuda.Event(enable_timing=True)
            self.t1 = torch.cuda.Event(enable_timing=True)
            self.t0.record(torch.cuda.current_stream(self.device))
        return self

    def __exit__(self, *exc):
        if self.sink is not None:
            self.t1.record(torch.cuda.current_stream(self.device))
            self.sink.setdefault(self.key, []).append((self.t0, self.t1))
        torch.cuda.nvtx.range_pop()
        return False


_profile_sink = None

# Every wait inside the tensor-core kernels is bounded; a wait that gives up writes a code to a status word on
# the device and the kernel unwinds, leaving wrong results behind a BMA_OK launch.  Reading the word costs a
# stream synchronisation, so the hot path does not do it: call ``device_status`` wherever the stream is
# synchronised anyway (tests and the benchmark do), or set BMA_CHECK_STATUS=1 to check after every launch group.
_check_status = os.environ.get("BMA_CHECK_STATUS", "0") not in ("", "0")


def device_status(device=None) -> int:
    """Reads and clears the status word of ``device`` (synchronises its current stream).  0 = no bounded wait
    or bounds check inside a kernel has given up since the last read; otherwise the code of the first that did."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        code = C.c_int32()
        rc = nat.lib().bma_device_status(_stream(dev), C.byref(code))
        if rc not in (nat.BMA_OK, nat.BMA_ERR_DEVICE_CHECK):
            nat.check(rc, "bma_device_status")
        return int(code.value)


def _maybe_check_status(dev, where):
    if _check_status:
        code = device_status(dev)
        if code:
            raise RuntimeError(f"{where}: a bounded wait inside a kernel gave up (device status {code}); results are invalid")


def set_profile_sink(sink):
    """Install (or remove with None) a dict that collects (start, end) CUDA event pairs per
    launch group: 'mask_compile', 'fwd', 'bwd_preprocess', 'bwd'."""
    global _profile_sink
    _profile_sink = sink


def attention_forward(Q, K, V, terms: _masks.MaskTerms, *, out_dtype=torch.float32, backend=nat.BMA_BACKEND_AUTO,
                      need_q_side: bool = False, scale=None, lists_fn=None, key_bias=None):
    """One forward launch sequence: mask compile at the kernel's tile size, then attention.
    Returns (O, lse, ctx) where ctx carries what the backward needs.

    ``scale`` replaces 1/sqrt(d).  ``lists_fn(q_tile, kv_tile, q_side)`` supplies ready-made
    block lists (struct, tensors) instead of compiling them from the mask terms; it returns
    None when it has none for that tile size.  ``key_bias``: float32 ``[Hq]`` on the device, the
    logits get ``+ key_bias[h] * k`` (see ``bma_attn_args.key_bias``)."""
    lib = nat.lib()
    dev = Q.device
    B, N, Hq, d = Q.shape
    L = K.shape[1]
    with torch.cuda.device(dev):
        a = _make_args(Q, K, V, backend, scale, key_bias)
        be, tq, tk = plan(Q, K, V, backend, key_bias=key_bias, scale=scale)
        dmask = _masks.to_device_mask(terms, N, L, dev)
        # when the backward pass will walk the same tile size, build its q-side lists in the same launches
        both_sides = need_q_side and plan(Q, K, V, backend, backward=True, key_bias=key_bias, scale=scale)[1:] == (tq, tk)
        with _Span(_profile_sink, "mask_compile", dev):
            ready = lists_fn(tq, tk, both_sides) if lists_fn is not None else None
            lists, lt = ready if ready is not None else compile_block_lists(dmask, B, Hq, N, L, tq, tk, dev, q_side=both_sides, conservative=True)
        O = torch.empty((B, N, Hq, d), dtype=out_dtype, device=dev)
        lse = torch.empty((B, Hq, N), dtype=torch.float32, device=dev)
        a.o, a.lse = _tensor(O), lse.data_ptr()
        with _Span(_profile_sink, "fwd", dev):
            nat.check(lib.bma_attn_fwd(C.byref(a), C.byref(dmask.spec), C.byref(lists), _stream(dev)), "bma_attn_fwd")
        _maybe_check_status(dev, "bma_attn_fwd")
    ctx = dict(dmask=dmask, lists=lists, list_tensors=lt, backend=be, scale=scale, lists_fn=lists_fn,
               lists_tile=(tq, tk), lists_have_q_side=both_sides, key_bias=key_bias)
    return O, lse, ctx


def attention_backward(Q, K, V, O, lse, dO, ctx, backend=nat.BMA_BACKEND_AUTO):
    """dQ, dK, dV through ``bma_attn_bwd_preprocess`` + ``bma_attn_bwd``."""
    lib = nat.lib()
    dev = Q.device
    B, N, Hq, d = Q.shape
    L = K.shape[1]
    with torch.cuda.device(dev):
        a = _make_args(Q, K, V, backend, ctx.get("scale"), ctx.get("key_bias"))
        be, tq, tk = plan(Q, K, V, backend, backward=True, key_bias=ctx.get("key_bias"), scale=ctx.get("scale"))
        with _Span(_profile_sink, "mask_compile_bwd", dev):
            if ctx.get("lists_have_q_side") and ctx.get("lists_tile") == (tq, tk):
                lists, lt = ctx["lists"], ctx["list_tensors"]      # built by the forward pass
            else:
                lists_fn = ctx.get("lists_fn")
                ready = lists_fn(tq, tk, True) if lists_fn is not None else None
                lists, lt = ready if ready is not None else compile_block_lists(ctx["dmask"], B, Hq, N, L, tq, tk, dev, q_side=True, conservative=True)
        if dO.stride(-1) != 1:
            dO = dO.contiguous()
        delta = torch.empty((B, Hq, N), dtype=torch.float32, device=dev)
        dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
        a.o, a.lse, a.d_o, a.delta = _tensor(O), lse.data_ptr(), _tensor(dO), delta.data_ptr()
        a.dq, a.dk, a.dv = _tensor(dQ), _tensor(dK), _tensor(dV)
        st = _stream(dev)
        do_bf16 = None
        if be == nat.BMA_BACKEND_TCGEN05 and dO.dtype != torch.bfloat16:
            do_bf16 = torch.empty((B, N, Hq, d), dtype=torch.bfloat16, device=dev)
        reuse = ctx.get("reuse")       # a dict the caller keeps for one (O, dO): delta and the bf16 cotangent are taken once
        if reuse is not None and "delta" in reuse and (do_bf16 is None or reuse["do_bf16"] is not None):
            delta, do_bf16 = reuse["delta"], (reuse["do_bf16"] if do_bf16 is not None else None)
            a.delta = delta.data_ptr()
        else:
            with _Span(_profile_sink, "bwd_preprocess", dev):
                nat.check(lib.bma_attn_bwd_preprocess(C.byref(a), do_bf16.data_ptr() if do_bf16 is not None else None, st),
                          "bma_attn_bwd_preprocess")
            if reuse is not None:
                reuse["delta"], reuse["do_bf16"] = delta, do_bf16
        if do_bf16 is not None:
            a.d_o = _tensor(do_bf16)
        ws_bytes = lib.bma_attn_bwd_workspace_bytes(C.byref(a))
        # dS hand-over between the two backward kernels: only for lists whose two sides name the same blocks.
        # The scratch is sized by the blocks the mask visits (fetched once per mask, see masks.visited_counts).
        lists_fn = ctx.get("lists_fn")
        visited = scratch = 0
        if be == nat.BMA_BACKEND_TCGEN05 and _scratch_limit > 0 and (lists_fn is None or getattr(lists_fn, "consistent", False)):
            if lists_fn is None:
                counts = _masks.visited_counts(ctx["dmask"], lists, dev)
            else:
                counts = lists_fn.visited_counts(lists, dev)
            visited = (C.c_int64 * len(counts))(*[int(c) for c in counts])
            scratch = lib.bma_attn_bwd_scratch_bytes(C.byref(a), C.byref(lists), visited)
        given = min(scratch, _scratch_limit, int(scratch * _scratch_fraction) if _scratch_fraction < 1.0 else scratch)
        if 0 < given < scratch and given < lib.bma_attn_bwd_scratch_min_bytes(C.byref(a), C.byref(lists), visited):
            given = 0          # not even the largest (batch, kv head) unit fits: the dQ kernel recomputes, no buffer is needed
        if given > 0:
            ws, ws_bytes = _backward_scratch(dev, max(given, ws_bytes)), max(given, ws_bytes)
        else:
            ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=dev)
        last_backward_info.update(scratch_bytes=int(scratch), workspace_bytes=int(ws_bytes), whole=bool(scratch and given >= scratch))
        mid = None
        if _profile_sink is not None and be == nat.BMA_BACKEND_TCGEN05 and (given == 0 or given >= scratch):
            # the library records this event between its dK/dV pass and its dQ pass (only when it runs as one range)
            mid = torch.cuda.Event(enable_timing=True)
            mid.record(torch.cuda.current_stream(dev))
        with _Span(_profile_sink, "bwd", dev) as span:
            nat.check(lib.bma_attn_bwd(C.byref(a), C.byref(ctx["dmask"].spec), C.byref(lists), ws.data_ptr(), ws_bytes,
                                       visited if visited else None, mid.cuda_event if mid is not None else None, st),
                      "bma_attn_bwd")
        _maybe_check_status(dev, "bma_attn_bwd")
        if mid is not None:
            _profile_sink.setdefault("bwd_dkdv", []).append((span.t0, mid))
            _profile_sink.setdefault("bwd_dq_replay" if given >= scratch > 0 else "bwd_dq_recompute", []).append((mid, span.t1))
    return dQ, dK, dV


# Scratch of the tensor-core backward (the dS tiles handed from the dK/dV kernel to the dQ kernel): 32 KB per block the
# mask VISITS (a causal mask: half of the dense grid; a sliding window or packed documents: a small fraction) plus a
# few MB of slot tables, in one buffer per (device, stream) that grows to the largest call seen and is reused by
# every call in that stream's order.  A problem whose scratch exceeds the limit runs range by range over (batch,
# kv head) units through the same buffer; when not even the largest unit fits, the dQ kernel recomputes S and dP.
_scratch_limit = int(float(os.environ.get("BMA_BWD_SCRATCH_GB", "10")) * (1 << 30))   # environment override, in GiB
_scratch_fraction = 1.0
_scratch_buffers = {}
last_backward_info = {}    # sizes of the most recent backward call (diagnostics, tests)


def set_backward_scratch_limit(nbytes: int, fraction: float = 1.0) -> None:
    """Upper bound in bytes of the backward scratch buffer; 0 switches the dS hand-over off.  Buffers above the new
    limit are freed at once.  ``fraction`` < 1 additionally caps every call at that share of what it would need,
    which forces the backward to run in ranges (a knob for tests and for measuring what ranges cost)."""
    global _scratch_limit, _scratch_fraction
    _scratch_limit, _scratch_fraction = int(nbytes), float(fraction)
    for key in [k for k, t in _scratch_buffers.items() if t.numel() > _scratch_limit]:
        del _scratch_buffers[key]


def release_backward_scratch() -> None:
    """Frees every scratch buffer (they come back at the next backward call that wants one)."""
    _scratch_buffers.clear()


def _backward_scratch(dev: torch.device, nbytes: int) -> torch.Tensor:
    # keyed by stream too: two backward passes in flight on different streams must not share slots
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), torch.cuda.current_stream(dev).cuda_stream)
    buf = _scratch_buffers.get(key)
    if buf is None or buf.numel() < nbytes:
        _scratch_buffers.pop(key, None)   # drop the old buffer before asking for the larger one
        buf = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
        _scratch_buffers[key] = buf
    return buf


class _MaskedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, terms, out_dtype, backend, scale=None, lists_fn=None, key_bias=None):
        need_grad = any(ctx.needs_input_grad[:3])
        O, lse, fctx = attention_forward(Q, K, V, terms, out_dtype=out_dtype, backend=backend, need_q_side=need_grad,
                                         scale=scale, lists_fn=lists_fn, key_bias=key_bias)
        ctx.save_for_backward(Q, K, V, O, lse)
        ctx.fctx, ctx.backend = fctx, backend
        ctx.mark_non_differentiable(lse)
        return O, lse

    @staticmethod
    def backward(ctx, dO, _dlse):
        Q, K, V, O, lse = ctx.saved_tensors
        dQ, dK, dV = attention_backward(Q, K, V, O, lse, dO, ctx.fctx, ctx.backend)
        return dQ, dK, dV, None, None, None, None, None, None


def masked_attention_via_map(
    Q: torch.Tensor,
    K: torch.Tensor,
    V: torch.Tensor,
    *,
    is_causal: bool = False,
    kernel_fn: Callable = default_kernel,
    mask_fn: Optional[Callable] = None,
    block_size: Optional[int] = None,
    window_size: Optional[Tuple[int, int]] = None,
    out_dtype: Optional[torch.dtype] = None,
    return_lse: bool = False,
    backend: int = nat.BMA_BACKEND_AUTO,
):
    """Drop-in for jaxmodules/attention.py:347-455.

    K, V: ``[B, L, Hkv, d]`` or ``[L, Hkv, d]``; Q: ``[B, N, Hq, d]`` or ``[N, Hq, d]``.
    ``kernel_fn``: ``default_kernel``, ``threshold_kernel(t)`` or any callable equal to
    ``exp(a * q.k + b)`` (see ``kernel_log_affine``); other kernels raise NotImplementedError.
    ``mask_fn(b, h, q, k)`` or ``mask_fn(h, q, k)``; ``is_causal`` excludes ``mask_fn``.
    ``block_size`` / ``window_size`` keep the reference's meaning: the key window is a whole
    number of ``block_size`` blocks, clamped at the sequence ends, applied on top of the mask
    (jaxmodules/attention.py:161-167, 199-204); without ``window_size`` the result does not
    depend on ``block_size``.  Rows without any allowed key return 0.

    Extras (keyword-only, defaulting to the reference's behaviour): ``out_dtype`` — the
    reference returns float32 for every input dtype, pass ``torch.bfloat16`` to halve the
    output traffic; ``return_lse`` — also return the log-sum-exp ``[B, Hq, N]``.
    """
    if K.ndim not in (3, 4):
        raise ValueError("K must have 3 or 4 dimensions")
    if Q.ndim not in (3, 4):
        raise ValueError("Q must have 3 or 4 dimensions")
    if V.ndim not in (3, 4):
        raise ValueError("V must have 3 or 4 dimensions")
    assert K.ndim == Q.ndim and V.ndim == Q.ndim, "Q, K, and V must have the same number of dimensions"

    added_batch_dim = Q.ndim == 3
    if added_batch_dim:
        Q, K, V = Q[None], K[None], V[None]

    if is_causal and mask_fn is not None:
        raise ValueError("cannot specify both 'is_causal' and 'mask_fn'!")
    scale, shift = kernel_log_affine(kernel_fn, K.shape[-1])

    assert K.shape[0] == Q.shape[0] == V.shape[0], "Q, K, and V must have the same batch dimension"
    B, N, Hq, dq = Q.shape
    _, L, Hk, d = K.shape
    _, Lv, Hv, dv = V.shape
    assert d == dq and Lv == L and dv == d, f"shape mismatch in K {tuple(K.shape)}, Q {tuple(Q.shape)} and V {tuple(V.shape)}"
    assert Hq % Hk == 0, "Hq must be divisible by Hk"
    assert Hv == Hk, "Hv must be equal to Hk"
    block_window(N, L, block_size, window_size)      # argument errors first, wherever the tensors live
    if not (Q.is_cuda and K.is_cuda and V.is_cuda):
        raise RuntimeError("masked_attention_via_map needs CUDA tensors; there is no CPU path")
    if Q.dtype not in _DTYPES or K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise TypeError("Q, K, V must share dtype float32 or bfloat16")

    if is_causal:
        terms = _masks.MaskTerms(causal=True)
    else:
        terms = _masks.terms_from_mask_fn(mask_fn, B, Hq, N, L, device=Q.device)

    window = block_window(N, L, block_size, window_size)
    if window is not None:
        terms = terms.merged(_masks.MaskTerms(window=window))

    fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
    O, lse = _MaskedAttention.apply(fix(Q), fix(K), fix(V), terms, out_dtype or torch.float32, backend,
                                    None if kernel_fn is default_kernel else scale)
    if shift != 0.0 and return_lse:
        lse = lse + shift
    if added_batch_dim:
        O, lse = O[0], lse[0]
    return (O, lse) if return_lse else O
