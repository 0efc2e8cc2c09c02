"""JAX side of the drop-in: the custom calls of ``csrc/bma_jax.cc`` registered with ``jax.ffi`` and wrapped in the
``jax.custom_vjp`` triple the reference uses (jaxmodules/attention.py:180 ``@partial(jax.custom_vjp,
nondiff_argnames=[...])``, :244-264 forward rule, :266-273 backward rule, :345 ``defvjp``).

NOT compiled or tested where this library is developed: jax is not installed there.  Importing this module without
jax raises ImportError; nothing else in the package imports it.  The tested binding is the torch/ctypes one
(``attention.py``).  Masks are the structured ones of ``jaxmodules_b200.masks`` (causal, sliding window, documents,
block window); their block lists are compiled on the device inside the jitted program, one custom call.
"""
from __future__ import annotations

import ctypes
from functools import partial
from pathlib import Path

import numpy as np

try:
    import jax
    import jax.numpy as jnp
except ImportError as e:      # the guard the rest of the package relies on
    raise ImportError("jaxmodules_b200.jax_binding needs jax (and libbma_jax.so built against its FFI headers)") from e

from . import _native as nat
from . import masks as _masks

TILE = 128                    # bma_attn_plan: bf16, head dimension 64 / 128 -> the tcgen05 kernels, 128 x 128 tiles
_TARGETS = {"bma_mask_compile": "BmaMaskCompile", "bma_attn_fwd": "BmaAttnFwd", "bma_attn_bwd": "BmaAttnBwd"}
_registered = False


def register(lib_path=None) -> None:
    """Registers the three XLA custom-call targets (once per process)."""
    global _registered
    if _registered:
        return
    lib = ctypes.CDLL(str(lib_path or Path(__file__).resolve().parent / "libbma_jax.so"))
    for target, symbol in _TARGETS.items():
        jax.ffi.register_ffi_target(target, jax.ffi.pycapsule(getattr(lib, symbol)), platform="CUDA")
    _registered = True


def _mask_attr(terms: _masks.MaskTerms, N: int, L: int):
    """The eleven leading int32 fields of ``bma_mask_spec`` and the segment-id array (or a dummy)."""
    dm = _masks.to_device_mask(_masks.MaskTerms(causal=terms.causal, band=terms.band, window=terms.window,
                                                q_offset=terms.q_offset, k_offset=terms.k_offset), N, L, "cpu")
    s = dm.spec
    flags = s.flags | (nat.BMA_MASK_SEGMENT if terms.seg_q is not None else 0)
    fields = [flags, N, L, s.q_offset, s.k_offset, s.band_left, s.band_right, s.win_block, s.win_left, s.win_right, s.win_nblk]
    seg = jnp.asarray(np.asarray(terms.seg_q), dtype=jnp.int32) if terms.seg_q is not None else jnp.zeros((1, 1), jnp.int32)
    return np.asarray(fields, dtype=np.int32), seg, (terms.seg_q.shape[0] if terms.seg_q is not None else 1)


def _lists(mask, seg, LB, B, H, N, L):
    """One custom call: the eight BlockMask arrays at the kernels' tile size (+ the compile's workspace)."""
    NQ, NKV = -(-N // TILE), -(-L // TILE)
    i32 = lambda *shape: jax.ShapeDtypeStruct(shape, jnp.int32)
    ws = nat.lib().bma_mask_compile_workspace_bytes(ctypes.byref(_spec_of(mask)), B, H, NQ, NKV)
    out = (i32(LB, 1, NQ), i32(LB, 1, NQ, NKV)) * 2 + (i32(LB, 1, NKV), i32(LB, 1, NKV, NQ)) * 2 + (jax.ShapeDtypeStruct((max(ws, 1),), jnp.uint8),)
    return jax.ffi.ffi_call("bma_mask_compile", out)(seg, mask=mask, B=np.int32(B), H=np.int32(H), tile=np.int32(TILE))[:8]


def _spec_of(mask):
    s = nat.MaskSpec()
    (s.flags, s.q_valid, s.k_valid, s.q_offset, s.k_offset, s.band_left, s.band_right,
     s.win_block, s.win_left, s.win_right, s.win_nblk) = (int(x) for x in mask)
    return s


@partial(jax.custom_vjp, nondiff_argnums=(3, 4))
def _attention(Q, K, V, terms, scale):
    return _attention_fwd(Q, K, V, terms, scale)[0]


def _attention_fwd(Q, K, V, terms, scale):
    B, N, Hq, d = Q.shape
    L = K.shape[1]
    mask, seg, LB = _mask_attr(terms, N, L)
    lists = _lists(mask, seg, LB, B, Hq, N, L)
    out = (jax.ShapeDtypeStruct((B, N, Hq, d), jnp.float32), jax.ShapeDtypeStruct((B, Hq, N), jnp.float32))
    O, lse = jax.ffi.ffi_call("bma_attn_fwd", out)(Q, K, V, seg, *lists[:4], mask=mask, scale=np.float32(scale), tile=np.int32(TILE))
    return O, (Q, K, V, O, lse, seg, lists)        # saves O and lse: the backward does not recompute the forward


def _attention_bwd(terms, scale, res, g):
    Q, K, V, O, lse, seg, lists = res
    B, N, Hq, d = Q.shape
    L = K.shape[1]
    mask, _, _ = _mask_attr(terms, N, L)
    NQ, NKV = -(-N // TILE), -(-L // TILE)
    scratch = 8 * B * Hq * (NQ * NKV + NQ + 2) + 4096 + 32768 * B * Hq * NQ * NKV      # dense bound: tables + one slot per block
    out = (jax.ShapeDtypeStruct(Q.shape, Q.dtype), jax.ShapeDtypeStruct(K.shape, K.dtype), jax.ShapeDtypeStruct(V.shape, V.dtype),
           jax.ShapeDtypeStruct((B, Hq, N), jnp.float32), jax.ShapeDtypeStruct(Q.shape, jnp.bfloat16),
           jax.ShapeDtypeStruct((scratch,), jnp.uint8))
    dQ, dK, dV = jax.ffi.ffi_call("bma_attn_bwd", out)(Q, K, V, O, lse, g.astype(jnp.float32), seg, *lists, mask=mask,
                                                       visited=np.zeros((0,), np.int64), scale=np.float32(scale),
                                                       tile=np.int32(TILE))[:3]
    return dQ, dK, dV


_attention.defvjp(_attention_fwd, _attention_bwd)


def masked_attention_via_map(Q, K, V, *, is_causal=False, kernel_fn=None, mask_fn=None, block_size=None, window_size=None):
    """jaxmodules/attention.py:347-455 for jax arrays ``[B, L, H, d]`` (bf16, d = 64 or 128) on a CUDA device."""
    from .attention import default_kernel, kernel_log_affine
    register()
    if is_causal and mask_fn is not None:
        raise ValueError("cannot specify both 'is_causal' and 'mask_fn'!")
    if mask_fn is not None and not isinstance(mask_fn, _masks.StructuredMask):
        raise NotImplementedError("the jax binding takes the structured masks of jaxmodules_b200.masks")
    terms = _masks.MaskTerms(causal=True) if is_causal else (mask_fn.terms if mask_fn is not None else _masks.MaskTerms())
    N, L = Q.shape[1], K.shape[1]
    if window_size is not None:
        bs = N if block_size is None else int(block_size)
        lb, rb = (window_size[0] + bs - 1) // bs, 1 + (window_size[1] + bs - 1) // bs
        terms = terms.merged(_masks.MaskTerms(window=(bs, lb, rb, -(-L // bs))))
    scale, _ = kernel_log_affine(kernel_fn or default_kernel, K.shape[-1])
    return _attention(Q, K, V, terms, scale)
