"""``BlockMask`` and its builders with the reference's names, fields, shapes and dtypes
(jaxmodules/block_mask.py), holding torch tensors instead of JAX arrays.

``create_block_mask`` — the part of the hot path — runs the CUDA mask-compile kernels through
the C ABI (``bma_mask_compile``) and has no CPU path.  The remaining constructors and
converters are the reference's host-side helpers, written with tensor ops.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch

from . import _native as nat
from . import masks as _masks


def extract_block_size(BLOCK_SIZE) -> Tuple[int, int]:
    """jaxmodules/block_mask.py:10-14."""
    if isinstance(BLOCK_SIZE, int):
        return BLOCK_SIZE, BLOCK_SIZE
    q, kv = BLOCK_SIZE
    return int(q), int(kv)


def _eval_mask(mask_mod, b, h, q_idx: torch.Tensor, k_idx: torch.Tensor) -> torch.Tensor:
    """mask_mod on a [len(q_idx), len(k_idx)] grid (host evaluation with NumPy broadcasting)."""
    import numpy as np
    q = q_idx.cpu().numpy().astype(np.int64)[:, None]
    k = k_idx.cpu().numpy().astype(np.int64)[None, :]
    try:
        out = np.broadcast_to(np.asarray(mask_mod(int(b), int(h), q, k)), (q.shape[0], k.shape[1])).astype(bool)
    except Exception:
        out = np.zeros((q.shape[0], k.shape[1]), dtype=bool)
        for i in range(q.shape[0]):
            for j in range(k.shape[1]):
                out[i, j] = bool(mask_mod(int(b), int(h), int(q[i, 0]), int(k[0, j])))
    return torch.from_numpy(out.copy())


@dataclass
class BlockMask:
    """Fields of jaxmodules/block_mask.py:17-42.  ``kv_*`` list PARTIAL blocks per q-block row,
    ``full_kv_*`` FULL blocks; ``q_*`` / ``full_q_*`` the same per kv-block column."""
    B: int
    H: int
    Q_LEN: int
    KV_LEN: int
    Q_BLOCK_SIZE: int
    KV_BLOCK_SIZE: int
    kv_num_blocks: torch.Tensor
    kv_indices: torch.Tensor
    q_num_blocks: Optional[torch.Tensor]
    q_indices: Optional[torch.Tensor]
    full_kv_num_blocks: Optional[torch.Tensor]
    full_kv_indices: Optional[torch.Tensor]
    full_q_num_blocks: Optional[torch.Tensor]
    full_q_indices: Optional[torch.Tensor]
    mask_mod: Callable

    # -- converters (jaxmodules/block_mask.py:44-165) ------------------------------------
    def get_mask_for_partial_block(self, b, h, q_block_idx, kv_block_idx) -> torch.Tensor:
        """jaxmodules/block_mask.py:44-66."""
        q0 = int(q_block_idx) * self.Q_BLOCK_SIZE
        k0 = int(kv_block_idx) * self.KV_BLOCK_SIZE
        return _eval_mask(self.mask_mod, b, h, torch.arange(q0, q0 + self.Q_BLOCK_SIZE),
                          torch.arange(k0, k0 + self.KV_BLOCK_SIZE))

    def materialize_mask(self) -> torch.Tensor:
        """Dense int32 0/1 mask [B, H, Q_LEN, KV_LEN] from the kv-side lists
        (jaxmodules/block_mask.py:68-129).  Out-of-range list entries behave as under JAX:
        reads clamp, writes are dropped."""
        QB, KVB = self.Q_BLOCK_SIZE, self.KV_BLOCK_SIZE
        kv_num, kv_idx = self.kv_num_blocks.cpu(), self.kv_indices.cpu()
        f_num, f_idx = self.full_kv_num_blocks.cpu(), self.full_kv_indices.cpu()
        NQ = kv_num.shape[-1]
        out = torch.zeros((self.B, self.H, self.Q_LEN, self.KV_LEN), dtype=torch.bool)

        def at(t, *ix):
            return int(t[tuple(min(int(i), n - 1) for i, n in zip(ix, t.shape))])

        for b in range(self.B):
            for h in range(self.H):
                for i in range(NQ):
                    for s in range(at(kv_num, b, h, i)):
                        j = at(kv_idx, b, h, i, s)
                        if (j + 1) * KVB > self.KV_LEN or (i + 1) * QB > self.Q_LEN:
                            continue
                        out[b, h, i * QB:(i + 1) * QB, j * KVB:(j + 1) * KVB] = self.get_mask_for_partial_block(b, h, i, j)
                    for s in range(at(f_num, b, h, i)):
                        j = at(f_idx, b, h, i, s)
                        if (j + 1) * KVB > self.KV_LEN or (i + 1) * QB > self.Q_LEN:
                            continue
                        out[b, h, i * QB:(i + 1) * QB, j * KVB:(j + 1) * KVB] = True
        return out.to(torch.int32)

    def get_full_blocks(self) -> torch.Tensor:
        """jaxmodules/block_mask.py:131-142."""
        rows, cols = self.full_kv_num_blocks.shape[-1], self.full_q_num_blocks.shape[-1]
        return get_dense_from_kv_blocks(self.B, self.H, rows, cols, self.full_kv_num_blocks, self.full_kv_indices)

    def get_partial_blocks(self) -> torch.Tensor:
        """jaxmodules/block_mask.py:144-155."""
        rows, cols = self.kv_num_blocks.shape[-1], self.q_num_blocks.shape[-1]
        return get_dense_from_kv_blocks(self.B, self.H, rows, cols, self.kv_num_blocks, self.kv_indices)

    def to_dense(self) -> torch.Tensor:
        """jaxmodules/block_mask.py:157-165 (bool + bool is logical or in JAX)."""
        return self.get_full_blocks() | self.get_partial_blocks()

    # -- constructors (jaxmodules/block_mask.py:167-378) -----------------------------------
    @classmethod
    def full_mask(cls, B, H, Q_LEN, KV_LEN, BLOCK_SIZE, device=None):
        """jaxmodules/block_mask.py:167-184."""
        QB, KVB = extract_block_size(BLOCK_SIZE)
        NKV, NQ = KV_LEN // KVB, Q_LEN // QB
        return cls.from_kv_blocks(
            kv_num_blocks=torch.zeros((B, H, NQ), dtype=torch.int32, device=device),
            kv_indices=torch.ones((B, H, NQ, 1), dtype=torch.int32, device=device),
            full_kv_num_blocks=torch.full((B, H, NQ), NKV, dtype=torch.int32, device=device),
            full_kv_indices=torch.arange(NKV, dtype=torch.int32, device=device).expand(B, H, NQ, NKV).contiguous(),
            BLOCK_SIZE=(QB, KVB), mask_mod=_masks.full_mask(), seq_lengths=(Q_LEN, KV_LEN))

    @classmethod
    def causal_mask(cls, B, H, Q_LEN, KV_LEN, BLOCK_SIZE, device=None):
        """jaxmodules/block_mask.py:186-225: strictly-lower block triangle full, diagonal partial."""
        QB, KVB = extract_block_size(BLOCK_SIZE)
        NKV, NQ = KV_LEN // KVB, Q_LEN // QB
        full = torch.tril(torch.ones((NQ, NKV), dtype=torch.bool, device=device), -1).expand(B, H, NQ, NKV)
        partial = torch.eye(NQ, NKV, dtype=torch.bool, device=device).expand(B, H, NQ, NKV)
        kv_num, kv_idx = get_sparse_kv_data_from_blocks(partial)
        q_num, q_idx = get_sparse_q_data_from_blocks(partial)
        fkv_num, fkv_idx = get_sparse_kv_data_from_blocks(full)
        fq_num, fq_idx = get_sparse_q_data_from_blocks(full)
        return cls(B=B, H=H, Q_LEN=Q_LEN, KV_LEN=KV_LEN, Q_BLOCK_SIZE=QB, KV_BLOCK_SIZE=KVB,
                   kv_num_blocks=kv_num, kv_indices=kv_idx, q_num_blocks=q_num, q_indices=q_idx,
                   full_kv_num_blocks=fkv_num, full_kv_indices=fkv_idx,
                   full_q_num_blocks=fq_num, full_q_indices=fq_idx, mask_mod=_masks.causal_mask())

    @classmethod
    def from_blocks(cls, partial_blocks, full_blocks, BLOCK_SIZE, mask_mod):
        """jaxmodules/block_mask.py:227-275."""
        QB, KVB = extract_block_size(BLOCK_SIZE)
        partial_blocks = torch.as_tensor(partial_blocks).bool()
        full_blocks = torch.as_tensor(full_blocks).bool()
        partial_blocks = torch.where(full_blocks, torch.zeros_like(partial_blocks), partial_blocks)
        B, H, NQ, NKV = partial_blocks.shape
        kv_num, kv_idx = get_sparse_kv_data_from_blocks(partial_blocks)
        q_num, q_idx = get_sparse_q_data_from_blocks(partial_blocks)
        fkv_num, fkv_idx = get_sparse_kv_data_from_blocks(full_blocks)
        fq_num, fq_idx = get_sparse_q_data_from_blocks(full_blocks)
        return cls(B=B, H=H, Q_LEN=NQ * QB, KV_LEN=NKV * KVB, Q_BLOCK_SIZE=QB, KV_BLOCK_SIZE=KVB,
                   kv_num_blocks=kv_num, kv_indices=kv_idx, q_num_blocks=q_num, q_indices=q_idx,
                   full_kv_num_blocks=fkv_num, full_kv_indices=fkv_idx,
                   full_q_num_blocks=fq_num, full_q_indices=fq_idx, mask_mod=mask_mod)

    @classmethod
    def from_kv_blocks(cls, kv_num_blocks, kv_indices, full_kv_num_blocks, full_kv_indices, BLOCK_SIZE, mask_mod,
                       seq_lengths=None, generate_q_blocks: bool = False):
        """jaxmodules/block_mask.py:277-378 (rank lifting :291-298, KV_LEN inference :303-337)."""
        QB, KVB = extract_block_size(BLOCK_SIZE)
        kv_num_blocks, kv_indices = torch.as_tensor(kv_num_blocks), torch.as_tensor(kv_indices)
        full_kv_num_blocks, full_kv_indices = torch.as_tensor(full_kv_num_blocks), torch.as_tensor(full_kv_indices)
        if kv_num_blocks.ndim < 3:
            kv_num_blocks = kv_num_blocks.reshape(1, 1, -1)
        if kv_indices.ndim < 4:
            kv_indices = kv_indices.reshape(1, 1, *kv_indices.shape[-2:])
        if full_kv_num_blocks.ndim < 3:
            full_kv_num_blocks = full_kv_num_blocks.reshape(1, 1, -1)
        if full_kv_indices.ndim < 4:
            full_kv_indices = full_kv_indices.reshape(1, 1, *full_kv_indices.shape[-2:])
        B, H = kv_num_blocks.shape[0], kv_num_blocks.shape[1]
        if seq_lengths is None:
            Q_LEN = kv_indices.shape[2] * QB

            def max_index(num, idx):
                cols = torch.arange(idx.shape[3], device=idx.device)
                valid = cols < num[..., None]
                return int(torch.where(valid, idx.long(), torch.full_like(idx, -(1 << 31), dtype=torch.long)).max())

            KV_LEN = (max(max_index(kv_num_blocks, kv_indices), max_index(full_kv_num_blocks, full_kv_indices)) + 1) * KVB
        else:
            Q_LEN, KV_LEN = seq_lengths
        NQ, NKV = Q_LEN // QB, KV_LEN // KVB
        if not generate_q_blocks:
            return cls(B=B, H=H, Q_LEN=Q_LEN, KV_LEN=KV_LEN, Q_BLOCK_SIZE=QB, KV_BLOCK_SIZE=KVB,
                       kv_num_blocks=kv_num_blocks, kv_indices=kv_indices, q_num_blocks=None, q_indices=None,
                       full_kv_num_blocks=full_kv_num_blocks, full_kv_indices=full_kv_indices,
                       full_q_num_blocks=None, full_q_indices=None, mask_mod=mask_mod)
        partial = get_dense_from_kv_blocks(B, H, NQ, NKV, kv_num_blocks, kv_indices)
        full = get_dense_from_kv_blocks(B, H, NQ, NKV, full_kv_num_blocks, full_kv_indices)
        return cls.from_blocks(partial_blocks=partial, full_blocks=full, BLOCK_SIZE=BLOCK_SIZE, mask_mod=mask_mod)


def get_partial_block(mask_mod, b, h, block_q_idx, block_kv_idx, Q_BLOCK_SIZE, KV_BLOCK_SIZE, B=None, H=None):
    """jaxmodules/block_mask.py:381-408."""
    q0, k0 = int(block_q_idx) * Q_BLOCK_SIZE, int(block_kv_idx) * KV_BLOCK_SIZE
    return _eval_mask(mask_mod, b, h, torch.arange(q0, q0 + Q_BLOCK_SIZE), torch.arange(k0, k0 + KV_BLOCK_SIZE))


def get_sparse_kv_data_from_blocks(blocks):
    """jaxmodules/block_mask.py:411-432: counts and stable argsort(-blocks), int32."""
    blocks = torch.as_tensor(blocks).to(torch.int32)
    if blocks.ndim == 2:
        blocks = blocks[None, None]
    num = blocks.sum(dim=-1).to(torch.int32)
    idx = torch.argsort(-blocks, dim=-1, stable=True).to(torch.int32)
    return num, idx


def get_sparse_q_data_from_blocks(blocks):
    """jaxmodules/block_mask.py:435-451."""
    return get_sparse_kv_data_from_blocks(torch.as_tensor(blocks).transpose(-1, -2))


def get_dense_from_kv_blocks(B, H, NUM_Q_BLOCKS, NUM_KV_BLOCKS, kv_num_blocks, kv_indices) -> torch.Tensor:
    """jaxmodules/block_mask.py:501-536: bool [B,H,NQ,NKV] with the first ``num`` entries of
    each row set."""
    kv_num_blocks, kv_indices = torch.as_tensor(kv_num_blocks), torch.as_tensor(kv_indices)
    dev = kv_indices.device
    width = kv_indices.shape[-1]
    valid = torch.arange(width, device=dev) < kv_num_blocks[..., None]
    valid = valid & (kv_indices >= 0) & (kv_indices < NUM_KV_BLOCKS)
    data = torch.zeros((B, H, NUM_Q_BLOCKS, NUM_KV_BLOCKS + 1), dtype=torch.bool, device=dev)
    tgt = torch.where(valid, kv_indices.long(), torch.full_like(kv_indices, NUM_KV_BLOCKS, dtype=torch.long))
    data.scatter_(-1, tgt.expand(B, H, NUM_Q_BLOCKS, width), torch.ones_like(tgt, dtype=torch.bool).expand(B, H, NUM_Q_BLOCKS, width))
    return data[..., :NUM_KV_BLOCKS].contiguous()


# ---------------------------------------------------------------------------------------
# CUDA builder
# ---------------------------------------------------------------------------------------

def compile_block_lists(dmask: "_masks.DeviceMask", B: int, H: int, N: int, L: int, q_block: int, kv_block: int,
                        device, *, out_B: Optional[int] = None, out_H: Optional[int] = None, q_side: bool = True,
                        floor_blocks: bool = False, stream=None, conservative: bool = False):
    """Runs ``bma_mask_compile`` and returns (lists struct, dict of tensors).

    ``floor_blocks`` reproduces create_block_mask's ``LEN // BLOCK`` block counts
    (jaxmodules/block_mask.py:468-469); the attention kernels use ceil so that ragged tails
    are covered.  out_B/out_H default to the smallest extents the mask allows (1 where it does
    not depend on the index).  ``conservative`` sets BMA_MASK_COMPILE_CONSERVATIVE: segment-id blocks
    that the per-block id ranges cannot decide are listed as partial without an element scan — fine
    for lists the attention kernels consume, never used for the arrays ``create_block_mask`` returns."""
    lib = nat.lib()
    if floor_blocks:
        NQ, NKV = N // q_block, L // kv_block
    else:
        NQ, NKV = -(-N // q_block), -(-L // kv_block)
    if NQ <= 0 or NKV <= 0:
        raise ValueError("sequence shorter than one block")
    LB = out_B if out_B is not None else (B if dmask.depends_b else 1)
    LH = out_H if out_H is not None else (H if dmask.depends_h else 1)
    spec = dmask.spec
    if floor_blocks or conservative:
        spec = nat.MaskSpec.from_buffer_copy(spec)
    if floor_blocks:
        spec.q_valid, spec.k_valid = min(spec.q_valid, NQ * q_block), min(spec.k_valid, NKV * kv_block)
    if conservative:
        spec.flags |= nat.BMA_MASK_COMPILE_CONSERVATIVE
    i32 = dict(dtype=torch.int32, device=device)
    t = dict(
        kv_num_blocks=torch.empty((LB, LH, NQ), **i32), kv_indices=torch.empty((LB, LH, NQ, NKV), **i32),
        full_kv_num_blocks=torch.empty((LB, LH, NQ), **i32), full_kv_indices=torch.empty((LB, LH, NQ, NKV), **i32),
        q_num_blocks=None, q_indices=None, full_q_num_blocks=None, full_q_indices=None)
    if q_side:
        t.update(q_num_blocks=torch.empty((LB, LH, NKV), **i32), q_indices=torch.empty((LB, LH, NKV, NQ), **i32),
                 full_q_num_blocks=torch.empty((LB, LH, NKV), **i32), full_q_indices=torch.empty((LB, LH, NKV, NQ), **i32))
    lists = nat.BlockLists()
    lists.B, lists.H, lists.NQ, lists.NKV, lists.q_block, lists.kv_block = LB, LH, NQ, NKV, q_block, kv_block
    lists.kv_num, lists.kv_idx = t["kv_num_blocks"].data_ptr(), t["kv_indices"].data_ptr()
    lists.full_kv_num, lists.full_kv_idx = t["full_kv_num_blocks"].data_ptr(), t["full_kv_indices"].data_ptr()
    if q_side:
        lists.q_num, lists.q_idx = t["q_num_blocks"].data_ptr(), t["q_indices"].data_ptr()
        lists.full_q_num, lists.full_q_idx = t["full_q_num_blocks"].data_ptr(), t["full_q_indices"].data_ptr()
    ws_bytes = lib.bma_mask_compile_workspace_bytes(C.byref(spec), B, H, NQ, NKV)
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=device)
    st = stream if stream is not None else torch.cuda.current_stream(device).cuda_stream
    nat.check(lib.bma_mask_compile(C.byref(spec), B, H, C.byref(lists), ws.data_ptr(), ws_bytes, st), "bma_mask_compile")
    t["_workspace"] = ws  # keep alive until the stream has consumed it
    return lists, t


def create_block_mask(mask_mod, B: int, H: int, Q_LEN: int, KV_LEN: int, BLOCK_SIZE, device=None) -> BlockMask:
    """create_block_mask of jaxmodules/block_mask.py:454-498 on the GPU.

    ``mask_mod`` is a structured mask from ``jaxmodules_b200.masks`` or any ``(b, h, q, k)``
    callable (evaluated once on the host into a bit table).  Raises when no CUDA device is
    available — there is no CPU implementation."""
    if not torch.cuda.is_available():
        raise RuntimeError("create_block_mask runs on a CUDA device; none is available")
    device = torch.device(device if device is not None else "cuda")
    QB, KVB = extract_block_size(BLOCK_SIZE)
    with torch.cuda.device(device):
        terms = _masks.terms_from_mask_fn(mask_mod, B, H, Q_LEN, KV_LEN, device=device)
        dmask = _masks.to_device_mask(terms, Q_LEN, KV_LEN, device)
        _, t = compile_block_lists(dmask, B, H, Q_LEN, KV_LEN, QB, KVB, device, out_B=B, out_H=H, q_side=True,
                                   floor_blocks=True)
    NQ, NKV = Q_LEN // QB, KV_LEN // KVB
    return BlockMask(B=B, H=H, Q_LEN=NQ * QB, KV_LEN=NKV * KVB, Q_BLOCK_SIZE=QB, KV_BLOCK_SIZE=KVB,
                     kv_num_blocks=t["kv_num_blocks"], kv_indices=t["kv_indices"],
                     q_num_blocks=t["q_num_blocks"], q_indices=t["q_indices"],
                     full_kv_num_blocks=t["full_kv_num_blocks"], full_kv_indices=t["full_kv_indices"],
                     full_q_num_blocks=t["full_q_num_blocks"], full_q_indices=t["full_q_indices"], mask_mod=mask_mod)
