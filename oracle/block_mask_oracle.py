"""CPU restatement (NumPy) of jaxmodules' BlockMask construction.  TEST INFRASTRUCTURE ONLY.

This file is the checker for the CUDA mask-compile kernel.  Only tests, the smoke
check and the CPU-baseline leg of the benchmark may import it; the product package
never does.

Parity status: PINNED for integer work.  Every literal known-answer array in the
reference's tests/test_block_mask.py (stored as tests/golden/block_mask_known_answers.json)
is reproduced by these functions (tests/test_oracle_block_mask.py), and so is every index array that the
reference's own create_block_mask / BlockMask.causal_mask / full_mask produce for the eleven masks of
tests/golden/reference_cases.py (the reference's source run on a stand-in for jax by
tests/golden/make_reference_vectors.py; tests/test_reference_vectors.py).

Each function names the reference code it follows (paths inside acutkosky/jaxmodules).
"""
from __future__ import annotations

import numpy as np


def extract_block_size(BLOCK_SIZE):
    """jaxmodules/block_mask.py:10-14 — an int means square blocks."""
    if isinstance(BLOCK_SIZE, (int, np.integer)):
        return int(BLOCK_SIZE), int(BLOCK_SIZE)
    q, kv = BLOCK_SIZE
    return int(q), int(kv)


def eval_mask(mask_mod, b, h, q_idx, k_idx):
    """Evaluate mask_mod(b, h, q, k) on a [len(q_idx), len(k_idx)] grid -> bool array.

    The reference builds the same grid with nested vmaps (array_from_coords,
    jaxmodules/block_mask.py:404-408).  Vectorised NumPy broadcasting is tried
    first; a scalar Python loop is the fallback for callables that only accept ints.
    """
    q = np.asarray(q_idx, dtype=np.int64)[:, None]
    k = np.asarray(k_idx, dtype=np.int64)[None, :]
    try:
        out = mask_mod(b, h, q, k)
        out = np.broadcast_to(np.asarray(out), (q.shape[0], k.shape[1]))
        return out.astype(bool)
    except Exception:
        out = np.zeros((q.shape[0], k.shape[1]), dtype=bool)
        for i, qq in enumerate(q[:, 0]):
            for j, kk in enumerate(k[0, :]):
                out[i, j] = bool(mask_mod(b, h, int(qq), int(kk)))
        return out


def get_partial_block(mask_mod, b, h, block_q_idx, block_kv_idx, Q_BLOCK_SIZE, KV_BLOCK_SIZE, B=None, H=None):
    """jaxmodules/block_mask.py:381-408 — dense mask of one (q-block, kv-block)."""
    q0 = block_q_idx * Q_BLOCK_SIZE
    k0 = block_kv_idx * KV_BLOCK_SIZE
    return eval_mask(mask_mod, b, h, np.arange(q0, q0 + Q_BLOCK_SIZE), np.arange(k0, k0 + KV_BLOCK_SIZE))


def get_sparse_kv_data_from_blocks(blocks):
    """jaxmodules/block_mask.py:411-432.

    num = row sum (int32); indices = argsort(-blocks) along the last axis.  jnp.argsort is
    stable, so a row reads [set indices ascending ..., unset indices ascending ...] at full
    width.
    """
    blocks = np.asarray(blocks).astype(np.int32)
    if blocks.ndim == 2:
        blocks = blocks[None, None]
    num = blocks.sum(axis=-1).astype(np.int32)
    idx = np.argsort(-blocks, axis=-1, kind="stable").astype(np.int32)
    return num, idx


def get_sparse_q_data_from_blocks(blocks):
    """jaxmodules/block_mask.py:435-451 — the same on the (q, kv) transpose."""
    blocks = np.asarray(blocks)
    return get_sparse_kv_data_from_blocks(np.swapaxes(blocks, -1, -2))


def get_dense_from_kv_blocks(B, H, NUM_Q_BLOCKS, NUM_KV_BLOCKS, kv_num_blocks, kv_indices):
    """jaxmodules/block_mask.py:501-536 — scatter the first num indices of each row."""
    data = np.zeros((B, H, NUM_Q_BLOCKS, NUM_KV_BLOCKS), dtype=bool)
    kv_num_blocks = np.asarray(kv_num_blocks)
    kv_indices = np.asarray(kv_indices)
    for b in range(B):
        for h in range(H):
            for i in range(NUM_Q_BLOCKS):
                for j in range(int(kv_num_blocks[b, h, i])):
                    data[b, h, i, kv_indices[b, h, i, j]] = True
    return data


def classify_blocks(mask_mod, B, H, Q_LEN, KV_LEN, BLOCK_SIZE):
    """Block classification of create_block_mask (jaxmodules/block_mask.py:466-491).

    partial = any ^ all, full = all, per (b, h, q-block, kv-block); floor division of the
    lengths as in lines 468-469.  Streams one q-block row at a time so that the dense
    B*H*Q_LEN*KV_LEN mask is never materialised.
    """
    QB, KVB = extract_block_size(BLOCK_SIZE)
    NQ, NKV = Q_LEN // QB, KV_LEN // KVB
    partial = np.zeros((B, H, NQ, NKV), dtype=bool)
    full = np.zeros((B, H, NQ, NKV), dtype=bool)
    k_all = np.arange(NKV * KVB)
    for b in range(B):
        for h in range(H):
            for i in range(NQ):
                row = eval_mask(mask_mod, b, h, np.arange(i * QB, (i + 1) * QB), k_all)
                row = row.reshape(QB, NKV, KVB)
                any_ = row.any(axis=(0, 2))
                all_ = row.all(axis=(0, 2))
                partial[b, h, i] = any_ ^ all_
                full[b, h, i] = all_
    return partial, full


def from_blocks(partial_blocks, full_blocks, BLOCK_SIZE):
    """BlockMask.from_blocks (jaxmodules/block_mask.py:227-275) as a dict of arrays."""
    QB, KVB = extract_block_size(BLOCK_SIZE)
    partial_blocks = np.asarray(partial_blocks).astype(bool)
    full_blocks = np.asarray(full_blocks).astype(bool)
    partial_blocks = np.where(full_blocks, False, partial_blocks)  # lines 241-243
    B, H, NQ, NKV = partial_blocks.shape
    kv_num, kv_idx = get_sparse_kv_data_from_blocks(partial_blocks)
    q_num, q_idx = get_sparse_q_data_from_blocks(partial_blocks)
    fkv_num, fkv_idx = get_sparse_kv_data_from_blocks(full_blocks)
    fq_num, fq_idx = get_sparse_q_data_from_blocks(full_blocks)
    return dict(
        B=B, H=H, Q_LEN=NQ * QB, KV_LEN=NKV * KVB, Q_BLOCK_SIZE=QB, KV_BLOCK_SIZE=KVB,
        kv_num_blocks=kv_num, kv_indices=kv_idx, q_num_blocks=q_num, q_indices=q_idx,
        full_kv_num_blocks=fkv_num, full_kv_indices=fkv_idx,
        full_q_num_blocks=fq_num, full_q_indices=fq_idx,
    )


def create_block_mask(mask_mod, B, H, Q_LEN, KV_LEN, BLOCK_SIZE):
    """create_block_mask (jaxmodules/block_mask.py:454-498) as a dict of int32 arrays."""
    partial, full = classify_blocks(mask_mod, B, H, Q_LEN, KV_LEN, BLOCK_SIZE)
    out = from_blocks(partial, full, BLOCK_SIZE)
    out["mask_mod"] = mask_mod
    return out


def causal_mask(B, H, Q_LEN, KV_LEN, BLOCK_SIZE):
    """BlockMask.causal_mask (jaxmodules/block_mask.py:186-225): tri(-1) full, eye partial."""
    QB, KVB = extract_block_size(BLOCK_SIZE)
    NQ, NKV = Q_LEN // QB, KV_LEN // KVB
    full = np.broadcast_to(np.tri(NQ, NKV, -1, dtype=bool), (B, H, NQ, NKV))
    partial = np.broadcast_to(np.eye(NQ, NKV, dtype=bool), (B, H, NQ, NKV))
    kv_num, kv_idx = get_sparse_kv_data_from_blocks(partial)
    q_num, q_idx = get_sparse_q_data_from_blocks(partial)
    fkv_num, fkv_idx = get_sparse_kv_data_from_blocks(full)
    fq_num, fq_idx = get_sparse_q_data_from_blocks(full)
    return dict(
        B=B, H=H, Q_LEN=Q_LEN, KV_LEN=KV_LEN, Q_BLOCK_SIZE=QB, KV_BLOCK_SIZE=KVB,
        kv_num_blocks=kv_num, kv_indices=kv_idx, q_num_blocks=q_num, q_indices=q_idx,
        full_kv_num_blocks=fkv_num, full_kv_indices=fkv_idx,
        full_q_num_blocks=fq_num, full_q_indices=fq_idx,
        mask_mod=lambda b, h, q, k: q >= k,
    )


def full_mask(B, H, Q_LEN, KV_LEN, BLOCK_SIZE):
    """BlockMask.full_mask (jaxmodules/block_mask.py:167-184): no partial blocks, a dummy
    width-1 kv_indices of ones, full_kv_indices = arange; q-side left as None."""
    QB, KVB = extract_block_size(BLOCK_SIZE)
    NQ, NKV = Q_LEN // QB, KV_LEN // KVB
    return dict(
        B=B, H=H, Q_LEN=Q_LEN, KV_LEN=KV_LEN, Q_BLOCK_SIZE=QB, KV_BLOCK_SIZE=KVB,
        kv_num_blocks=np.zeros((B, H, NQ), np.int32),
        kv_indices=np.ones((B, H, NQ, 1), np.int32),
        full_kv_num_blocks=np.full((B, H, NQ), NKV, np.int32),
        full_kv_indices=np.broadcast_to(np.arange(NKV, dtype=np.int32), (B, H, NQ, NKV)).copy(),
        q_num_blocks=None, q_indices=None, full_q_num_blocks=None, full_q_indices=None,
        mask_mod=lambda b, h, q, k: True,
    )


def infer_kv_len(kv_num_blocks, kv_indices, full_kv_num_blocks, full_kv_indices, KV_BLOCK_SIZE):
    """KV_LEN inference of BlockMask.from_kv_blocks without seq_lengths
    (jaxmodules/block_mask.py:303-337): (largest index inside any valid prefix + 1) blocks."""
    def max_index(num, idx):
        num = np.asarray(num)
        idx = np.asarray(idx)
        cols = np.arange(idx.shape[-1])
        valid = cols < num[..., None]
        # rows with no valid entry contribute int32(-inf) in the reference, i.e. a very
        # negative value that never wins the maximum
        vals = np.where(valid, idx, np.iinfo(np.int32).min)
        return int(vals.max())
    return (max(max_index(kv_num_blocks, kv_indices), max_index(full_kv_num_blocks, full_kv_indices)) + 1) * KV_BLOCK_SIZE


def materialize_mask(bm):
    """BlockMask.materialize_mask (jaxmodules/block_mask.py:68-129): int32 0/1 dense mask
    from the kv-side lists; partial blocks are filled by re-evaluating mask_mod."""
    B, H = bm["B"], bm["H"]
    QB, KVB = bm["Q_BLOCK_SIZE"], bm["KV_BLOCK_SIZE"]
    NQ = np.asarray(bm["kv_num_blocks"]).shape[-1]
    out = np.zeros((B, H, bm["Q_LEN"], bm["KV_LEN"]), dtype=bool)

    def at(arr, *ix):
        # JAX gathers clamp out-of-range indices; the reference's own test
        # (tests/test_block_mask.py:86-88) relies on it with a 2-row full_kv_num_blocks.
        arr = np.asarray(arr)
        return int(arr[tuple(min(int(i), n - 1) for i, n in zip(ix, arr.shape))])

    for b in range(B):
        for h in range(H):
            for i in range(NQ):
                for s in range(at(bm["kv_num_blocks"], b, h, i)):
                    j = at(bm["kv_indices"], b, h, i, s)
                    if (j + 1) * KVB > bm["KV_LEN"]:
                        continue  # JAX drops out-of-range scatter updates (test_block_mask.py:84-86 has one)
                    out[b, h, i * QB:(i + 1) * QB, j * KVB:(j + 1) * KVB] = get_partial_block(
                        bm["mask_mod"], b, h, i, j, QB, KVB)
                for s in range(at(bm["full_kv_num_blocks"], b, h, i)):
                    j = at(bm["full_kv_indices"], b, h, i, s)
                    if (j + 1) * KVB > bm["KV_LEN"]:
                        continue
                    out[b, h, i * QB:(i + 1) * QB, j * KVB:(j + 1) * KVB] = True
    return out.astype(np.int32)
