"""Pins the block-mask oracle on every known-answer vector of the reference's
tests/test_block_mask.py (stored in tests/golden/block_mask_known_answers.json)."""
import numpy as np

from oracle import block_mask_oracle as bo


def test_create_block_mask_dense(golden_block_mask, named_masks):
    for name in ("create_causal_8x8_block4", "create_mod3_8x8_block4"):
        g = golden_block_mask[name]
        bm = bo.create_block_mask(named_masks[g["mask"]], g["B"], g["H"], g["Q_LEN"], g["KV_LEN"], g["BLOCK_SIZE"])
        assert (bm["B"], bm["H"], bm["Q_LEN"], bm["KV_LEN"]) == (g["B"], g["H"], g["Q_LEN"], g["KV_LEN"])
        assert bm["Q_BLOCK_SIZE"] == bm["KV_BLOCK_SIZE"] == g["BLOCK_SIZE"]
        dense = bo.materialize_mask(bm)
        expect = np.broadcast_to(np.array(g["dense_mask_bh"], dtype=np.int32), dense.shape)
        assert dense.dtype == np.int32 and np.array_equal(dense, expect)


def test_from_kv_blocks(golden_block_mask, named_masks):
    g = golden_block_mask["from_kv_blocks_banded"]
    bm = dict(B=1, H=1, Q_LEN=g["seq_lengths"][0], KV_LEN=g["seq_lengths"][1], Q_BLOCK_SIZE=2, KV_BLOCK_SIZE=2,
              kv_num_blocks=np.array(g["kv_num_blocks"]), kv_indices=np.array(g["kv_indices"]),
              full_kv_num_blocks=np.array(g["full_kv_num_blocks"]), full_kv_indices=np.array(g["full_kv_indices"]),
              mask_mod=named_masks[g["mask"]])
    assert np.array_equal(bo.materialize_mask(bm)[0, 0], np.array(g["dense_mask_bh"]))


def test_from_kv_blocks_inferred_lengths(golden_block_mask):
    g = golden_block_mask["from_kv_blocks_inferred"]
    kv_len = bo.infer_kv_len(np.array(g["kv_num_blocks"]), np.array(g["kv_indices"]),
                             np.array(g["full_kv_num_blocks"]), np.array(g["full_kv_indices"]), g["BLOCK_SIZE"])
    assert kv_len == g["expected_KV_LEN"]
    assert np.array(g["kv_indices"]).shape[2] * g["BLOCK_SIZE"] == g["expected_Q_LEN"]


def test_get_partial_block(golden_block_mask, named_masks):
    g = golden_block_mask["get_partial_block_checkerboard"]
    blk = bo.get_partial_block(named_masks[g["mask"]], 0, 0, 0, 0, g["Q_BLOCK_SIZE"], g["KV_BLOCK_SIZE"], 1, 1)
    assert np.array_equal(blk.astype(int), np.array(g["expected"]))


def test_sparse_kv_and_q(golden_block_mask):
    for name, fn in (("sparse_kv", bo.get_sparse_kv_data_from_blocks), ("sparse_q", bo.get_sparse_q_data_from_blocks)):
        g = golden_block_mask[name]
        num, idx = fn(np.array(g["blocks"]))
        rel = np.array(g["relevant"])
        assert np.array_equal(num, np.array(g["expected_num_blocks"]))
        assert np.array_equal(idx * rel, np.array(g["expected_indices"]) * rel)
        assert num.dtype == np.int32 and idx.dtype == np.int32
    # the 2-D form broadcasts to [1,1,...] (tests/test_block_mask.py:199-203)
    num2, idx2 = bo.get_sparse_kv_data_from_blocks(np.array(golden_block_mask["sparse_kv"]["blocks"])[0, 0])
    assert num2.shape == (1, 1, 2) and idx2.shape == (1, 1, 2, 2)


def test_dense_from_kv(golden_block_mask):
    g = golden_block_mask["dense_from_kv"]
    dense = bo.get_dense_from_kv_blocks(1, 1, g["NUM_Q_BLOCKS"], g["NUM_KV_BLOCKS"], np.array(g["kv_num_blocks"]),
                                        np.array(g["kv_indices"]))
    assert np.array_equal(dense.astype(int), np.array(g["expected"]))


def test_classmethods(golden_block_mask):
    for name, fn in (("classmethod_causal", bo.causal_mask), ("classmethod_full", bo.full_mask)):
        g = golden_block_mask[name]
        bm = fn(g["B"], g["H"], g["Q_LEN"], g["KV_LEN"], g["BLOCK_SIZE"])
        dense = bo.materialize_mask(bm)
        assert np.array_equal(dense, np.broadcast_to(np.array(g["dense_mask_bh"]), dense.shape))


def test_index_layout_is_stable_argsort():
    """Full-width rows: set indices ascending, then unset ascending (jnp.argsort is stable)."""
    blocks = np.array([[0, 1, 0, 1, 1, 0]])
    num, idx = bo.get_sparse_kv_data_from_blocks(blocks)
    assert num.tolist() == [[[3]]] and idx.tolist() == [[[[1, 3, 4, 0, 2, 5]]]]


def test_streaming_classification_matches_dense():
    rng = np.random.default_rng(0)
    table = rng.random((2, 3, 24, 40)) < 0.5
    table[:, :, 8:16, 8:24] = True
    table[:, :, 16:24, 0:16] = False
    fn = lambda b, h, q, k: table[b, h, q, k]
    partial, full = bo.classify_blocks(fn, 2, 3, 24, 40, (8, 8))
    blocks = table.reshape(2, 3, 3, 8, 5, 8)
    any_ = blocks.any(axis=(3, 5))
    all_ = blocks.all(axis=(3, 5))
    assert np.array_equal(partial, any_ ^ all_) and np.array_equal(full, all_)
