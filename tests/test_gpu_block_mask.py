"""Parity of the CUDA mask-compile kernels (through the C ABI) with the oracle restatement of
create_block_mask — bit exact on every array the reference's BlockMask holds."""
import numpy as np
import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200 import masks as M
from oracle import block_mask_oracle as bo

pytestmark = pytest.mark.gpu

FIELDS = ["kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices",
          "q_num_blocks", "q_indices", "full_q_num_blocks", "full_q_indices"]


def assert_same(bm: jm.BlockMask, ref: dict):
    for k in ("B", "H", "Q_LEN", "KV_LEN", "Q_BLOCK_SIZE", "KV_BLOCK_SIZE"):
        assert getattr(bm, k) == ref[k], k
    for f in FIELDS:
        got = getattr(bm, f).cpu().numpy()
        assert got.dtype == np.int32 and got.shape == ref[f].shape, f
        assert np.array_equal(got, ref[f]), f


def test_known_answers(golden_block_mask, named_masks):
    for name in ("create_causal_8x8_block4", "create_mod3_8x8_block4"):
        g = golden_block_mask[name]
        bm = jm.create_block_mask(named_masks[g["mask"]], g["B"], g["H"], g["Q_LEN"], g["KV_LEN"], g["BLOCK_SIZE"])
        dense = bm.materialize_mask()
        assert torch.equal(dense, torch.tensor(g["dense_mask_bh"], dtype=torch.int32).expand_as(dense))
        assert_same(bm, bo.create_block_mask(named_masks[g["mask"]], g["B"], g["H"], g["Q_LEN"], g["KV_LEN"], g["BLOCK_SIZE"]))


CASES = [
    ("causal", lambda: M.causal_mask(), 2, 3, 96, 96, 16),
    ("causal_rect", lambda: M.causal_mask(), 1, 2, 64, 160, (16, 32)),
    ("full", lambda: M.full_mask(), 2, 2, 64, 64, 32),
    ("sliding", lambda: M.sliding_window_mask(20, 7), 1, 2, 128, 128, 16),
    ("sliding_sym", lambda: M.sliding_window_mask(256, 256), 1, 1, 2048, 2048, 128),
    ("causal_band", lambda: M.and_masks(M.causal_mask(), M.sliding_window_mask(33, 1000)), 1, 2, 256, 256, 32),
    ("floor_lengths", lambda: M.causal_mask(), 1, 1, 70, 90, 16),
]


@pytest.mark.parametrize("name,make,B,H,QL,KL,BS", CASES, ids=[c[0] for c in CASES])
def test_structured_masks(name, make, B, H, QL, KL, BS):
    m = make()
    assert_same(jm.create_block_mask(m, B, H, QL, KL, BS), bo.create_block_mask(m, B, H, QL, KL, BS))


def _segments(B, L, lo, hi, seed):
    rng = np.random.default_rng(seed)
    seg = np.zeros((B, L), dtype=np.int32)
    for b in range(B):
        pos, sid = 0, 0
        while pos < L:
            n = int(rng.integers(lo, hi + 1))
            seg[b, pos:pos + n] = sid
            pos += n
            sid += 1
    return seg


@pytest.mark.parametrize("causal", [False, True])
def test_document_masks(causal):
    B, H, L, BS = 3, 2, 512, 32
    seg = _segments(B, L, 20, 130, seed=4)
    m = M.document_mask(seg, causal=causal)
    assert_same(jm.create_block_mask(m, B, H, L, L, BS), bo.create_block_mask(m, B, H, L, L, BS))
    # unsorted ids exercise the element scan behind the min/max summaries
    seg2 = np.random.default_rng(5).integers(0, 3, size=(B, L)).astype(np.int32)
    seg2[:, 64:160] = 1
    m2 = M.document_mask(seg2, causal=causal)
    assert_same(jm.create_block_mask(m2, B, H, L, L, BS), bo.create_block_mask(m2, B, H, L, L, BS))


def test_arbitrary_callables_via_bit_table():
    rng = np.random.default_rng(7)
    table = rng.random((2, 3, 96, 160)) < 0.5
    table[:, :, 32:64, 64:128] = True
    table[:, :, 64:96, 0:96] = False
    fn = lambda b, h, q, k: table[b, h, q, k]
    assert_same(jm.create_block_mask(fn, 2, 3, 96, 160, 32), bo.create_block_mask(fn, 2, 3, 96, 160, 32))
    head = lambda b, h, q, k: np.where(h % 2 == 0, q >= k, (q + k) % 2 == 0)
    assert_same(jm.create_block_mask(head, 1, 4, 64, 64, 8), bo.create_block_mask(head, 1, 4, 64, 64, 8))


def test_config_shapes_row_replication():
    """Block geometry of the dense-causal and sliding-window benchmark shapes (per (b,h) rows are
    identical, so the oracle is evaluated for one (b,h) and broadcast)."""
    for m, B, H, L in ((M.causal_mask(), 8, 32, 4096), (M.sliding_window_mask(256, 256), 4, 16, 8192)):
        bm = jm.create_block_mask(m, B, H, L, L, 128)
        ref = bo.create_block_mask(m, 1, 1, L, L, 128)
        for f in FIELDS:
            got = getattr(bm, f).cpu().numpy()
            assert np.array_equal(got, np.broadcast_to(ref[f], got.shape)), f


def test_properties_at_long_context():
    """L = 131072, block 128 (1024 x 1024 blocks): counts and index rows of the causal mask follow
    closed forms; a checksum of every row is compared instead of an oracle run."""
    L, BS = 131072, 128
    bm = jm.create_block_mask(M.causal_mask(), 1, 2, L, L, BS)
    n = L // BS
    ar = torch.arange(n, device="cuda", dtype=torch.int32)
    assert torch.equal(bm.kv_num_blocks[0, 0], torch.ones_like(ar))
    assert torch.equal(bm.full_kv_num_blocks[0, 1], ar)
    assert torch.equal(bm.full_q_num_blocks[0, 0], n - 1 - ar)
    assert torch.equal(bm.kv_indices[0, 0, :, 0], ar)                                # the diagonal block
    assert torch.equal(bm.full_kv_indices.sum(-1)[0, 0].long(), torch.full((n,), n * (n - 1) // 2, device="cuda"))  # a permutation
    rows = bm.full_kv_indices[0, 1]
    assert torch.equal(rows[n - 1, : n - 1], ar[: n - 1]) and int(rows[n - 1, n - 1]) == n - 1
    assert torch.equal(bm.full_q_indices[0, 0, 0, : n - 1], ar[1:])


def test_conservative_lists_cover_the_exact_ones():
    """BMA_MASK_COMPILE_CONSERVATIVE (used for the lists the attention kernels walk): full blocks are
    exact, every exactly-partial block is listed, and the only extra entries are undecided segment blocks."""
    from jaxmodules_b200.block_mask import compile_block_lists, get_dense_from_kv_blocks
    rng = np.random.default_rng(0)
    B, H, L, blk = 2, 1, 2048, 128
    seg = np.sort(rng.integers(0, 9, size=(B, L)), axis=1).astype(np.int32)
    for causal in (False, True):
        terms = M.document_mask(seg, causal=causal).terms
        dmask = M.to_device_mask(terms, L, L, "cuda")
        dense = {}
        for mode in (False, True):
            _, t = compile_block_lists(dmask, B, H, L, L, blk, blk, "cuda", q_side=False, conservative=mode)
            n = L // blk
            dense[mode] = (get_dense_from_kv_blocks(t["kv_num_blocks"].shape[0], 1, n, n, t["full_kv_num_blocks"], t["full_kv_indices"]),
                           get_dense_from_kv_blocks(t["kv_num_blocks"].shape[0], 1, n, n, t["kv_num_blocks"], t["kv_indices"]))
        (full_e, part_e), (full_c, part_c) = dense[False], dense[True]
        assert torch.equal(full_e, full_c)
        assert bool((part_c | ~part_e).all())            # exact partial blocks are a subset
        extra = part_c & ~part_e
        assert int(extra.sum()) < int(part_e.sum())      # and only a few undecided blocks are added
