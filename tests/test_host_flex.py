"""Host-side logic of flex_attention: argument checks in the reference's order, the element
mask a BlockMask implies (bit table route), list fitting and route selection.  No GPU."""
import numpy as np
import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200 import masks as M
from jaxmodules_b200.flex import _ReadyLists, _effective_table, flex_attention, flex_route


def unpack(table, L):
    bits = np.unpackbits(table.numpy().view(np.uint8), axis=-1, bitorder="little")
    return torch.from_numpy(bits[..., :L].astype(bool))


def banded(b, h, q, k):
    return (q >= k) & (q - k <= b + 2 * h)


def block_mask_on_cpu(mask_fn, B, H, L, S, block):
    q = torch.arange(L)[:, None]
    k = torch.arange(S)[None, :]
    dense = torch.stack([torch.stack([torch.broadcast_to(torch.as_tensor(mask_fn(b, h, q, k)), (L, S)) for h in range(H)])
                         for b in range(B)])
    blocks = dense.reshape(B, H, L // block, block, S // block, block)
    full = blocks.all(dim=5).all(dim=3)
    part = blocks.any(dim=5).any(dim=3) & ~full
    return jm.BlockMask.from_blocks(part, full, block, mask_fn), dense


def test_argument_checks_come_first():
    q = torch.zeros(2, 4, 8, 16)
    with pytest.raises(NotImplementedError):
        flex_attention(q, q, q, return_lse=True)
    with pytest.raises(NotImplementedError):
        flex_attention(q, q, q, score_mod=lambda s, b, h, qi, ki: s * s)
    with pytest.raises(AssertionError, match="same sequence length"):
        flex_attention(q, q, q[:, :, :7])
    with pytest.raises(AssertionError, match="enable_gqa"):
        flex_attention(q, q[:, :2], q[:, :2])
    bm, _ = block_mask_on_cpu(banded, 2, 4, 8, 8, 4)
    with pytest.raises(AssertionError, match="query length must match"):
        flex_attention(torch.zeros(2, 4, 12, 16), q, q, block_mask=bm)
    with pytest.raises(RuntimeError, match="CUDA"):
        flex_attention(q, q, q)


def test_effective_table_is_the_mask_for_consistent_lists():
    bm, dense = block_mask_on_cpu(banded, 2, 4, 8, 8, 4)
    assert torch.equal(unpack(_effective_table(bm, 1, 4), 8), dense)
    # head broadcast: H == 1 lists, mask evaluated with head 0
    bm1, dense1 = block_mask_on_cpu(banded, 2, 1, 8, 8, 4)
    t = _effective_table(bm1, 1, 4)
    assert t.shape[:2] == (2, 1) and torch.equal(unpack(t, 8), dense1)


def test_effective_table_follows_the_lists_and_the_kv_head():
    bm, dense = block_mask_on_cpu(banded, 1, 4, 8, 8, 4)
    full, part = bm.get_full_blocks().clone(), bm.get_partial_blocks().clone()
    part[0, 2, 1, 0] = False                       # a block the mask allows but the lists omit
    full[0, 3, 0, 1] = True                        # a block the mask forbids, listed as full
    cut = jm.BlockMask.from_blocks(part, full, 4, banded)
    got = unpack(_effective_table(cut, 2, 4), 8)   # group size 2: query heads 2, 3 -> kv head 1
    want = torch.zeros_like(dense)
    for hq in range(4):
        q, k = torch.arange(8)[:, None], torch.arange(8)[None, :]
        want[0, hq] = banded(0, hq // 2, q, k)
    want[0, 2, 4:, :4] = False
    # partial blocks of head hq keep only what mask_mod(kv head) allows inside listed blocks
    blocks = (full | part)[0].repeat_interleave(4, dim=1).repeat_interleave(4, dim=2)
    want[0] &= blocks
    want[0, 3, :4, 4:] = True
    assert torch.equal(got, want)


def test_scalar_only_mask_mod():
    def scalar_only(b, h, q, k):
        if not isinstance(q, int):
            raise TypeError("ints only")
        return q >= k
    bm, dense = block_mask_on_cpu(lambda b, h, q, k: q >= k, 1, 1, 8, 8, 4)
    bm.mask_mod = scalar_only
    assert torch.equal(unpack(_effective_table(bm, 1, 1), 8), dense)


def test_ready_lists_fit_pads_and_clamps():
    bm = jm.BlockMask.full_mask(1, 1, 16, 16, 4)
    ready = _ReadyLists(bm, "cpu")
    num, idx = ready._fit(bm.kv_num_blocks, bm.kv_indices, 4)      # width-1 list of the reference
    assert idx.shape == (1, 1, 4, 4) and idx.dtype == torch.int32 and int(num.max()) == 0
    num, idx = ready._fit(torch.tensor([[[9, 2]]]), torch.tensor([[[[7, -3, 1], [0, 1, 2]]]]), 4)
    assert num.tolist() == [[[3, 2]]] and idx[0, 0, 0].tolist() == [3, 0, 1, 0]
    assert ready(8, 8, False) is None                              # other tile size: not usable


def test_route_without_structure_is_table():
    bm, _ = block_mask_on_cpu(banded, 1, 1, 8, 8, 4)
    assert flex_route(bm, 1, 1, [(4, 4)], "cpu") == "table"
    assert flex_route(None, 1, 1, [(64, 64)], "cpu") == "terms"
    bm = jm.BlockMask.causal_mask(1, 1, 256, 256, 128)
    assert flex_route(bm, 1, 1, [(128, 128), (128, 128)], "cpu") == "lists"
    seg = M.document_mask(np.zeros((2, 256), dtype=np.int32))
    bm.mask_mod = seg
    assert flex_route(bm, 2, 1, [(128, 128)], "cpu") == "table"    # batch-broadcast lists, per-batch mask


def test_score_mod_affine_family():
    """score_mod = a * score + w[h] * k + (constant along k) is recognised by probing; the rest is refused."""
    from jaxmodules_b200.flex import score_mod_affine
    a, w = score_mod_affine(lambda s, b, h, q, k: s + 0.1 * (q - k), 2, 4, 8, 8)       # tests/test_attention.py:131-132
    assert a == pytest.approx(1.0) and np.allclose(w, -0.1)
    slopes = np.array([0.5, 0.25, 0.125, 0.0625])
    a, w = score_mod_affine(lambda s, b, h, q, k: 2 * s + slopes[h] * (k - q) + b, 2, 4, 64, 64)   # ALiBi with a batch offset
    assert a == pytest.approx(2.0) and np.allclose(w, slopes)
    for bad in (lambda s, b, h, q, k: s * s, lambda s, b, h, q, k: s + 0.01 * k * k,
                lambda s, b, h, q, k: s + 0.1 * b * k, lambda s, b, h, q, k: s + 0.01 * q * k,
                lambda s, b, h, q, k: np.tanh(s)):
        with pytest.raises(NotImplementedError):
            score_mod_affine(bad, 2, 2, 16, 16)


def test_ready_lists_consistency_check():
    """The backward may hand dS tiles from the kv-major to the query-major kernel only when both list
    sides name the same blocks; user-made q-side arrays are compared with the kv side once."""
    bm = jm.BlockMask.causal_mask(1, 1, 512, 512, 128)
    assert _ReadyLists(bm, "cpu").consistent
    tampered = jm.BlockMask.causal_mask(1, 1, 512, 512, 128)
    tampered.q_num_blocks = tampered.q_num_blocks.clone()
    tampered.q_num_blocks[0, 0, 1] = 0                         # a partial block the kv side still lists
    assert not _ReadyLists(tampered, "cpu").consistent
    kv_only = jm.BlockMask.from_kv_blocks(bm.kv_num_blocks, bm.kv_indices, bm.full_kv_num_blocks, bm.full_kv_indices,
                                          BLOCK_SIZE=128, mask_mod=bm.mask_mod, seq_lengths=(512, 512))
    assert _ReadyLists(kv_only, "cpu").consistent              # q side derived from the kv side
