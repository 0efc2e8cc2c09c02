"""Host-side mirror of the reference interface: BlockMask constructors/converters against the
reference's known answers, mask factories, bit-table packing, and the argument checks of
masked_attention_via_map that fire before any CUDA work."""
import numpy as np
import math

import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200 import masks as M


def test_constructors_match_known_answers(golden_block_mask, named_masks):
    g = golden_block_mask["classmethod_causal"]
    bm = jm.BlockMask.causal_mask(g["B"], g["H"], g["Q_LEN"], g["KV_LEN"], g["BLOCK_SIZE"])
    assert (bm.B, bm.H, bm.Q_LEN, bm.KV_LEN, bm.Q_BLOCK_SIZE, bm.KV_BLOCK_SIZE) == (2, 2, 8, 8, 4, 4)
    assert torch.equal(bm.materialize_mask(), torch.tensor(g["dense_mask_bh"], dtype=torch.int32).expand(2, 2, 8, 8))
    g = golden_block_mask["classmethod_full"]
    bm = jm.BlockMask.full_mask(g["B"], g["H"], g["Q_LEN"], g["KV_LEN"], g["BLOCK_SIZE"])
    assert torch.equal(bm.materialize_mask(), torch.ones(2, 2, 8, 8, dtype=torch.int32))
    assert bm.kv_indices.shape == (2, 2, 2, 1) and bm.q_num_blocks is None


def test_from_kv_blocks(golden_block_mask, named_masks):
    g = golden_block_mask["from_kv_blocks_banded"]
    bm = jm.BlockMask.from_kv_blocks(torch.tensor(g["kv_num_blocks"]), torch.tensor(g["kv_indices"]),
                                     torch.tensor(g["full_kv_num_blocks"]), torch.tensor(g["full_kv_indices"]),
                                     BLOCK_SIZE=g["BLOCK_SIZE"], mask_mod=named_masks[g["mask"]], seq_lengths=tuple(g["seq_lengths"]))
    assert torch.equal(bm.materialize_mask()[0, 0], torch.tensor(g["dense_mask_bh"], dtype=torch.int32))
    g = golden_block_mask["from_kv_blocks_inferred"]
    bm = jm.BlockMask.from_kv_blocks(torch.tensor(g["kv_num_blocks"]), torch.tensor(g["kv_indices"]),
                                     torch.tensor(g["full_kv_num_blocks"]), torch.tensor(g["full_kv_indices"]),
                                     BLOCK_SIZE=g["BLOCK_SIZE"], mask_mod=named_masks[g["mask"]])
    assert (bm.Q_LEN, bm.KV_LEN, bm.B, bm.H) == (g["expected_Q_LEN"], g["expected_KV_LEN"], 1, 1)
    dense = bm.materialize_mask()
    assert dense.shape == (1, 1, 6, 8) and dense.min() >= 0 and dense.max() <= 1
    # rank lifting and q-side generation
    bm2 = jm.BlockMask.from_kv_blocks(torch.tensor([1, 2]), torch.tensor([[0, 0], [0, 1]]), torch.tensor([0, 0]),
                                      torch.tensor([[0, 0], [0, 0]]), BLOCK_SIZE=2, mask_mod=named_masks["parity"],
                                      seq_lengths=(4, 4), generate_q_blocks=True)
    assert bm2.q_num_blocks.tolist() == [[[2, 1]]] and bm2.kv_num_blocks.shape == (1, 1, 2)


def test_sparse_dense_converters(golden_block_mask, named_masks):
    for name, fn in (("sparse_kv", jm.get_sparse_kv_data_from_blocks), ("sparse_q", jm.get_sparse_q_data_from_blocks)):
        g = golden_block_mask[name]
        num, idx = fn(torch.tensor(g["blocks"]))
        rel = torch.tensor(g["relevant"])
        assert num.dtype == torch.int32 and idx.dtype == torch.int32
        assert num.tolist() == g["expected_num_blocks"]
        assert torch.equal(idx * rel, torch.tensor(g["expected_indices"], dtype=torch.int32) * rel)
    g = golden_block_mask["dense_from_kv"]
    dense = jm.get_dense_from_kv_blocks(1, 1, 2, 2, torch.tensor(g["kv_num_blocks"]), torch.tensor(g["kv_indices"]))
    assert dense.int().tolist() == g["expected"]
    g = golden_block_mask["get_partial_block_checkerboard"]
    blk = jm.get_partial_block(named_masks["parity"], 0, 0, 0, 0, 4, 4, 1, 1)
    assert blk.int().tolist() == g["expected"]
    assert jm.extract_block_size(4) == (4, 4) and jm.extract_block_size((2, 8)) == (2, 8)


def test_from_blocks_removes_full_from_partial():
    partial = torch.tensor([[[[1, 1], [0, 1]]]])
    full = torch.tensor([[[[0, 1], [0, 0]]]])
    bm = jm.BlockMask.from_blocks(partial, full, 4, lambda b, h, q, k: True)
    assert bm.kv_num_blocks.tolist() == [[[1, 1]]] and bm.full_kv_num_blocks.tolist() == [[[1, 0]]]
    assert bm.to_dense().int().tolist() == [[[[1, 1], [0, 1]]]]
    assert (bm.Q_LEN, bm.KV_LEN) == (8, 8)


def test_mask_factories_agree_with_plain_predicates():
    q = np.arange(12)[:, None]
    k = np.arange(12)[None, :]
    assert np.array_equal(M.causal_mask()(0, 0, q, k), q >= k)
    assert np.array_equal(M.sliding_window_mask(3, 2)(0, 0, q, k), (k >= q - 3) & (k <= q + 2))
    seg = np.array([[0, 0, 0, 1, 1, 2, 2, 2, 2, 3, 3, 3]])
    got = M.document_mask(seg, causal=True)(0, 0, q, k)
    assert np.array_equal(got, (seg[0][q] == seg[0][k]) & (k <= q))
    both = M.and_masks(M.causal_mask(), M.sliding_window_mask(4, 0))
    assert both.terms.causal and both.terms.band == (4, 0)
    assert np.array_equal(both(0, 0, q, k), (q >= k) & (k >= q - 4))
    assert M.argcount(lambda h, q, k: True) == 3 and M.argcount(both) == 4


def test_bitmap_packing():
    fn = lambda b, h, q, k: (q * 7 + k * 3 + h + b) % 5 < 2
    bm = M.bitmap_from_callable(fn, 2, 3, 5, 70, batch_dependent=True)
    assert bm.shape == (2, 3, 5, 3) and bm.dtype == torch.int32
    words = bm.numpy().view(np.uint32)
    for (b, h, q, k) in [(0, 0, 0, 0), (1, 2, 4, 69), (1, 1, 3, 31), (0, 2, 2, 32), (1, 0, 1, 64)]:
        assert ((words[b, h, q, k // 32] >> (k % 32)) & 1) == int(fn(b, h, q, k))
    assert (words[..., 2] >> 6).max() == 0  # bits past L are clear
    t = M.terms_from_mask_fn(lambda h, q, k: q >= k, 4, 2, 8, 8)
    assert t.bitmap.shape[0] == 1  # 3-argument masks are batch independent


def test_argument_errors_precede_cuda():
    Q, K, V = torch.randn(8, 2, 16), torch.randn(8, 2, 16), torch.randn(8, 2, 16)
    with pytest.raises(ValueError):
        jm.masked_attention_via_map(Q, K, V, is_causal=True, mask_fn=lambda h, q, k: True)
    with pytest.raises(AssertionError):
        jm.masked_attention_via_map(Q, torch.randn(8, 2, 32), V)
    with pytest.raises(ValueError):
        jm.masked_attention_via_map(torch.randn(8, 16), K, V)
    with pytest.raises(AssertionError):
        jm.masked_attention_via_map(Q[None], K, V)
    with pytest.raises(AssertionError):
        jm.masked_attention_via_map(torch.randn(8, 3, 16), K, V)   # Hq % Hkv != 0
    with pytest.raises(NotImplementedError):    # not an exponential of the dot product
        jm.masked_attention_via_map(Q, K, V, kernel_fn=lambda q, k: 1.0 + (q @ k) ** 2)
    with pytest.raises(NotImplementedError):    # depends on more than the dot product
        jm.masked_attention_via_map(Q, K, V, kernel_fn=lambda q, k: math.exp(float(q @ k) - float(q @ q)))
    with pytest.raises(RuntimeError):   # CPU tensors: there is no CPU path
        jm.masked_attention_via_map(Q, K, V)


def test_no_cpu_path_for_create_block_mask():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError):
        jm.create_block_mask(lambda b, h, q, k: q >= k, 1, 1, 8, 8, 4)


def test_kernel_log_affine():
    """kernel_fn family of the CUDA path: exp(a*q.k + b), found from the marker functions or by probing."""
    from jaxmodules_b200.attention import kernel_log_affine
    d = 16
    assert kernel_log_affine(jm.default_kernel, d) == (0.25, 0.0)
    a, b = kernel_log_affine(jm.threshold_kernel(2.0), d)
    assert a == 1.0 and b == pytest.approx(-0.5)
    assert kernel_log_affine(jm.threshold_kernel(None), d) == (1.0, 0.0)
    # the custom kernel of the reference's tests/test_mapped_attention.py:1135-1136, in NumPy and in torch
    a, b = kernel_log_affine(lambda q, k: np.exp(np.dot(q, k) / (2 * np.sqrt(k.shape[-1]))), d)
    assert a == pytest.approx(0.125, abs=1e-9) and b == pytest.approx(0.0, abs=1e-9)
    a, b = kernel_log_affine(lambda q, k: torch.exp(torch.dot(q, k) * 0.3 - 1.5), d)
    assert a == pytest.approx(0.3, abs=1e-9) and b == pytest.approx(-1.5, abs=1e-9)
    # the marker functions evaluate like the reference's kernels
    q, k = torch.arange(4.0) / 4, torch.ones(4)
    assert float(jm.default_kernel(q, k)) == pytest.approx(math.exp(1.5 / 2))
    assert float(jm.threshold_kernel(1.0)(q, k)) == pytest.approx(math.exp(1.5 - 0.5))


def test_ring_wait_turns_transport_errors_into_ring_transfer_error():
    """Host-side failure handling of the ring, without any process group: a request whose wait raises (a time-out, a
    peer that went away) must surface as RingTransferError naming the step; a healthy one passes through."""
    from jaxmodules_b200 import sharding as S

    class Req:
        def __init__(self, fail):
            self.fail, self.timeouts = fail, []

        def wait(self, timeout=None):
            self.timeouts.append(timeout)
            if self.fail:
                raise RuntimeError("Timed out waiting 3000ms for recv operation to complete")

    ok = Req(False)
    S._wait_all([ok], 3.0, "step 0")
    assert ok.timeouts[0].total_seconds() == 3.0
    S._wait_all([Req(False)], None, "step 0")          # no deadline: plain wait()
    with pytest.raises(S.RingTransferError, match="step 5.*Timed out"):
        S._wait_all([Req(False), Req(True)], 1.0, "rank 0: K/V rotation, ring step 5")


def test_mask_caches_and_scratch_knobs():
    """Host-side state: the per-callable table cache is keyed by function object and shape, device copies of a mask's
    arrays are made once per (tensor, device, version), and lowering the scratch limit drops larger buffers."""
    import torch
    from jaxmodules_b200 import attention as A
    from jaxmodules_b200 import masks as M
    M.clear_mask_cache()
    fn = lambda b, h, q, k: (q + k) % 2 == 0
    t1 = M.terms_from_mask_fn(fn, 1, 1, 8, 8)
    assert M.terms_from_mask_fn(fn, 1, 1, 8, 8) is t1                       # same function object, same shape: cached
    assert M.terms_from_mask_fn(fn, 1, 1, 8, 16) is not t1                  # another shape
    assert M.terms_from_mask_fn(lambda b, h, q, k: (q + k) % 2 == 0, 1, 1, 8, 8) is not t1   # another object
    M.clear_mask_cache()
    assert M.terms_from_mask_fn(fn, 1, 1, 8, 8) is not t1
    seg = torch.zeros((2, 16), dtype=torch.int64)
    a = M._on_device(seg, "cpu", torch.int32)
    assert a.dtype == torch.int32 and M._on_device(seg, "cpu", torch.int32) is a
    seg[0, 0] = 1                                                           # an in-place write bumps the version
    b = M._on_device(seg, "cpu", torch.int32)
    assert b is not a and int(b[0, 0]) == 1
    same = torch.zeros((2, 16), dtype=torch.int32)
    assert M._on_device(same, "cpu", torch.int32) is same                   # already in place: no copy
    limit, frac = A._scratch_limit, A._scratch_fraction
    try:
        A._scratch_buffers[("test", 0)] = torch.empty(1024, dtype=torch.uint8)
        A.set_backward_scratch_limit(512)
        assert ("test", 0) not in A._scratch_buffers and A._scratch_limit == 512
        A._scratch_buffers[("test", 1)] = torch.empty(16, dtype=torch.uint8)
        A.release_backward_scratch()
        assert not A._scratch_buffers
    finally:
        A.set_backward_scratch_limit(limit, frac)


def test_ring_step_calls_join_untouched_segment_pairs():
    """Zig-zag layout under a causal mask: the first ring step is two diagonal calls plus one unmasked call, every later
    step ONE unmasked call over two segments; the joined calls cover exactly the pairs the mask does not empty."""
    from jaxmodules_b200 import sharding as S
    world, n = 4, 64
    layout = S.zigzag_layout(n)
    for terms in (M.MaskTerms(causal=True), M.MaskTerms(band=(40, 8)), M.MaskTerms(causal=True, band=(70, 1 << 20))):
        for rank in range(world):
            q_segs = S._segments(layout, rank, world)
            for s, owner in enumerate(S.ring_schedule(rank, world)):
                k_segs = S._segments(layout, owner, world)
                calls = S._step_calls(terms, q_segs, k_segs)
                if terms.causal and terms.band is None:
                    assert len(calls) == (3 if s == 0 else 1)
                    assert all(not c[4].causal for c in calls) == (s > 0)
                covered = set()
                for ql, qn, kl, kn, t in calls:
                    for sl, sg, sn in q_segs:
                        for tl, tg, tn in k_segs:
                            if ql <= sl < ql + qn and kl <= tl < kl + kn:
                                assert (sl, tl) not in covered
                                covered.add((sl, tl))
                                if not (t.causal or t.band):     # an unmasked call: the mask must leave the pair whole
                                    assert S._pair_is_full(terms, sg, sn, tg, tn)
                                else:                            # a masked call is one pair with its global offsets
                                    assert (qn, kn) == (sn, tn) and (t.q_offset, t.k_offset) == (sg, tg)
                want = {(sl, tl) for sl, sg, sn in q_segs for tl, tg, tn in k_segs if not S._pair_is_empty(terms, sg, sn, tg, tn)}
                assert covered == want
    # masks with table or segment terms are never joined into unmasked calls
    seg = torch.zeros((1, 4 * n), dtype=torch.int32)
    t = M.MaskTerms(causal=True, seg_q=seg, seg_k=seg)
    assert not S._pair_is_full(t, 128, 32, 0, 32)
