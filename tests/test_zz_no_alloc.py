"""The allocation-free block-mask entry point (bma_mask_compile_static) against the regular one.

Some hosts of this library may not allocate device memory while they run: a custom-call handler
inside a compiled program has only the buffers its compiler planned, and a serving loop that
froze its memory pool cannot grow it.  For them the library carries its own fixed scratch array.
This test calls that entry point through the C ABI twice in a row and requires the block lists
to be bit-identical to those of bma_mask_compile (integer work, so no tolerance), and checks
that a mask too large for the fixed array is refused.  It is collected last so that a failure
here cannot hide another test's result."""
import ctypes as C

import numpy as np
import pytest
import torch

from jaxmodules_b200 import _native as nat
from jaxmodules_b200 import masks as M
from jaxmodules_b200.block_mask import compile_block_lists

pytestmark = pytest.mark.gpu

FIELDS = ["kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices",
          "q_num_blocks", "q_indices", "full_q_num_blocks", "full_q_indices"]


def _static_lists(dmask, B, H, N, L, blk, device):
    """Output buffers are allocated here, by the caller; the entry point itself allocates nothing."""
    NQ, NKV = -(-N // blk), -(-L // blk)
    LB, LH = (B if dmask.depends_b else 1), (H if dmask.depends_h else 1)
    i32 = dict(dtype=torch.int32, device=device)
    t = dict(kv_num_blocks=torch.full((LB, LH, NQ), -7, **i32), kv_indices=torch.full((LB, LH, NQ, NKV), -7, **i32),
             full_kv_num_blocks=torch.full((LB, LH, NQ), -7, **i32), full_kv_indices=torch.full((LB, LH, NQ, NKV), -7, **i32),
             q_num_blocks=torch.full((LB, LH, NKV), -7, **i32), q_indices=torch.full((LB, LH, NKV, NQ), -7, **i32),
             full_q_num_blocks=torch.full((LB, LH, NKV), -7, **i32), full_q_indices=torch.full((LB, LH, NKV, NQ), -7, **i32))
    lists = nat.BlockLists()
    lists.B, lists.H, lists.NQ, lists.NKV, lists.q_block, lists.kv_block = LB, LH, NQ, NKV, blk, blk
    lists.kv_num, lists.kv_idx = t["kv_num_blocks"].data_ptr(), t["kv_indices"].data_ptr()
    lists.full_kv_num, lists.full_kv_idx = t["full_kv_num_blocks"].data_ptr(), t["full_kv_indices"].data_ptr()
    lists.q_num, lists.q_idx = t["q_num_blocks"].data_ptr(), t["q_indices"].data_ptr()
    lists.full_q_num, lists.full_q_idx = t["full_q_num_blocks"].data_ptr(), t["full_q_indices"].data_ptr()
    return lists, t


def _segments(B, L, seed):
    rng = np.random.default_rng(seed)
    seg = np.zeros((B, L), dtype=np.int32)
    for b in range(B):
        pos, sid = 0, 0
        while pos < L:
            n = int(rng.integers(40, 300))
            seg[b, pos:pos + n] = sid
            pos += n
            sid += 1
    return seg


def _devices():
    # the array's device address is looked up once per device: cover a second GPU where the box has one
    return [0, 1] if torch.cuda.device_count() >= 2 else [0]


@pytest.mark.parametrize("index", _devices())
def test_static_scratch_matches_workspace_variant_twice(index):
    lib = nat.lib()
    dev = torch.device("cuda", index)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert lib.bma_mask_compile_static_limit() == 4 << 20
    # two different masks back to back: the second call reuses the array the first one left dirty
    cases = [
        (M.document_mask(_segments(3, 2048, seed=11), causal=True), 3, 2, 2048, 2048, 64),
        (M.and_masks(M.causal_mask(), M.sliding_window_mask(300, 1 << 20)), 2, 4, 4096, 4096, 128),
    ]
    for mask, B, H, N, L, blk in cases:
        terms = M.terms_from_mask_fn(mask, B, H, N, L)
        dmask = M.to_device_mask(terms, N, L, dev)
        _, want = compile_block_lists(dmask, B, H, N, L, blk, blk, dev, q_side=True)
        lists, got = _static_lists(dmask, B, H, N, L, blk, dev)
        nat.check(lib.bma_mask_compile_static(C.byref(dmask.spec), B, H, C.byref(lists), stream), "bma_mask_compile_static")
        torch.cuda.synchronize(dev)
        for f in FIELDS:
            assert torch.equal(got[f], want[f]), f
        # what the entry point exists for: a further call (the device address is known by now) allocates nothing --
        # neither through the caching allocator nor behind its back (free device memory as the driver reports it)
        free_before, _ = torch.cuda.mem_get_info(dev)
        stats_before = torch.cuda.memory_stats(dev)
        nat.check(lib.bma_mask_compile_static(C.byref(dmask.spec), B, H, C.byref(lists), stream), "bma_mask_compile_static")
        torch.cuda.synchronize(dev)
        stats_after = torch.cuda.memory_stats(dev)
        for k in ("allocation.all.allocated", "segment.all.allocated", "num_alloc_retries"):
            assert stats_after.get(k, 0) == stats_before.get(k, 0), k
        assert torch.cuda.mem_get_info(dev)[0] >= free_before - (1 << 20)     # a cudaMalloc would take at least 2 MiB
        for f in FIELDS:
            assert torch.equal(got[f], want[f]), f
    torch.cuda.set_device(0)


def test_static_scratch_rejects_oversized_masks():
    lib = nat.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    # 4096 x 4096 blocks of a batch-dependent mask need 3 * 16 MiB of flags: beyond the 4 MiB array
    B, H, N, blk = 3, 1, 4096 * 16, 16
    seg = torch.zeros((B, N), dtype=torch.int32)
    dmask = M.to_device_mask(M.MaskTerms(seg_q=seg, seg_k=seg), N, N, dev)
    lists = nat.BlockLists()
    lists.B, lists.H, lists.NQ, lists.NKV, lists.q_block, lists.kv_block = B, 1, N // blk, N // blk, blk, blk
    dummy = torch.zeros(16, dtype=torch.int32, device=dev)   # never written: the call is refused first
    lists.kv_num = lists.kv_idx = lists.full_kv_num = lists.full_kv_idx = dummy.data_ptr()
    need = lib.bma_mask_compile_workspace_bytes(C.byref(dmask.spec), B, H, lists.NQ, lists.NKV)
    assert need > lib.bma_mask_compile_static_limit()
    rc = lib.bma_mask_compile_static(C.byref(dmask.spec), B, H, C.byref(lists), torch.cuda.current_stream(dev).cuda_stream)
    assert rc == nat.BMA_ERR_LIMIT
    assert b"limit" in lib.bma_error_string(rc)
