"""Mask programs: tracing a Python mask_fn into three-address code, the host twin of the device
interpreter, and (on a GPU) the bit table built by bma_mask_table_build — bit exact against the
function evaluated over the index grid, for the mask_fns of the reference's tests."""
import ctypes as C

import numpy as np
import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200 import _native as nat
from jaxmodules_b200 import mask_program as P
from jaxmodules_b200 import masks as M


# tests/test_mapped_attention.py:1261-1264, 1291-1299 and tests/test_attention.py:77-91 of the reference
def batch_sliding_window(b, h, q, k):
    return abs(q - k) <= b + 1


def complex_batch(b, h, q, k):
    window_ok = abs(q - k) <= ((b % 2) * 2) + ((h % 2) + 1)
    return P.where(((b % 2) == 1) & ((h % 2) == 0), window_ok & (((q + k) % 2) == 0), window_ok)


def causal(b, h, q, k):
    return q >= k


def alternating(b, h, q, k):
    return (q + k) % 2 == 0


def batch_head_sliding(b, h, q, k):
    return (q >= k) & (q - k <= b + h)


def arithmetic_zoo(b, h, q, k):
    return ~(((q - k) // 3 + (k % 5) * 2 - (q >> 1) ^ (k << 2)) % 7 < 3) | (P.minimum(q, 9) == P.maximum(k - 4, 0)) | (-q + k == 1)


SEG = np.array([[0] * 5 + [1] * 20 + [2] * 15, [0] * 17 + [1] * 23])
SEG_TABLE = P.Table(SEG)


def documents(b, h, q, k):
    return (SEG_TABLE[b, q] == SEG_TABLE[b, k]) & (k <= q)


FOUR_ARG = [batch_sliding_window, complex_batch, causal, alternating, batch_head_sliding, arithmetic_zoo, documents]


def grid(fn, B, H, N, L, nargs=4):
    b, h, q, k = np.ix_(np.arange(B), np.arange(H), np.arange(N), np.arange(L))
    out = fn(b, h, q, k) if nargs == 4 else fn(h, q, k)
    return np.broadcast_to(out, (B, H, N, L)).astype(bool)


@pytest.mark.parametrize("fn", FOUR_ARG, ids=lambda f: f.__name__)
def test_trace_matches_function(fn):
    B, H, N, L = 2, 3, 40, 37
    prog = P.trace(fn)
    b, h, q, k = np.ix_(np.arange(B), np.arange(H), np.arange(N), np.arange(L))
    assert np.array_equal(P.run_on_host(prog, b, h, q, k), grid(fn, B, H, N, L))
    assert prog.uses_b == (fn not in (causal, alternating, arithmetic_zoo))
    assert prog.uses_h == (fn in (complex_batch, batch_head_sliding))


def test_three_argument_masks_and_constants():
    prog = P.trace(lambda h, q, k: (k <= q) & (h < 2), nargs=3)
    b, h, q, k = np.ix_(np.arange(1), np.arange(4), np.arange(8), np.arange(8))
    assert np.array_equal(P.run_on_host(prog, b, h, q, k), grid(lambda h, q, k: (k <= q) & (h < 2), 1, 4, 8, 8, nargs=3))
    assert P.run_on_host(P.trace(lambda b, h, q, k: True), 0, 0, 1, 2) and not P.run_on_host(P.trace(lambda b, h, q, k: False), 0, 0, 1, 2)
    assert P.run_on_host(P.trace(lambda b, h, q, k: q), 0, 0, 1, 2) and not P.run_on_host(P.trace(lambda b, h, q, k: b), 0, 0, 1, 2)


def test_untraceable_functions_are_refused():
    for fn in (lambda b, h, q, k: (q >= k) if q > 3 else True,          # branches on a traced value
               lambda b, h, q, k: np.abs(q - k) < 3,                     # NumPy function
               lambda b, h, q, k: q / 2 > k,                             # float arithmetic
               lambda b, h, q, k: [0, 1, 0][q % 3] == 1,                 # container indexing
               lambda b, h, q, k: q >= k and k >= 0):                    # boolean operator
        with pytest.raises(P.TraceError):
            P.trace(fn)
    def long_chain(b, h, q, k):
        x = q
        for i in range(nat.PROGRAM_MAX_INSTR):
            x = x + k
        return x > 0
    with pytest.raises(P.TraceError):
        P.trace(long_chain)


def test_python_division_semantics_on_host_twin():
    prog = P.trace(lambda b, h, q, k: ((q - 7) // 3 == -2) | ((q - 7) % 3 == 2) | (q // (k - k) == 0))
    q = np.arange(12)
    want = (((q - 7) // 3) == -2) | (((q - 7) % 3) == 2) | True     # division by zero yields 0 in a program
    assert np.array_equal(P.run_on_host(prog, 0, 0, q, 5), want)


def test_table_build_rejects_bad_programs_before_any_launch():
    lib = nat.lib()
    c = nat.MaskProgram()
    call = lambda: lib.bma_mask_table_build(C.byref(c), 1, 1, 8, 8, 0, 0, C.c_void_p(16), None)
    c.n_instr = 0
    assert call() == nat.BMA_ERR_ARG
    c.n_instr = 1
    c.code[0:4] = [nat.OP["ADD"], 2, 4, 0]         # reads value 4, which this instruction itself defines
    assert call() == nat.BMA_ERR_ARG
    c.code[0:4] = [99, 0, 0, 0]
    assert call() == nat.BMA_ERR_ARG
    c.code[0:4] = [nat.OP["LOAD1"], 0, 2, 0]       # no table 0
    assert call() == nat.BMA_ERR_ARG
    c.n_instr = nat.PROGRAM_MAX_INSTR + 1
    assert call() == nat.BMA_ERR_ARG


@pytest.mark.gpu
@pytest.mark.parametrize("fn", FOUR_ARG, ids=lambda f: f.__name__)
def test_device_table_is_bit_exact(fn):
    B, H, N, L = 2, 3, 40, 37        # L not a multiple of 32: padding bits must be zero
    prog = P.trace(fn)
    bits = P.build_table(prog, B, H, N, L, "cuda")
    Bm, Hm = (B if prog.uses_b else 1), (H if prog.uses_h else 1)
    assert bits.shape == (Bm, Hm, N, 2) and bits.dtype == torch.int32
    want = M.bitmap_from_callable(fn, Bm, Hm, N, L, batch_dependent=True)
    assert torch.equal(bits.cpu(), want)
    # a shifted box (sequence shards): offsets are added before the program runs
    shifted = P.build_table(prog, B, H, 8, 24, "cuda", q_offset=16, k_offset=8).cpu()
    full = torch.from_numpy(grid(fn, Bm, Hm, N, L)[:, :, 16:24, 8:32].copy())
    unpacked = torch.from_numpy(np.unpackbits(shifted.numpy().view(np.uint8), axis=-1, bitorder="little")[..., :24].astype(bool))
    assert torch.equal(unpacked, full)


@pytest.mark.gpu
def test_traced_masks_drive_block_mask_and_attention():
    from oracle import attention_oracle as ao
    from oracle import block_mask_oracle as bo
    B, H, N, d = 4, 4, 64, 16
    bm = jm.create_block_mask(complex_batch, B, H, N, N, 16)
    ref = bo.create_block_mask(complex_batch, B, H, N, N, 16)
    for f in ("kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices", "q_num_blocks", "q_indices"):
        assert np.array_equal(getattr(bm, f).cpu().numpy(), ref[f]), f
    g = torch.Generator().manual_seed(0)
    Q, K, V = (torch.randn(B, N, H, d, generator=g) for _ in range(3))
    for fn in (batch_sliding_window, complex_batch):
        out = jm.masked_attention_via_map(Q.cuda(), K.cuda(), V.cuda(), mask_fn=fn)
        want = ao.masked_attention_dense(Q.numpy(), K.numpy(), V.numpy(), mask_fn=fn)["O"]
        assert np.abs(out.cpu().numpy() - want).max() < 1e-4


def _tiles_to_dense(cls, slot, bits, N, L):
    """Expands the tile form back into a dense bool array [Bm, Hm, N, L] on the host."""
    cls, slot, bits = cls.cpu().numpy(), slot.cpu().numpy(), bits.cpu().numpy().view(np.uint32)
    Bm, Hm, TQ, TK = cls.shape
    out = np.zeros((Bm, Hm, TQ * 128, TK * 128), dtype=bool)
    for b, h, tq, tk in np.ndindex(Bm, Hm, TQ, TK):
        c = cls[b, h, tq, tk]
        if c == 2:
            out[b, h, tq * 128:(tq + 1) * 128, tk * 128:(tk + 1) * 128] = True
        elif c == 1:
            words = bits[slot[b, h, tq, tk]]                       # [2, 128, 4]: by query row, by key row
            tile = np.unpackbits(words[0].view(np.uint8).reshape(128, 16), axis=-1, bitorder="little").astype(bool)
            by_key = np.unpackbits(words[1].view(np.uint8).reshape(128, 16), axis=-1, bitorder="little").astype(bool)
            assert np.array_equal(by_key, tile.T)                 # the transposed copy the kv-major kernel reads
            out[b, h, tq * 128:(tq + 1) * 128, tk * 128:(tk + 1) * 128] = tile
    return out[:, :, :N, :L]


@pytest.mark.gpu
@pytest.mark.parametrize("fn", [batch_sliding_window, complex_batch, causal, alternating, documents], ids=lambda f: f.__name__)
def test_device_tiles_are_bit_exact(fn):
    """The TILES form of a traced mask: classes and bits equal the function over the index grid; whole and empty tiles
    carry no bits; ragged edges are class 2 when every VALID pair is allowed."""
    B, H, N, L = 2, 3, 300, 40 if fn is documents else 421
    if fn is documents:
        N = 40
    prog = P.trace(fn)
    cls, slot, bits = P.build_tiles(prog, B, H, N, L, "cuda")
    Bm, Hm = (B if prog.uses_b else 1), (H if prog.uses_h else 1)
    want = grid(fn, Bm, Hm, N, L)
    got = _tiles_to_dense(cls, slot, bits, N, L)
    # a class-2 tile at a ragged edge claims "allowed" outside the box too: compare inside the box only
    assert np.array_equal(got, want)
    cut = int((cls == 1).sum())
    assert bits.shape[0] == max(cut, 1) and sorted(slot[cls == 1].cpu().tolist()) == list(range(cut))
    if fn is causal:                     # 3 x 4 tiles: the diagonal ones are cut, above it empty, below it whole
        c = cls[0, 0].cpu().numpy()
        assert (c == np.array([[1, 0, 0, 0], [2, 1, 0, 0], [2, 2, 1, 0]])).all()


@pytest.mark.gpu
def test_traced_mask_takes_the_tile_form_and_matches_the_table(monkeypatch):
    """The same traced, batch- and head-dependent mask through the dense bit table and through the tile form: identical
    block lists (exact and conservative), identical attention results on both backends, bf16 gradients included."""
    from oracle import attention_oracle as ao
    fn = lambda b, h, q, k: (abs(q - k) <= 40 * (b + 1) + 17 * h) & ((q + k) % (h + 2) != 0)
    B, H, N, d = 2, 2, 640, 128
    assert M.terms_from_mask_fn(fn, B, H, N, N, device="cuda").bitmap is not None
    table_bm = jm.create_block_mask(fn, B, H, N, N, 64)
    M.clear_mask_cache()
    monkeypatch.setattr(M, "TILES_ABOVE_BITS", 0)
    terms = M.terms_from_mask_fn(fn, B, H, N, N, device="cuda")
    assert terms.tiles is not None and terms.bitmap is None
    tiles_bm = jm.create_block_mask(fn, B, H, N, N, 64)          # 64-blocks: two per tile edge, scanned from the tile bits
    for f in ("kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices", "q_num_blocks", "q_indices", "full_q_indices"):
        assert torch.equal(getattr(tiles_bm, f), getattr(table_bm, f)), f
    g = torch.Generator().manual_seed(0)
    Q, K, V = (torch.randn(B, N, H, d, generator=g).to(torch.bfloat16) for _ in range(3))
    dO = torch.randn(B, N, H, d, generator=g)
    ref = ao.masked_attention_dense(Q.float().numpy(), K.float().numpy(), V.float().numpy(), mask_fn=fn, dO=dO.numpy())
    for backend in (nat.BMA_BACKEND_AUTO, nat.BMA_BACKEND_SIMT):
        q, k, v = (t.cuda().requires_grad_(True) for t in (Q, K, V))
        out = jm.masked_attention_via_map(q, k, v, mask_fn=fn, backend=backend)
        out.backward(dO.cuda())
        for name, got in (("O", out), ("dQ", q.grad), ("dK", k.grad), ("dV", v.grad)):
            err = np.abs(got.detach().float().cpu().numpy() - ref[name])
            assert (err / np.maximum(1.0, np.abs(ref[name]))).max() <= 2e-2 and err.mean() <= 2e-3, (backend, name, err.max())
    M.clear_mask_cache()


@pytest.mark.gpu
def test_batch_head_dependent_mask_at_16k_without_a_table():
    """L = 16384 with a mask that depends on batch and head (tests/test_mapped_attention.py:1249-1307 at scale): the
    dense table would be 2 x 2 x 16384^2 bits = 128 MiB; the tile form stores the ~130 cut tiles per (b, h) (1 MB in all).
    Checked on sampled query rows against a dense float32 computation over all keys."""
    B, H, L, d = 2, 2, 16384, 128
    fn = lambda b, h, q, k: (k <= q) & (q - k <= 1000 * (b + 1) + 300 * h)
    M.clear_mask_cache()
    terms = M.terms_from_mask_fn(fn, B, H, L, L, device="cuda")
    assert terms.tiles is not None and terms.tiles[2].numel() * 4 < 8 << 20
    g = torch.Generator(device="cuda").manual_seed(2)
    Q, K, V = (torch.randn(B, L, H, d, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    O = jm.masked_attention_via_map(Q, K, V, mask_fn=fn)
    rows = torch.tensor([0, 1, 127, 128, 1500, 5000, 9999, 16383], device="cuda")
    ki = torch.arange(L, device="cuda")[None, :]
    for b in range(B):
        for h in range(H):
            s = (Q[b, rows, h].float() @ K[b, :, h].float().T) / d ** 0.5
            allowed = (ki <= rows[:, None]) & (rows[:, None] - ki <= 1000 * (b + 1) + 300 * h)
            p = torch.softmax(s.masked_fill(~allowed, float("-inf")), dim=-1)
            assert float((O[b, rows, h] - p @ V[b, :, h].float()).abs().max()) <= 2e-2
    M.clear_mask_cache()
