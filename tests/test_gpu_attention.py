"""Parity of the CUDA attention path (package -> ctypes -> C ABI -> kernels) with the float64
dense oracle, on the reference's test shapes, the benchmark configurations (reduced where the
oracle would take minutes) and size-independent properties at full size.

Tolerances against the oracle on O, dQ, dK and dV: float32 I/O max-abs 1e-4, mean-abs 1e-5;
bfloat16 I/O max-abs 2e-2, mean-abs 2e-3.  Per tensor:

* O is float32 for every input dtype, so its bound is ABSOLUTE everywhere.
* dQ, dK, dV come back in bfloat16.  With the 1/sqrt(d)-scaled inputs of BASELINE config 2 they
  stay below 8 and the bound is absolute there too (``absolute=ALL``).  For unscaled N(0,1)
  inputs gradients reach 8 and more, where one bfloat16 ulp (2^-4 at 8) already exceeds an absolute
  2e-2 whatever the kernel does; for those the max bound is |got - ref| <= tol * max(1, |ref|)
  (2 % above 1, i.e. ten bfloat16 roundings).

``check`` returns the observed errors; with ``BMA_PARITY_LOG=<file>`` every call appends them
as one JSON line, so the margins can be read after a run."""
import ctypes as C
import json
import math
import os

import numpy as np
import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200 import masks as M
from jaxmodules_b200 import _native as nat
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (1e-4, 1e-5), torch.bfloat16: (2e-2, 2e-3)}


def gen(shape, seed, dtype, scale=1.0):
    x = np.random.Generator(np.random.PCG64(seed)).standard_normal(shape, dtype=np.float32) * scale
    return torch.from_numpy(x).to(dtype)


def run(Q, K, V, dO, **kw):
    Qc, Kc, Vc = (x.cuda().requires_grad_(True) for x in (Q, K, V))
    O = jm.masked_attention_via_map(Qc, Kc, Vc, **kw)
    O.backward(dO.cuda().to(O.dtype))
    torch.cuda.synchronize()
    return O.detach().cpu(), Qc.grad.cpu(), Kc.grad.cpu(), Vc.grad.cpu()


ALL = ("O", "dQ", "dK", "dV")


def log_margins(what, stats):
    path = os.environ.get("BMA_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"case": what, **stats}) + "\n")


def check(got, ref, dtype, what, absolute=("O",)):
    """Asserts the bounds and returns {tensor: {max_abs, mean_abs, scaled_max, ref_max}}.  Tensors named in
    ``absolute`` must meet the max bound as a plain absolute error; the others relative to max(1, |ref|).
    float32 results are always held to the absolute bound."""
    max_tol, mean_tol = TOL[dtype]
    stats = {}
    for name, g in zip(ALL, got):
        r = np.asarray(ref[name], dtype=np.float64)
        gn = g.float().numpy().astype(np.float64)
        assert np.isfinite(gn).all(), f"{what}: {name} has non-finite values"
        err = np.abs(gn - r)
        scaled = err / np.maximum(1.0, np.abs(r))
        st = dict(max_abs=float(err.max()), mean_abs=float(err.mean()), scaled_max=float(scaled.max()), ref_max=float(np.abs(r).max()))
        stats[name] = st
        worst = st["max_abs"] if (name in absolute or dtype == torch.float32) else st["scaled_max"]
        assert worst <= max_tol and st["mean_abs"] <= mean_tol, f"{what}: {name} {st}"
    log_margins(what, stats)
    return stats


def oracle(Q, K, V, dO, **kw):
    kw = dict(kw)
    kw.pop("backend", None)
    kw.pop("out_dtype", None)
    return ao.masked_attention_dense(Q.float().numpy(), K.float().numpy(), V.float().numpy(), dO=dO.float().numpy(), **kw)


SMALL_MASKS = {
    "causal": dict(is_causal=True),
    "none": dict(),
    "sliding": dict(mask_fn=lambda h, q, k: (q - 2 <= k) & (k <= q + 2)),
    "alternating": dict(mask_fn=lambda h, q, k: (q + k) % 2 == 0),
    "head_specific": dict(mask_fn=lambda h, q, k: np.where(h % 2 == 0, q >= k, (q + k) % 2 == 0)),
    "batch_dependent": dict(mask_fn=lambda b, h, q, k: q + b >= k),
    "empty_rows": dict(mask_fn=lambda h, q, k: k < q),
}


@pytest.mark.parametrize("mask", list(SMALL_MASKS))
@pytest.mark.parametrize("block_size", [None, 4])
def test_reference_small_shapes_f32(mask, block_size):
    # shapes of the reference's tests/test_mapped_attention.py:303-430: N=L=8, H=4, d=16
    B, N, L, H, d = 2, 8, 8, 4, 16
    Q, K, V, dO = (gen((B, N if i in (0, 3) else L, H, d), i, torch.float32) for i in range(4))
    kw = dict(SMALL_MASKS[mask], block_size=block_size)
    check(run(Q, K, V, dO, **kw), oracle(Q, K, V, dO, **kw), torch.float32, mask)


def test_3d_inputs_gqa_and_rectangular():
    # tests/test_mapped_attention.py:564-605: N=32, L=64, Hq=8, Hkv=4, d=64, causal, no batch axis
    Q, K, V, dO = gen((32, 8, 64), 0, torch.float32), gen((64, 4, 64), 1, torch.float32), gen((64, 4, 64), 2, torch.float32), gen((32, 8, 64), 3, torch.float32)
    got = run(Q, K, V, dO, is_causal=True)
    assert got[0].shape == (32, 8, 64) and got[2].shape == (64, 4, 64)
    check(got, oracle(Q, K, V, dO, is_causal=True), torch.float32, "gqa")


def test_padding_path():
    # tests/test_mapped_attention.py:1076-1112: N=10, L=13, block 4
    Q, K, V, dO = gen((2, 10, 4, 16), 0, torch.float32), gen((2, 13, 4, 16), 1, torch.float32), gen((2, 13, 4, 16), 2, torch.float32), gen((2, 10, 4, 16), 3, torch.float32)
    for kw in (dict(is_causal=True, block_size=4), dict(block_size=4, window_size=(3, 2)),
               dict(mask_fn=lambda b, h, q, k: (q + k + b) % 3 != 0, block_size=4)):
        check(run(Q, K, V, dO, **kw), oracle(Q, K, V, dO, **kw), torch.float32, str(kw))


@pytest.mark.parametrize("window", [(1, 1), (16, 1), (17, 1), (40, 40)])
def test_window_size_semantics(window):
    # tests/test_mapped_attention.py:1593-1648: the block window restricts even a permissive mask
    N = L = 128
    Q, K, V, dO = (gen((1, N, 2, 32), i, torch.float32) for i in range(4))
    kw = dict(block_size=16, window_size=window)
    check(run(Q, K, V, dO, **kw), oracle(Q, K, V, dO, **kw), torch.float32, f"window{window}")
    kw = dict(block_size=16, window_size=window, is_causal=True)
    check(run(Q, K, V, dO, **kw), oracle(Q, K, V, dO, **kw), torch.float32, f"causal window{window}")


def test_window_larger_than_sequence_raises():
    Q = torch.randn(1, 32, 2, 16, device="cuda")
    with pytest.raises(ValueError):
        jm.masked_attention_via_map(Q, Q, Q, block_size=8, window_size=(30, 30))


def test_block_size_invariance_and_zero_inputs():
    Q, K, V, dO = (gen((1, 64, 2, 32), i, torch.float32) for i in range(4))
    outs = [run(Q, K, V, dO, is_causal=True, block_size=bs)[0] for bs in (4, 8, 16, None)]
    for o in outs[1:]:
        assert torch.equal(o, outs[0])          # block_size only matters through window_size
    z = torch.zeros(1, 16, 2, 32, device="cuda")
    assert torch.count_nonzero(jm.masked_attention_via_map(z, z, z, is_causal=True)) == 0
    big = jm.masked_attention_via_map(Q.cuda() * 100, K.cuda() * 100, V.cuda(), is_causal=True)
    assert torch.isfinite(big).all()            # max-subtracted softmax does not overflow


def test_config1_causal_f32_full():
    # BASELINE config 1: fp32, B=2, L=128, H=8, d=64, block_size=32, causal
    Q, K, V, dO = (gen((2, 128, 8, 64), i, torch.float32) for i in range(4))
    kw = dict(is_causal=True, block_size=32)
    got = run(Q, K, V, dO, **kw)
    check(got, oracle(Q, K, V, dO, **kw), torch.float32, "config1")
    port = ao.masked_attention_via_map(Q, K, V, dO=dO, **kw)     # the faithful blockwise port agrees too
    for g, p in zip(got, port):
        assert (g - p).abs().max() < 1e-4


def document_segments(B, L, lo, hi, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    seg = np.zeros((B, L), dtype=np.int32)
    for b in range(B):
        pos, sid = 0, 0
        while pos < L:
            n = int(rng.integers(lo, hi + 1))
            seg[b, pos:pos + n] = sid
            pos += n
            sid += 1
    return seg


BF16_CASES = {
    # reduced copies of BASELINE configs 2-4 (same d, block size, mask family, value scales)
    "config2_causal": dict(B=1, L=1024, H=2, d=128, scale=1 / math.sqrt(128), kw=lambda L: dict(is_causal=True, block_size=128)),
    "config3_sliding": dict(B=1, L=2048, H=2, d=128, scale=1.0,
                            kw=lambda L: dict(mask_fn=M.sliding_window_mask(256, 256), window_size=(256, 256), block_size=128)),
    "config4_documents": dict(B=2, L=2048, H=2, d=128, scale=1.0,
                              kw=lambda L: dict(mask_fn=M.document_mask(document_segments(2, L, 64, 700, 4), causal=True), block_size=128)),
    "ragged_gqa": dict(B=1, L=300, H=4, d=128, scale=1.0, kw=lambda L: dict(is_causal=True, block_size=64), Hkv=2, N=200),
    "d64": dict(B=1, L=512, H=2, d=64, scale=1.0, kw=lambda L: dict(is_causal=True, block_size=128)),
    # block windows whose block size is not the kernels' tile (several window blocks per 128-query tile), clamped at both ends
    "window_block32": dict(B=1, L=1024, H=2, d=128, scale=1.0, kw=lambda L: dict(block_size=32, window_size=(100, 40))),
    "window_block48_causal": dict(B=1, L=960, H=2, d=128, scale=1.0, kw=lambda L: dict(is_causal=True, block_size=48, window_size=(200, 0))),
    "d64_gqa_sliding_ragged": dict(B=2, L=700, H=4, d=64, scale=1.0, Hkv=2, N=333,
                                   kw=lambda L: dict(mask_fn=M.sliding_window_mask(150, 20), block_size=64)),
    "d64_documents": dict(B=2, L=1024, H=2, d=64, scale=1.0,
                          kw=lambda L: dict(mask_fn=M.document_mask(document_segments(2, L, 64, 400, 5), causal=True), block_size=128)),
}


@pytest.mark.parametrize("forward", ["auto", "persistent", "one_item_per_cta"])
@pytest.mark.parametrize("name", list(BF16_CASES))
def test_bf16_configs(name, forward, monkeypatch):
    if forward != "auto":      # force one of the two tensor-core forward kernels (read by the library at each call)
        monkeypatch.setenv("BMA_FWD_PERSISTENT", "1" if forward == "persistent" else "0")
    c = BF16_CASES[name]
    N, Hkv = c.get("N", c["L"]), c.get("Hkv", c["H"])
    Q = gen((c["B"], N, c["H"], c["d"]), 0, torch.bfloat16, c["scale"])
    K = gen((c["B"], c["L"], Hkv, c["d"]), 1, torch.bfloat16, c["scale"])
    V = gen((c["B"], c["L"], Hkv, c["d"]), 2, torch.bfloat16, c["scale"])
    dO = gen((c["B"], N, c["H"], c["d"]), 3, torch.float32)
    kw = c["kw"](c["L"])
    got = run(Q, K, V, dO, **kw)
    assert got[0].dtype == torch.float32 and got[1].dtype == torch.bfloat16   # O float32 like the reference
    # the 1/sqrt(d)-scaled shape is held to the absolute bound on every tensor
    check(got, oracle(Q, K, V, dO, **kw), torch.bfloat16, name, absolute=ALL if name == "config2_causal" else ("O",))


@pytest.mark.parametrize("d", [128, 64])
def test_bf16_output_option(d):
    """out_dtype=torch.bfloat16 (the tensor-core kernel stores O through its other staging path):
    equal to the float32 output rounded to bf16, ragged tail included; gradients unchanged in kind."""
    B, N, L, H = 2, 333, 700, 2
    Q = gen((B, N, H, d), 0, torch.bfloat16).cuda().requires_grad_(True)
    K, V = (gen((B, L, H, d), i, torch.bfloat16).cuda().requires_grad_(True) for i in (1, 2))
    kw = dict(mask_fn=M.sliding_window_mask(200, 30), block_size=64)
    o32 = jm.masked_attention_via_map(Q, K, V, **kw)
    o16 = jm.masked_attention_via_map(Q, K, V, out_dtype=torch.bfloat16, **kw)
    assert o16.dtype == torch.bfloat16 and o16.shape == o32.shape
    assert (o16.float() - o32).abs().max() <= 2 ** -8 * o32.abs().max().clamp(min=1.0)
    o16.backward(torch.ones_like(o16))
    g16 = Q.grad.clone(); Q.grad = None
    o32.backward(torch.ones_like(o32))
    assert torch.isfinite(g16).all() and (g16.float() - Q.grad.float()).abs().max() < 3e-2


def test_simt_and_auto_backends_agree_bf16():
    """The exact-FP32 SIMT kernels cross-check whatever backend AUTO selects."""
    Q, K, V = (gen((1, 512, 2, 128), i, torch.bfloat16) for i in range(3))
    dO = gen((1, 512, 2, 128), 3, torch.float32)
    a = run(Q, K, V, dO, is_causal=True)
    b = run(Q, K, V, dO, is_causal=True, backend=nat.BMA_BACKEND_SIMT)
    for x, y in zip(a, b):
        assert (x.float() - y.float()).abs().max() <= 2e-2


@pytest.mark.parametrize("d,G,mask", [(128, 1, "causal"), (128, 2, "band"), (64, 1, "segments"), (128, 1, "ragged")])
def test_backward_ds_hand_over_matches_recompute(d, G, mask):
    """The tensor-core backward with the scratch buffer (dK/dV kernel stores every dS tile, the dQ kernel
    replays them) against the same backward without it (dQ kernel recomputes S and dP), and both against
    the exact-FP32 SIMT kernels."""
    from jaxmodules_b200 import attention as A
    N = L = 640 if mask != "ragged" else 600
    Q = gen((2, N, 2 * G, d), 0, torch.bfloat16)
    K, V = (gen((2, L, 2, d), i, torch.bfloat16) for i in (1, 2))
    dO = gen((2, N, 2 * G, d), 3, torch.float32)
    kw = dict(is_causal=True)
    if mask == "band":
        kw = dict(mask_fn=M.sliding_window_mask(100, 30))
    if mask == "segments":
        seg = np.sort(np.random.Generator(np.random.PCG64(5)).integers(0, 4, size=(2, L)), axis=1).astype(np.int32)
        kw = dict(mask_fn=M.and_masks(M.document_mask(seg), M.causal_mask()))
    limit = A._scratch_limit
    try:
        with_scratch = run(Q, K, V, dO, **kw)
        info = dict(A.last_backward_info)
        assert info["whole"] and info["scratch_bytes"] > 0
        # compact addressing: 32 KB per VISITED block plus the slot tables, well below the dense grid of 2 x 2G x 5 x 5 blocks
        if mask in ("causal", "segments"):
            assert info["scratch_bytes"] < 0.75 * 32768 * 2 * 2 * G * 5 * 5
        for fraction in (0.6, 0.35):              # 4 (batch, kv head) units: one batch per range, then one unit per range
            A.set_backward_scratch_limit(limit, fraction)
            in_ranges = run(Q, K, V, dO, **kw)
            assert not A.last_backward_info["whole"] and A.last_backward_info["workspace_bytes"] < info["scratch_bytes"]
            assert all(torch.equal(x, y) for x, y in zip(with_scratch, in_ranges))
        A.set_backward_scratch_limit(0)
        recomputed = run(Q, K, V, dO, **kw)
    finally:
        A.set_backward_scratch_limit(limit)
    exact = run(Q, K, V, dO, backend=nat.BMA_BACKEND_SIMT, **kw)
    for x, y, z in zip(with_scratch, recomputed, exact):
        assert torch.isfinite(x.float()).all()
        assert (x.float() - y.float()).abs().max() <= 2e-2 * max(1.0, float(z.float().abs().max()))
        assert (x.float() - z.float()).abs().max() <= 2e-2 * max(1.0, float(z.float().abs().max()))
        assert (x.float() - z.float()).abs().mean() <= 2e-3


def test_rows_without_keys_inside_a_visited_tile_bf16():
    """More queries than keys under a band mask: the q tile where the band runs out has rows with and rows without an
    allowed key.  The rows without must give O = 0 and lse = -inf (jaxmodules/attention.py:99-100) on the tensor-core
    path too, whose polynomial exponential does not return an exact 0 for a masked score."""
    N, L = 832, 383
    Q = gen((1, N, 2, 128), 0, torch.bfloat16)
    K, V = (gen((1, L, 1, 128), i, torch.bfloat16) for i in (1, 2))
    O, lse = jm.masked_attention_via_map(Q.cuda(), K.cuda(), V.cuda(), mask_fn=M.sliding_window_mask(216, 42), block_size=100,
                                         return_lse=True)
    last = L - 1 + 216                     # last query that still sees key L-1
    assert float(O[:, last + 1:].abs().max()) == 0.0 and bool(torch.isinf(lse[..., last + 1:]).all())
    assert bool(torch.isfinite(lse[..., :last + 1]).all()) and float(O[:, :last + 1].abs().max()) > 0.1


def test_full_size_properties_config2():
    """BASELINE config 2 at full size (B=8, L=4096, H=32, d=128, bf16 causal): properties that do
    not need the oracle — row 0 attends only key 0 so O[:,0] == V[:,0]; the output is a convex
    combination of values; a (b,h) slice recomputed alone is bit-identical; dV column sums equal
    dO column sums (softmax rows sum to 1)."""
    B, L, H, d = 8, 4096, 32, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    Q, K, V = (torch.randn(B, L, H, d, device="cuda", generator=g).mul_(1 / math.sqrt(d)).to(torch.bfloat16) for _ in range(3))
    Q.requires_grad_(True); K.requires_grad_(True); V.requires_grad_(True)
    O = jm.masked_attention_via_map(Q, K, V, is_causal=True, block_size=128)
    assert torch.isfinite(O).all()
    assert (O[:, 0] - V[:, 0].float()).abs().max() < 1e-6
    vmax = V.float().abs().amax(dim=1, keepdim=True)
    assert (O.abs() <= vmax + 1e-3).all()
    sl = jm.masked_attention_via_map(Q[3:4, :, 5:6].detach().contiguous(), K[3:4, :, 5:6].detach().contiguous(),
                                     V[3:4, :, 5:6].detach().contiguous(), is_causal=True, block_size=128)
    assert torch.equal(sl, O[3:4, :, 5:6])
    dO = torch.randn(B, L, H, d, device="cuda", generator=g)
    O.backward(dO)
    for t in (Q.grad, K.grad, V.grad):
        assert torch.isfinite(t).all()
    lhs = V.grad.float().sum(dim=1)
    rhs = dO.to(torch.bfloat16).float().sum(dim=1) if False else dO.sum(dim=1)
    assert (lhs - rhs).abs().max() / rhs.abs().max() < 2e-2


FULL_SIZE = {
    # BASELINE configs 2, 3 and 4 and the L=8192 causal target shape, at their full sizes
    "config2_causal": dict(B=8, L=4096, H=32, scale=1 / math.sqrt(128), absolute=ALL,
                           kw=lambda seg: dict(is_causal=True, block_size=128), dense=lambda seg, b, q, k: k <= q),
    "config3_sliding": dict(B=4, L=8192, H=16, kw=lambda seg: dict(mask_fn=M.sliding_window_mask(256, 256), window_size=(256, 256), block_size=128),
                            dense=lambda seg, b, q, k: (k >= q - 256) & (k <= q + 256)),
    "config4_documents": dict(B=4, L=16384, H=16, kw=lambda seg: dict(mask_fn=M.document_mask(seg, causal=True), block_size=128),
                              dense=lambda seg, b, q, k: (seg[b][q] == seg[b][k]) & (k <= q)),
    "target_causal_8192": dict(B=4, L=8192, H=32, kw=lambda seg: dict(is_causal=True, block_size=128),
                               dense=lambda seg, b, q, k: k <= q),
}


def dense_fp32_slice(q, k, v, do, allowed, scale, chunk=2048):
    """float32 attention of ONE (batch, head) slice on the GPU, written out densely in query chunks:
    q [N,d], k, v [L,d], do [N,d]; ``allowed(qi, ki)`` -> bool [n, L] for query rows qi.  Returns
    O, dQ, dK, dV, lse with the formulas of the numerical contract (P = exp(s - lse), delta = rowsum(dO*O),
    dS = P * (dO V^T - delta)).  No tensor-core arithmetic: torch float32 matmul with TF32 off."""
    assert not torch.backends.cuda.matmul.allow_tf32
    N, L = q.shape[0], k.shape[0]
    O, dQ, lse = torch.empty_like(q), torch.empty_like(q), torch.empty(N, device=q.device)
    dK, dV = torch.zeros_like(k), torch.zeros_like(v)
    ki = torch.arange(L, device=q.device)[None, :]
    for q0 in range(0, N, chunk):
        sl = slice(q0, min(N, q0 + chunk))
        qi = torch.arange(sl.start, sl.stop, device=q.device)[:, None]
        m = allowed(qi, ki)
        s = (q[sl] @ k.T) * scale
        s.masked_fill_(~m, float("-inf"))
        row_lse = torch.logsumexp(s, dim=-1)
        dead = torch.isinf(row_lse)
        p = torch.exp(s - torch.where(dead, torch.zeros_like(row_lse), row_lse)[:, None])
        o = p @ v
        dp = do[sl] @ v.T
        ds = p * (dp - (do[sl] * o).sum(dim=-1, keepdim=True))
        O[sl], lse[sl] = o, row_lse
        dQ[sl] = (ds @ k) * scale
        dK += (ds.T @ q[sl]) * scale
        dV += p.T @ do[sl]
        del s, p, dp, ds, m
    return dict(O=O, dQ=dQ, dK=dK, dV=dV, lse=lse)


def compare_slice(got, ref, what, absolute=("O",)):
    """bf16 bounds on one slice (device tensors); returns the observed errors."""
    stats = {}
    for name in ALL:
        g, r = got[name].detach().float(), ref[name]
        err = (g - r).abs()
        scaled = err / r.abs().clamp(min=1.0)
        st = dict(max_abs=float(err.max()), mean_abs=float(err.mean()), scaled_max=float(scaled.max()), ref_max=float(r.abs().max()))
        stats[name] = st
        worst = st["max_abs"] if name in absolute else st["scaled_max"]
        assert bool(torch.isfinite(g).all()) and worst <= 2e-2 and st["mean_abs"] <= 2e-3, (what, name, st)
    log_margins(what, stats)
    return stats


@pytest.mark.parametrize("forward", ["auto", "other"])
@pytest.mark.parametrize("name", list(FULL_SIZE))
def test_full_size_slices_against_dense_fp32(name, forward, monkeypatch):
    """Full-size runs of the BASELINE shapes; two (batch, head) slices of the result — slices are
    independent of one another — are compared with a dense float32 torch attention of the same slice on
    the GPU.  bf16 tolerances as above: O absolute everywhere; every tensor absolute for config 2, whose
    inputs carry the 1/sqrt(d) scale."""
    c = FULL_SIZE[name]
    if forward == "other":     # the tensor-core forward kernel that AUTO does not pick for this mask
        monkeypatch.setenv("BMA_FWD_PERSISTENT", "0" if name == "config3_sliding" else "1")
    B, L, H, d = c["B"], c["L"], c["H"], 128
    g = torch.Generator(device="cuda").manual_seed(1)
    Q, K, V = (torch.randn(B, L, H, d, device="cuda", generator=g).mul_(c.get("scale", 1.0)).to(torch.bfloat16).requires_grad_(True)
               for _ in range(3))
    dO = torch.randn(B, L, H, d, device="cuda", generator=g)
    seg_np = document_segments(B, L, 256, 4096, 4)
    O = jm.masked_attention_via_map(Q, K, V, **c["kw"](seg_np))
    O.backward(dO)
    seg = torch.from_numpy(seg_np).cuda()
    for b, h in ((0, 0), (B - 1, H - 1)):
        q, k, v = (t[b, :, h].detach().float() for t in (Q, K, V))
        ref = dense_fp32_slice(q, k, v, dO[b, :, h], lambda qi, ki: c["dense"](seg, b, qi, ki), 1 / math.sqrt(d))
        got = dict(O=O[b, :, h], dQ=Q.grad[b, :, h], dK=K.grad[b, :, h], dV=V.grad[b, :, h])
        compare_slice(got, ref, f"full size {name} (b={b}, h={h})", absolute=c.get("absolute", ("O",)))


def test_config5_long_context_against_dense_fp32():
    """BASELINE config 5 at its full sequence length (B=1, L=131072, d=128, bf16 causal) with 2 of the 32
    heads — heads are independent.  One head alone would need 34 GB of backward scratch, so the backward takes
    the recomputing dQ kernel, and the kv lists are 1024 tiles long (the 16-bit merged list).  Every row of one
    head's O, lse, dQ, dK, dV is compared with a dense float32 torch attention over all 131072 keys, computed in
    query chunks."""
    B, L, H, d = 1, 131072, 2, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    Q, K, V = (torch.randn(B, L, H, d, device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True) for _ in range(3))
    dO = torch.randn(B, L, H, d, device="cuda", generator=g)
    O, lse = jm.masked_attention_via_map(Q, K, V, is_causal=True, block_size=128, return_lse=True)
    O.backward(dO)
    h = 1
    q, k, v = (t[0, :, h].detach().float() for t in (Q, K, V))
    ref = dense_fp32_slice(q, k, v, dO[0, :, h], lambda qi, ki: ki <= qi, 1 / math.sqrt(d), chunk=1024)
    got = dict(O=O[0, :, h], dQ=Q.grad[0, :, h], dK=K.grad[0, :, h], dV=V.grad[0, :, h])
    compare_slice(got, ref, "config 5, L=131072 (head 1 of 2)")
    assert float((lse[0, h] - ref["lse"]).abs().max()) <= 1e-3


def test_virtual_ring_offsets_and_merge():
    """The sequence-partition path on one GPU: every (query chunk, key chunk) pair is attended with
    global offsets in the mask description and merged with bma_attn_merge, exactly what the ring
    does step by step; the result must match the unsplit attention."""
    from jaxmodules_b200 import sharding as S
    B, L, H, d, world = 1, 1024, 2, 128, 4
    Q, K, V = (gen((B, L, H, d), i, torch.bfloat16).cuda() for i in range(3))
    n = L // world
    # the third mask is an arbitrary traced function in the tile form: its tiles are indexed by GLOBAL positions, so the
    # shards only move the offsets
    from jaxmodules_b200 import mask_program as P
    tiles = P.build_tiles(P.trace(lambda b, h, q, k: (k <= q) & ((q - k) % 3 != 1) | (k == q)), B, H, L, L, "cuda")
    for terms in (M.MaskTerms(causal=True), M.MaskTerms(band=(300, 40)), M.MaskTerms(tiles=tiles)):
        full, full_lse = S.cuda_attend(Q, K, V, terms)
        for r in range(world):
            O = lse = None
            for owner in S.ring_schedule(r, world):
                t = M.MaskTerms(causal=terms.causal, band=terms.band, tiles=terms.tiles, q_offset=r * n, k_offset=owner * n)
                O_s, lse_s = S.cuda_attend(Q[:, r * n:(r + 1) * n], K[:, owner * n:(owner + 1) * n].contiguous(),
                                           V[:, owner * n:(owner + 1) * n].contiguous(), t)
                O, lse = (O_s, lse_s) if O is None else S.cuda_merge(O, lse, O_s, lse_s)
            torch.cuda.synchronize()
            assert (O - full[:, r * n:(r + 1) * n]).abs().max() < 2e-3
            sl = full_lse[:, :, r * n:(r + 1) * n]
            finite = torch.isfinite(sl)
            assert torch.equal(torch.isfinite(lse), finite) and (lse[finite] - sl[finite]).abs().max() < 1e-4


def test_virtual_ring_backward():
    """Backward of the sequence partition on one GPU: each (query chunk, key chunk) pair is
    differentiated with the queries' FINAL output and log-sum-exp and global offsets in the mask;
    summed over the pairs the gradients must equal those of the unsplit attention."""
    from jaxmodules_b200 import sharding as S
    B, L, H, d, world = 1, 1024, 2, 128, 4
    Q, K, V = (gen((B, L, H, d), i, torch.bfloat16).cuda() for i in range(3))
    dO = gen((B, L, H, d), 3, torch.float32).cuda()
    n = L // world
    for terms in (M.MaskTerms(causal=True), M.MaskTerms(band=(300, 40))):
        O, lse = S.cuda_attend(Q, K, V, terms)
        ref = S.cuda_backward(Q, K, V, O, lse, dO, terms)
        acc = [torch.zeros(B, L, H, d, device="cuda") for _ in range(3)]
        for r in range(world):
            qs = slice(r * n, (r + 1) * n)
            for owner in S.ring_schedule(r, world):
                ks = slice(owner * n, (owner + 1) * n)
                t = M.MaskTerms(causal=terms.causal, band=terms.band, q_offset=r * n, k_offset=owner * n)
                dq, dk, dv = S.cuda_backward(Q[:, qs].contiguous(), K[:, ks].contiguous(), V[:, ks].contiguous(),
                                             O[:, qs].contiguous(), lse[:, :, qs].contiguous(), dO[:, qs].contiguous(), t)
                acc[0][:, qs] += dq
                acc[1][:, ks] += dk
                acc[2][:, ks] += dv
        torch.cuda.synchronize()
        for got, want, name in zip(acc, ref, ("dQ", "dK", "dV")):
            err = (got - want.float()).abs() / want.float().abs().clamp(min=1.0)
            assert err.max() < 3e-2 and err.mean() < 2e-3, (name, float(err.max()), float(err.mean()))


def test_tensor_core_backend_is_selected():
    """bf16 with head dim 128 must run on the tcgen05 kernels (no silent fall-back to SIMT)."""
    from jaxmodules_b200 import attention as A
    Q = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16, device="cuda")
    assert A.plan(Q, Q, Q)[0] == nat.BMA_BACKEND_TCGEN05 and A.plan(Q, Q, Q, backward=True)[0] == nat.BMA_BACKEND_TCGEN05
    Q64 = torch.zeros(1, 256, 2, 64, dtype=torch.bfloat16, device="cuda")
    assert A.plan(Q64, Q64, Q64)[0] == nat.BMA_BACKEND_TCGEN05 and A.plan(Q64, Q64, Q64, backward=True)[0] == nat.BMA_BACKEND_TCGEN05
    Q32 = torch.zeros(1, 256, 2, 32, dtype=torch.bfloat16, device="cuda")
    assert A.plan(Q32, Q32, Q32)[0] == nat.BMA_BACKEND_SIMT
    Qf = torch.zeros(1, 256, 2, 64, dtype=torch.float32, device="cuda")
    assert A.plan(Qf, Qf, Qf)[0] == nat.BMA_BACKEND_SIMT
    rc = C.c_int32()
    assert nat.lib().bma_device_status(torch.cuda.current_stream().cuda_stream, C.byref(rc)) == nat.BMA_OK and rc.value == 0


@pytest.mark.parametrize("dtype,d", [(torch.float32, 16), (torch.bfloat16, 128)], ids=["f32_simt", "bf16_tcgen05"])
def test_kernel_fn_family(dtype, d):
    """kernel_fn = exp(a*q.k + b): threshold_kernel (jaxmodules/attention.py:18-36) and the custom
    kernel of the reference's tests/test_mapped_attention.py:1122-1142; forward, lse and gradients."""
    B, N, H = 1, 256, 2
    scale = 1.0 if dtype == torch.float32 else 0.3     # keeps exp(q.k) representable without the 1/sqrt(d)
    Q, K, V = (gen((B, N, H, d), i, dtype, scale) for i in range(3))
    dO = gen((B, N, H, d), 3, torch.float32)
    custom = lambda q, k: np.exp(np.dot(q, k) / (2 * np.sqrt(k.shape[-1])))
    for kernel_fn, kernel in ((jm.threshold_kernel(3.0), (1.0, -3.0 / math.sqrt(d))), (jm.threshold_kernel(), (1.0, 0.0)),
                              (custom, (0.5 / math.sqrt(d), 0.0))):
        got = run(Q, K, V, dO, is_causal=True, kernel_fn=kernel_fn)
        ref = ao.masked_attention_dense(Q.float().numpy(), K.float().numpy(), V.float().numpy(), dO=dO.numpy(),
                                        is_causal=True, kernel=kernel)
        check(got, ref, dtype, f"kernel {kernel}")
        _, lse = jm.masked_attention_via_map(Q.cuda(), K.cuda(), V.cuda(), is_causal=True, kernel_fn=kernel_fn, return_lse=True)
        assert np.abs(lse.cpu().numpy() - ref["lse"]).max() <= (1e-4 if dtype == torch.float32 else 2e-2)
    default = run(Q, K, V, dO, is_causal=True)
    assert not torch.allclose(got[0], default[0], rtol=1e-2)      # the reference's own assertion (:1141-1142)


def test_negative_scale_kernel_bf16():
    """kernel_fn = exp(-q.k / sqrt(d)): the logit scale is negative, so the running maximum of the scaled scores is
    the MINIMUM of the raw ones.  Inputs are large enough (logit range beyond 2^127 in either direction) that
    exponentials taken against the wrong extreme would overflow; the tensor-core forward must stay finite and
    match the oracle.  O is held to the absolute bf16 bound; the gradients of these 5x-scaled inputs reach 15 and
    carry the bf16 rounding of dS times |K| = 5, so they are held to 2e-2 / 2e-3 of their own largest entry."""
    B, N, H, d = 1, 384, 2, 128
    Q, K, V = gen((B, N, H, d), 0, torch.bfloat16, 5.0), gen((B, N, H, d), 1, torch.bfloat16, 5.0), gen((B, N, H, d), 2, torch.bfloat16)
    dO = gen((B, N, H, d), 3, torch.float32)
    neg = lambda q, k: np.exp(-np.dot(q, k) / np.sqrt(k.shape[-1]))
    from jaxmodules_b200 import attention as A
    assert A.plan(Q.cuda(), K.cuda(), V.cuda(), scale=-1 / math.sqrt(d))[0] == nat.BMA_BACKEND_TCGEN05
    got = run(Q, K, V, dO, is_causal=True, kernel_fn=neg)
    ref = ao.masked_attention_dense(Q.float().numpy(), K.float().numpy(), V.float().numpy(), dO=dO.numpy(), is_causal=True,
                                    kernel=(-1 / math.sqrt(d), 0.0))
    for name, g in zip(ALL, got):
        g, r = g.float().numpy().astype(np.float64), ref[name]
        assert np.isfinite(g).all(), name
        err, top = np.abs(g - r), (1.0 if name == "O" else max(1.0, float(np.abs(r).max())))
        assert err.max() <= 2e-2 * top and err.mean() <= 2e-3 * top, (name, err.max(), err.mean(), top)


@pytest.mark.parametrize("N,L", [(1, 1), (1, 128), (128, 1), (5, 300), (300, 5), (129, 129), (127, 257)])
@pytest.mark.parametrize("d", [128, 64])
def test_degenerate_lengths_bf16(N, L, d):
    """Single tokens, one side shorter than a tile, lengths one past a tile boundary: the tensor-core kernels clip every
    tile against the valid box (TMA zero fill on the way in, clipped stores on the way out).  GQA 4:1, with and
    without a mask, forward and backward against the oracle."""
    B, Hq, Hkv = 2, 4, 1
    Q = gen((B, N, Hq, d), 0, torch.bfloat16)
    K, V = (gen((B, L, Hkv, d), i, torch.bfloat16) for i in (1, 2))
    dO = gen((B, N, Hq, d), 3, torch.float32)
    # block_size 7 divides none of the lengths: the reference's padding path, which takes any number of keys
    # (jaxmodules/attention.py:426-437); without window_size the result does not depend on it
    for kw in (dict(block_size=7), dict(mask_fn=M.sliding_window_mask(3, 100), block_size=7)):
        got = run(Q, K, V, dO, **kw)
        # The oracle gets the cotangent as the tensor-core backward uses it, rounded to bf16: with one key, 512 (query,
        # head) cotangents add up in a single dV row, and the rounding of each of them -- not of anything the kernels
        # compute -- would dominate the comparison (0.2 absolute on a sum whose terms cancel to 4).
        ref = oracle(Q, K, V, dO.to(torch.bfloat16).float(), **kw)
        for name, g in zip(ALL, got):
            g, r = g.float().numpy().astype(np.float64), ref[name]
            assert np.isfinite(g).all(), name
            err = np.abs(g - r)
            # O absolute.  Gradients relative to their own largest entry: a handful of keys collect the bf16-rounded dS and
            # P of up to 1200 (query, head) rows each, and the sum of those roundings grows with the row count while
            # single entries cancel towards zero
            top = 1.0 if name == "O" else max(1.0, float(np.abs(r).max()))
            assert err.max() <= 2e-2 * top and err.mean() <= 2e-3 * top, (N, L, d, sorted(kw), name, err.max(), err.mean(), top)


def test_mask_that_allows_nothing_bf16():
    """mask_fn == False everywhere: every row is empty, O = 0, lse = -inf and all gradients are exactly zero
    (jaxmodules/attention.py:99-100), without a single block in the lists."""
    Q, K, V = (gen((1, 256, 2, 128), i, torch.bfloat16) for i in range(3))
    dO = gen((1, 256, 2, 128), 3, torch.float32)
    never = lambda b, h, q, k: (q < 0) & (k < 0)
    got = run(Q, K, V, dO, mask_fn=never)
    for t in got:
        assert float(t.float().abs().max()) == 0.0
    _, lse = jm.masked_attention_via_map(Q.cuda(), K.cuda(), V.cuda(), mask_fn=never, return_lse=True)
    assert bool(torch.isinf(lse).all())
