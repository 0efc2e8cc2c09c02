"""The cases behind tests/golden/reference_vectors.npz: shapes, seeds, masks and call arguments, shared by the generator
(which runs the reference's own source on them) and by the tests (which run the oracle and the CUDA path on them).

Inputs are not stored: they are regenerated from numpy PCG64 seeds.  A mask is written once with plain integer operators, so
that the same function body serves torch tensors under vmap (the generator), numpy index grids (the oracle) and the
package's tracer; masks that read a segment table come in one flavour per consumer (``flavour`` = "torch", "numpy",
"package").  Results above ``FULL_BELOW`` elements are stored as a seeded sample of ``SAMPLE`` entries plus ``PROJECTIONS``
float64 inner products with seeded normal vectors over the WHOLE tensor, so that every element is still pinned."""
import zlib

import numpy as np

FULL_BELOW, SAMPLE, PROJECTIONS = 2049, 1024, 4


def normal(shape, seed, scale=1.0):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal(shape, dtype=np.float32) * np.float32(scale)


def segments(B, L, lo, hi, seed):
    """Per-row document ids: consecutive runs with lengths uniform in [lo, hi], truncated at L."""
    rng = np.random.Generator(np.random.PCG64(seed))
    seg = np.zeros((B, L), dtype=np.int64)
    for b in range(B):
        pos = sid = 0
        while pos < L:
            n = int(rng.integers(lo, hi + 1))
            seg[b, pos:pos + n] = sid
            pos, sid = pos + n, sid + 1
    return seg


def documents_causal(seg, flavour):
    if flavour == "torch":
        import torch
        t = torch.from_numpy(seg)
        return lambda b, h, q, k: (t[b, q] == t[b, k]) & (q >= k)
    if flavour == "numpy":
        return lambda b, h, q, k: (seg[b, q] == seg[b, k]) & (q >= k)
    from jaxmodules_b200 import masks as M
    import torch
    return M.document_mask(torch.from_numpy(seg.astype(np.int32)), causal=True)


def plain(fn):
    return lambda flavour: fn


# ---- masked_attention_via_map --------------------------------------------------------------------------------------
# shape = (B or None for 3-d inputs, N, L, Hq, Hkv, d); kw without the mask; mask(flavour) -> mask_fn or None
ATTENTION = {
    # BASELINE config 1 (the reference's CPU-runnable case)
    "config1_causal_f32": dict(shape=(2, 128, 128, 8, 8, 64), kw=dict(is_causal=True, block_size=32)),
    "causal_block8": dict(shape=(2, 32, 32, 4, 4, 16), kw=dict(is_causal=True, block_size=8)),
    "causal_no_block_size": dict(shape=(1, 24, 24, 2, 2, 16), kw=dict(is_causal=True)),
    "gqa_causal_left_window": dict(shape=(2, 32, 32, 4, 2, 16), kw=dict(is_causal=True, block_size=8, window_size=(8, 0))),
    "mqa_blocks_of_7_padded": dict(shape=(1, 30, 30, 4, 1, 16), kw=dict(block_size=7),
                                   mask=plain(lambda b, h, q, k: (q // 7) == (k // 7))),
    "padded_rectangular_window": dict(shape=(2, 10, 13, 4, 4, 16), kw=dict(block_size=4, window_size=(3, 2))),
    "cross_rectangular_unmasked": dict(shape=(1, 24, 40, 2, 2, 8), kw=dict(block_size=8)),
    "band_inside_window": dict(shape=(2, 64, 64, 2, 2, 16), kw=dict(block_size=8, window_size=(8, 8)),
                               mask=plain(lambda b, h, q, k: (q - k <= 8) & (k - q <= 8))),
    "window_not_block_multiple": dict(shape=(1, 64, 64, 2, 1, 16), kw=dict(block_size=16, window_size=(17, 1))),
    "batch_and_head_dependent": dict(shape=(2, 16, 16, 4, 4, 16), kw=dict(),
                                     mask=plain(lambda b, h, q, k: (q + k + b + h) % 3 != 0)),
    "three_argument_mask_rows_without_keys": dict(shape=(1, 16, 16, 2, 2, 16), kw=dict(block_size=4),
                                                  mask=plain(lambda h, q, k: k < q)),
    "packed_documents_causal": dict(shape=(2, 64, 64, 4, 2, 16), kw=dict(block_size=16),
                                    mask=lambda flavour: documents_causal(segments(2, 64, 5, 24, 7), flavour)),
    "three_dimensional_inputs_gqa": dict(shape=(None, 16, 32, 4, 2, 32), kw=dict(is_causal=True)),
    # kernel_fn: the reference's threshold_kernel (dot product NOT divided by sqrt(d)) and a custom exp(a q.k)
    "threshold_kernel_causal": dict(shape=(1, 32, 32, 2, 2, 16), kw=dict(is_causal=True, block_size=8), input_scale=0.5,
                                    kernel=("threshold", 0.7)),
    "custom_exponential_kernel_gqa": dict(shape=(2, 16, 24, 4, 2, 16), kw=dict(block_size=8), input_scale=0.7,
                                          kernel=("exponential", 0.3)),
    # bfloat16 inputs: the reference then computes its scores in bfloat16 (no max subtraction, float32 running sums)
    "bf16_gqa_causal_d128": dict(shape=(1, 256, 256, 2, 1, 128), kw=dict(is_causal=True, block_size=128), dtype="bfloat16"),
    "bf16_documents_d128": dict(shape=(1, 256, 256, 2, 2, 128), kw=dict(block_size=128), dtype="bfloat16",
                                mask=lambda flavour: documents_causal(segments(1, 256, 20, 90, 11), flavour)),
    # the shapes of BASELINE configs 3 and 4 at L = 1024 (8 x 8 blocks of 128): band inside a block window, packed documents
    "bf16_band_window_8_blocks": dict(shape=(1, 1024, 1024, 2, 2, 128), kw=dict(block_size=128, window_size=(256, 256)),
                                      dtype="bfloat16", mask=plain(lambda b, h, q, k: (q - k <= 256) & (k - q <= 256))),
    "bf16_documents_8_blocks": dict(shape=(2, 1024, 1024, 4, 2, 128), kw=dict(block_size=128), dtype="bfloat16",
                                    mask=lambda flavour: documents_causal(segments(2, 1024, 64, 400, 4), flavour)),
    "bf16_causal_d64_8_blocks": dict(shape=(1, 1024, 1024, 4, 4, 64), kw=dict(is_causal=True, block_size=128), dtype="bfloat16"),
}


def attention_inputs(name):
    """(Q, K, V, dO) as float32 ndarrays (bfloat16 cases: round them to bfloat16 before use)."""
    c = ATTENTION[name]
    B, N, L, Hq, Hkv, d = c["shape"]
    lead = () if B is None else (B,)
    base = zlib.crc32(name.encode()) % (2 ** 31)
    s = c.get("input_scale", 1.0)
    return (normal(lead + (N, Hq, d), base + 0, s), normal(lead + (L, Hkv, d), base + 1, s),
            normal(lead + (L, Hkv, d), base + 2, s), normal(lead + (N, Hq, d), base + 3))


def attention_kwargs(name, flavour, reference_module=None):
    """Keyword arguments of the call for one consumer.  ``kernel``: the generator ("torch") takes the reference's own
    threshold_kernel from ``reference_module`` or a jnp lambda; the oracle ("numpy") takes the (a, b) of exp(a q.k + b);
    the package takes its threshold_kernel or a torch lambda, which it probes."""
    c = ATTENTION[name]
    kw = dict(c["kw"])
    if "mask" in c:
        kw["mask_fn"] = c["mask"](flavour)
    if "kernel" in c:
        kind, value = c["kernel"]
        d = c["shape"][5]
        if flavour == "torch":
            import jax.numpy as jnp
            kw["kernel_fn"] = (reference_module.threshold_kernel(value) if kind == "threshold"
                               else (lambda q, k: jnp.exp(value * jnp.dot(q, k))))
        elif flavour == "numpy":
            kw["kernel"] = (1.0, -value / d ** 0.5) if kind == "threshold" else (value, 0.0)
        else:
            import torch
            import jaxmodules_b200 as jm
            kw["kernel_fn"] = jm.threshold_kernel(value) if kind == "threshold" else (lambda q, k: torch.exp(value * torch.dot(q, k)))
    return kw


def geometry_cases(count=240):
    """Random (shape, block_size, window_size, is_causal) combinations — most of them invalid in some way — for which
    the generator records whether the reference raises.  Returns dicts with N, L, Hq, Hkv, d, kw."""
    rng = np.random.Generator(np.random.PCG64(2024))
    cases = []
    for _ in range(count):
        Hkv = int(rng.integers(1, 3))
        Hq = Hkv * int(rng.choice([1, 2])) if rng.random() < 0.85 else Hkv + 1 + int(rng.integers(0, 2))
        N = int(rng.integers(1, 33))
        L = N if rng.random() < 0.4 else int(rng.integers(1, 33))
        kw = {}
        if rng.random() < 0.5:
            kw["is_causal"] = True
        r = rng.random()
        if r < 0.45:
            kw["block_size"] = int(rng.integers(1, 13))
        elif r < 0.7:
            divisors = [x for x in range(1, N + 1) if N % x == 0]
            kw["block_size"] = int(rng.choice(divisors))
        if "block_size" in kw and rng.random() < 0.6:
            bs = kw["block_size"]
            kw["window_size"] = (int(rng.integers(0, 3 * bs + 1)), int(rng.integers(0, 2 * bs + 1)))
        elif rng.random() < 0.1:
            kw["window_size"] = (int(rng.integers(0, N + 1)), int(rng.integers(0, N + 1)))
        cases.append(dict(N=N, L=L, Hq=Hq, Hkv=Hkv, d=8, kw=kw))
    return cases


# ---- create_block_mask / BlockMask constructors ---------------------------------------------------------------------
BLOCK_MASK_FIELDS = ["kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices",
                     "q_num_blocks", "q_indices", "full_q_num_blocks", "full_q_indices"]

BLOCK_MASK = {
    "causal": dict(args=(2, 2, 64, 64, 16), mask=plain(lambda b, h, q, k: q >= k)),
    "sliding_window_5": dict(args=(1, 2, 64, 64, 8), mask=plain(lambda b, h, q, k: (q - k <= 5) & (k - q <= 5))),
    "rectangular_blocks_mod3": dict(args=(1, 1, 32, 64, (8, 16)), mask=plain(lambda b, h, q, k: (q + k) % 3 == 0)),
    "rectangular_causal": dict(args=(1, 2, 32, 96, (8, 32)), mask=plain(lambda b, h, q, k: q >= k)),
    "batch_and_head_dependent": dict(args=(2, 3, 32, 32, 8), mask=plain(lambda b, h, q, k: (k <= q + 4 * h) & (k >= 8 * b))),
    "documents_causal": dict(args=(2, 1, 64, 64, 8),
                             mask=lambda flavour: documents_causal(segments(2, 64, 5, 24, 3), flavour)),
    "everything": dict(args=(1, 2, 32, 32, 8), mask=plain(lambda b, h, q, k: q >= 0)),
    "nothing": dict(args=(1, 1, 32, 32, 8), mask=plain(lambda b, h, q, k: q < 0)),
    "constructor_causal_mask": dict(args=(2, 2, 48, 48, 16), constructor="causal_mask"),
    "constructor_causal_mask_rectangular": dict(args=(1, 1, 32, 64, (8, 16)), constructor="causal_mask"),
    "constructor_full_mask": dict(args=(1, 2, 32, 64, (16, 8)), constructor="full_mask"),
}


# ---- flex_attention --------------------------------------------------------------------------------------------------
# shape = (B, Hq, Hkv, L, S, E); block_mask = (mask(flavour), B, H, BLOCK) or None
def _alibi(score, b, h, q, k):
    return score - (h + 1) * 0.125 * (q - k)


FLEX = {
    "unmasked": dict(shape=(2, 4, 4, 8, 8, 16)),
    "gqa_causal": dict(shape=(2, 4, 2, 16, 16, 8), block_mask=(plain(lambda b, h, q, k: q >= k), 2, 4, 4), enable_gqa=True),
    "sliding_scale_half": dict(shape=(2, 4, 4, 16, 16, 16), scale=0.5,
                               block_mask=(plain(lambda b, h, q, k: (q >= k) & (q - k <= 2)), 2, 4, 4)),
    "broadcast_block_mask": dict(shape=(2, 4, 4, 16, 16, 8), block_mask=(plain(lambda b, h, q, k: (q + k) % 2 == 0), 1, 1, 4)),
    "batch_head_mask": dict(shape=(2, 4, 4, 16, 16, 8), block_mask=(plain(lambda b, h, q, k: (q >= k) & (q - k <= b + h)), 2, 4, 4)),
    "alibi_score_mod_causal": dict(shape=(1, 4, 4, 16, 16, 16), score_mod=_alibi,
                                   block_mask=(plain(lambda b, h, q, k: q >= k), 1, 4, 8)),
    "scale_zero": dict(shape=(1, 2, 2, 8, 8, 16), scale=0.0),
}


def flex_inputs(name):
    """(query, key, value, d_out) in the [B, H, L, E] layout of flex_attention."""
    B, Hq, Hkv, L, S, E = FLEX[name]["shape"]
    base = zlib.crc32(("flex/" + name).encode()) % (2 ** 31)
    return (normal((B, Hq, L, E), base), normal((B, Hkv, S, E), base + 1), normal((B, Hkv, S, E), base + 2),
            normal((B, Hq, L, E), base + 3))


# ---- storage ---------------------------------------------------------------------------------------------------------
def sample_index(key, size):
    """The flat indices that are stored for a large tensor (seeded by the entry's name)."""
    seed = zlib.crc32(key.encode())
    return np.sort(np.random.Generator(np.random.PCG64(seed)).choice(size, SAMPLE, replace=False))


def projection_vectors(key, size):
    seed = zlib.crc32(key.encode()) + 2 ** 32
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((PROJECTIONS, size))


def pack(key, x, out):
    """Adds tensor ``x`` to the dict ``out`` under ``key``: whole if small, else sample + projections."""
    x = np.asarray(x, dtype=np.float32)
    out[key + "/shape"] = np.asarray(x.shape, dtype=np.int64)
    if x.size < FULL_BELOW:
        out[key + "/full"] = x
    else:
        flat = x.reshape(-1)
        out[key + "/sample"] = flat[sample_index(key, x.size)]
        out[key + "/projections"] = projection_vectors(key, x.size) @ flat.astype(np.float64)


def compare(key, got, stored, max_tol, rms_tol):
    """Largest absolute error over the stored entries (scaled by max(1, |ref|)), after asserting the shape and that
    the projections over the whole tensor agree to ``rms_tol * sqrt(size)``."""
    got = np.asarray(got, dtype=np.float64)
    assert tuple(stored[key + "/shape"]) == got.shape, (key, got.shape)
    assert np.isfinite(got).all(), key
    if key + "/full" in stored:
        ref = stored[key + "/full"].astype(np.float64)
        err = np.abs(got - ref) / np.maximum(1.0, np.abs(ref))
        assert np.sqrt(np.mean((got - ref) ** 2)) <= rms_tol, (key, "rms")
    else:
        flat = got.reshape(-1)
        ref = stored[key + "/sample"].astype(np.float64)
        err = np.abs(flat[sample_index(key, flat.size)] - ref) / np.maximum(1.0, np.abs(ref))
        proj = projection_vectors(key, flat.size) @ flat
        gap = np.abs(proj - stored[key + "/projections"]).max()
        assert gap <= 4.0 * rms_tol * np.sqrt(flat.size), (key, "projection", gap)
    assert err.max() <= max_tol, (key, float(err.max()))
    return float(err.max())
