"""The oracle against vectors produced by the reference's own source (tests/golden/reference_vectors.npz, written by
tests/golden/make_reference_vectors.py): this is what pins the oracle's float path, and its integer path on more masks
than the reference's tests state inline.

float32: 1e-4 max-abs as for the CUDA path, in practice 1e-6.  The bfloat16 cases compare the float64 truth with a
reference that rounds its scores to bfloat16: 2e-2 max, relative to max(1, |ref|)."""
import sys
import types
from pathlib import Path

import numpy as np
import pytest
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import reference_cases as rc  # noqa: E402

from oracle import attention_oracle as ao  # noqa: E402
from oracle import block_mask_oracle as bo  # noqa: E402
from oracle.flex_oracle import flex_attention_oracle  # noqa: E402

ALL = ("O", "dQ", "dK", "dV")


@pytest.fixture(scope="module")
def vectors():
    return np.load(GOLDEN / "reference_vectors.npz")


def bf16_round(x):
    return torch.from_numpy(x).to(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("name", list(rc.ATTENTION))
def test_attention_oracle_matches_the_reference_source(vectors, name):
    Q, K, V, dO = rc.attention_inputs(name)
    bf16 = rc.ATTENTION[name].get("dtype") == "bfloat16"
    if bf16:
        Q, K, V = bf16_round(Q), bf16_round(K), bf16_round(V)
    assert str(vectors[f"attention/{name}/dtype"]) == "torch.float32"      # the reference returns float32 for every input
    kw = rc.attention_kwargs(name, "numpy")
    lead = (None,) if Q.ndim == 3 else ()
    add = (lambda x: x[None]) if Q.ndim == 3 else (lambda x: x)
    dense = ao.masked_attention_dense(add(Q), add(K), add(V), dO=add(dO), **kw)
    tol = (2e-2, 4e-3) if bf16 else (1e-4, 1e-5)
    for key in ALL:
        got = dense[key][0] if lead else dense[key]
        rc.compare(f"attention/{name}/{key}", got, vectors, *tol)
    if not bf16 and "kernel" not in kw:
        # the faithful blockwise restatement (same walk as the reference, float32) agrees as well
        port = ao.masked_attention_via_map(Q, K, V, dO=dO, **kw)
        for key, got in zip(ALL, port):
            rc.compare(f"attention/{name}/{key}", got.numpy(), vectors, 1e-4, 1e-5)


@pytest.mark.parametrize("name", list(rc.BLOCK_MASK))
def test_block_mask_oracle_is_bit_exact(vectors, name):
    case = rc.BLOCK_MASK[name]
    if "constructor" in case:
        bm = getattr(bo, case["constructor"])(*case["args"])
    else:
        bm = bo.create_block_mask(case["mask"]("numpy"), *case["args"])
    for f in ("B", "H", "Q_LEN", "KV_LEN", "Q_BLOCK_SIZE", "KV_BLOCK_SIZE"):
        assert bm[f] == int(vectors[f"block_mask/{name}/{f}"]), f
    for f in rc.BLOCK_MASK_FIELDS:
        key = f"block_mask/{name}/{f}"
        if key in vectors:
            assert bm[f].dtype == np.int32 and np.array_equal(bm[f], vectors[key]), f
    dense = bo.materialize_mask(bm).astype(np.uint8)
    assert np.array_equal(np.packbits(dense.reshape(-1)), vectors[f"block_mask/{name}/dense_packed"])


@pytest.mark.parametrize("name", list(rc.FLEX))
def test_flex_oracle_matches_the_reference_source(vectors, name):
    case = rc.FLEX[name]
    q, k, v, do = (torch.from_numpy(x) for x in rc.flex_inputs(name))
    kw = {key: case[key] for key in ("scale", "enable_gqa", "score_mod") if key in case}
    if "block_mask" in case:
        mask, b, h, block = case["block_mask"]
        d = bo.create_block_mask(mask("numpy"), b, h, case["shape"][3], case["shape"][4], block)
        t = {key: (torch.from_numpy(np.asarray(val)) if isinstance(val, np.ndarray) else val) for key, val in d.items()}
        t["mask_mod"] = mask("numpy")
        kw["block_mask"] = types.SimpleNamespace(**t)
    out = flex_attention_oracle(q, k, v, **kw)
    rc.compare(f"flex/{name}/O", np.asarray(out), vectors, 1e-4, 1e-5)


def test_argument_errors_match_the_reference(vectors):
    """The shape / block / window combinations the reference accepts are exactly those the package's host-side check
    and the oracle's blockwise port accept (240 random combinations, 128 of them valid)."""
    from jaxmodules_b200.attention import block_window
    accepted = vectors["geometry/accepted"]
    cases = rc.geometry_cases()
    assert len(cases) == len(accepted)
    for case, ok in zip(cases, accepted):
        heads_ok = case["Hq"] % case["Hkv"] == 0
        try:
            block_window(case["N"], case["L"], case["kw"].get("block_size"), case["kw"].get("window_size"))
            mine = heads_ok
        except ValueError:
            mine = False
        assert mine == bool(ok), case
        Q = torch.from_numpy(rc.normal((1, case["N"], case["Hq"], case["d"]), 1))
        K = torch.from_numpy(rc.normal((1, case["L"], case["Hkv"], case["d"]), 2))
        try:
            ao.masked_attention_via_map(Q, K, K, **case["kw"])
            port = True
        except Exception:
            port = False
        assert port == bool(ok), case
