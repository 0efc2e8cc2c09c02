"""The CUDA path against vectors produced by the reference's own source (tests/golden/reference_vectors.npz, written by
tests/golden/make_reference_vectors.py on the cases of tests/golden/reference_cases.py).

float32 inputs: 1e-4 max-abs (relative to max(1, |ref|)), 1e-5 rms.  bfloat16 inputs: the reference rounds its scores to
bfloat16 and this library keeps them in float32, so the two differ by the reference's own rounding — 3e-2 max, 5e-3 rms.
Block lists: bit exact."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200.flex import flex_attention

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import reference_cases as rc  # noqa: E402

pytestmark = pytest.mark.gpu
ALL = ("O", "dQ", "dK", "dV")


@pytest.fixture(scope="module")
def vectors():
    return np.load(GOLDEN / "reference_vectors.npz")


@pytest.mark.parametrize("name", list(rc.ATTENTION))
def test_attention_matches_the_reference_source(vectors, name):
    bf16 = rc.ATTENTION[name].get("dtype") == "bfloat16"
    dtype = torch.bfloat16 if bf16 else torch.float32
    Q, K, V, dO = (torch.from_numpy(x).to(dtype).cuda() for x in rc.attention_inputs(name))
    Q, K, V = (x.requires_grad_(True) for x in (Q, K, V))
    O = jm.masked_attention_via_map(Q, K, V, **rc.attention_kwargs(name, "package"))
    assert O.dtype == torch.float32
    O.backward(dO.float())
    tol = (3e-2, 5e-3) if bf16 else (1e-4, 1e-5)
    for key, got in zip(ALL, (O, Q.grad, K.grad, V.grad)):
        rc.compare(f"attention/{name}/{key}", got.detach().float().cpu().numpy(), vectors, *tol)


@pytest.mark.parametrize("name", list(rc.BLOCK_MASK))
def test_block_lists_are_bit_exact(vectors, name):
    case = rc.BLOCK_MASK[name]
    if "constructor" in case:
        bm = getattr(jm.BlockMask, case["constructor"])(*case["args"], device="cuda")
    else:
        bm = jm.create_block_mask(case["mask"]("package"), *case["args"], device="cuda")
    for f in ("B", "H", "Q_LEN", "KV_LEN", "Q_BLOCK_SIZE", "KV_BLOCK_SIZE"):
        assert getattr(bm, f) == int(vectors[f"block_mask/{name}/{f}"]), f
    for f in rc.BLOCK_MASK_FIELDS:
        key = f"block_mask/{name}/{f}"
        if key in vectors and getattr(bm, f) is not None:
            got = getattr(bm, f).cpu().numpy()
            assert got.dtype == np.int32 and np.array_equal(got, vectors[key]), f
    dense = bm.materialize_mask().cpu().numpy().astype(np.uint8)
    assert np.array_equal(np.packbits(dense.reshape(-1)), vectors[f"block_mask/{name}/dense_packed"])


@pytest.mark.parametrize("name", list(rc.FLEX))
def test_flex_attention_matches_the_reference_source(vectors, name):
    case = rc.FLEX[name]
    q, k, v, do = (torch.from_numpy(x).cuda() for x in rc.flex_inputs(name))
    q, k, v = (x.requires_grad_(True) for x in (q, k, v))
    kw = {key: case[key] for key in ("scale", "enable_gqa", "score_mod") if key in case}
    if "block_mask" in case:
        mask, b, h, block = case["block_mask"]
        kw["block_mask"] = jm.create_block_mask(mask("package"), b, h, case["shape"][3], case["shape"][4], block, device="cuda")
    out = flex_attention(q, k, v, **kw)
    out.backward(do)
    for key, got in zip(ALL, (out, q.grad, k.grad, v.grad)):
        rc.compare(f"flex/{name}/{key}", got.detach().cpu().numpy(), vectors, 1e-4, 1e-5)
