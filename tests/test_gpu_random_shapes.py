"""Seeded random shapes on the tensor-core path against the float64 dense oracle and against the
exact-FP32 SIMT kernels: ragged and rectangular lengths, odd numbers of tiles, GQA groups, both head
dimensions, every structured mask family, with the backward scratch whole, split into ranges, and absent."""
import numpy as np
import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200 import _native as nat
from jaxmodules_b200 import attention as A
from jaxmodules_b200 import masks as M
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu


def _case(seed):
    rng = np.random.Generator(np.random.PCG64(1000 + seed))
    d = int(rng.choice([64, 128]))
    Hkv = int(rng.integers(1, 4))
    G = int(rng.choice([1, 1, 2, 4]))
    B = int(rng.integers(1, 4))
    L = int(rng.integers(1, 9)) * 128 - int(rng.choice([0, 0, 1, 37, 100]))
    N = L if rng.random() < 0.6 else max(1, int(rng.integers(1, 9)) * 128 - int(rng.choice([0, 5, 64])))
    kind = str(rng.choice(["causal", "band", "segments", "window", "none"]))
    if N != L and kind in ("segments", "window"):
        kind = "band"
    kw = {}
    if kind == "causal":
        kw = dict(is_causal=True)
    elif kind == "band":
        kw = dict(mask_fn=M.sliding_window_mask(int(rng.integers(0, 300)), int(rng.integers(0, 200))))
    elif kind == "segments":
        seg = np.sort(rng.integers(0, 5, size=(B, L)), axis=1).astype(np.int32)
        kw = dict(mask_fn=M.document_mask(seg, causal=bool(rng.integers(0, 2))))
    elif kind == "window":
        kw = dict(is_causal=True, window_size=(int(rng.integers(1, 300)), 0), block_size=128)
        L = N = int(rng.integers(4, 9)) * 128  # the reference needs whole blocks and left + right <= number of blocks
    if N != L:
        kw["block_size"] = 100  # N is no multiple of it: the padding path, which takes any number of keys (jaxmodules/attention.py:426-437)
    scratch = str(rng.choice(["whole", "ranges", "none"]))
    return dict(B=B, N=N, L=L, Hq=Hkv * G, Hkv=Hkv, d=d, kind=kind, kw=kw, scratch=scratch, seed=seed)


def _run(Q, K, V, dO, **kw):
    Qc, Kc, Vc = (x.cuda().requires_grad_(True) for x in (Q, K, V))
    O = jm.masked_attention_via_map(Qc, Kc, Vc, **kw)
    O.backward(dO.cuda())
    torch.cuda.synchronize()
    return [t.float().cpu() for t in (O.detach(), Qc.grad, Kc.grad, Vc.grad)]


@pytest.mark.parametrize("forward", ["auto", "persistent", "one_item_per_cta"])
@pytest.mark.parametrize("seed", range(24))
def test_random_shape_matches_exact_kernels(seed, forward, monkeypatch):
    # both tensor-core forward kernels on every case (the library reads BMA_FWD_PERSISTENT at each call)
    if forward != "auto":
        monkeypatch.setenv("BMA_FWD_PERSISTENT", "1" if forward == "persistent" else "0")
    c = _case(seed)
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn(c["B"], c["N"], c["Hq"], c["d"], generator=g).to(torch.bfloat16)
    K, V = (torch.randn(c["B"], c["L"], c["Hkv"], c["d"], generator=g).to(torch.bfloat16) for _ in range(2))
    dO = torch.randn(c["B"], c["N"], c["Hq"], c["d"], generator=g)
    limit = A._scratch_limit
    try:   # "ranges": 45 % of what the call needs, i.e. the backward runs as three or more ranges where the units allow
        A.set_backward_scratch_limit(0 if c["scratch"] == "none" else limit, 0.45 if c["scratch"] == "ranges" else 1.0)
        got = _run(Q, K, V, dO, **c["kw"])
    finally:
        A.set_backward_scratch_limit(limit)
    want = _run(Q, K, V, dO, backend=nat.BMA_BACKEND_SIMT, **c["kw"])
    ref = ao.masked_attention_dense(Q.float().numpy(), K.float().numpy(), V.float().numpy(), dO=dO.numpy(), **c["kw"])
    for name, x in zip(("O", "dQ", "dK", "dV"), got):      # the oracle: same bounds as below
        y = torch.from_numpy(ref[name]).float()
        err = (x - y).abs()
        assert float((err / y.abs().clamp(min=1.0)).max()) <= 2e-2 and float(err.mean()) <= 2e-3 * (1.0 + float(y.abs().mean())), \
            f"{c}: {name} against the oracle: max {float(err.max()):.3e} mean {float(err.mean()):.3e}"
    for name, x, y in zip(("O", "dQ", "dK", "dV"), got, want):
        assert torch.isfinite(x).all(), f"{c}: {name} not finite"
        err = (x - y).abs()
        # bf16 tolerances: max-abs 2e-2 relative to max(1, |ref|); mean-abs 2e-3 plus the share of the bf16 rounding of the
        # outputs themselves (2^-9 of their mean size: 28 keys can collect the gradient of 250 unscaled queries each)
        assert float((err / y.abs().clamp(min=1.0)).max()) <= 2e-2 and float(err.mean()) <= 2e-3 * (1.0 + float(y.abs().mean())), \
            f"{c}: {name} max {float(err.max()):.3e} mean {float(err.mean()):.3e}"
