"""Writes tests/golden/reference_vectors.npz by EXECUTING THE REFERENCE'S OWN SOURCE on the cases of reference_cases.py.

jax is not installed where this library is developed, so the reference (acutkosky/jaxmodules: jaxmodules/attention.py,
jaxmodules/block_mask.py, jaxmodules/vectorize.py — imported unmodified from a checkout, never copied) runs on
tests/golden/jax_stand_in: the jax API it uses, implemented on torch CPU tensors.  What the vectors pin:

* masked_attention_via_map (attention.py:347-455) with its custom_vjp forward and backward rules (:180-345): O, dQ, dK, dV;
* create_block_mask and the BlockMask constructors (block_mask.py:167-290, 454-498): every index array, as integers;
* flex_attention (attention.py:458-692): O and the autodiff gradients.

The block walk, window clamp, padding, head mapping, running average and the structure of the backward rule are the
reference's; the floating-point primitives underneath are torch's, not XLA's, so float agreement with a real jax run is
to rounding, not to the bit.  Integer results do not depend on that.

The stand-in is itself validated by the reference's own test files (run_reference_tests_on_stand_in.py: 93 passed).

    python tests/golden/make_reference_vectors.py /path/to/jaxmodules-checkout
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE / "jax_stand_in"))
sys.path.insert(0, str(HERE))


def main(checkout: str):
    sys.path.insert(0, checkout)
    import torch
    import jaxmodules.attention as ref_attention
    import jaxmodules.block_mask as ref_block_mask
    import reference_cases as rc

    assert "jax_stand_in" in sys.modules["jax"].__file__
    out = {}

    for name in rc.ATTENTION:
        case = rc.ATTENTION[name]
        dtype = getattr(torch, case.get("dtype", "float32"))
        Q, K, V, dO = (torch.from_numpy(x).to(dtype) for x in rc.attention_inputs(name))
        Q, K, V = (x.requires_grad_(True) for x in (Q, K, V))
        O = ref_attention.masked_attention_via_map(Q, K, V, **rc.attention_kwargs(name, "torch", ref_attention))
        O.backward(dO.to(O.dtype))
        out[f"attention/{name}/dtype"] = np.asarray(str(O.dtype))
        for key, x in (("O", O), ("dQ", Q.grad), ("dK", K.grad), ("dV", V.grad)):
            rc.pack(f"attention/{name}/{key}", x.detach().float().numpy(), out)
        print("attention", name, tuple(O.shape), O.dtype)

    # which argument combinations the reference accepts (shape and window checks); the values themselves are covered above
    outcomes = []
    for case in rc.geometry_cases():
        Q = torch.from_numpy(rc.normal((1, case["N"], case["Hq"], case["d"]), 1))
        K = torch.from_numpy(rc.normal((1, case["L"], case["Hkv"], case["d"]), 2))
        try:
            ref_attention.masked_attention_via_map(Q, K, K, **case["kw"])
            outcomes.append(1)
        except Exception:
            outcomes.append(0)
    out["geometry/accepted"] = np.asarray(outcomes, dtype=np.uint8)
    print("geometry", len(outcomes), "cases,", int(sum(outcomes)), "accepted")

    for name, case in rc.BLOCK_MASK.items():
        if "constructor" in case:
            bm = getattr(ref_block_mask.BlockMask, case["constructor"])(*case["args"])
        else:
            bm = ref_block_mask.create_block_mask(case["mask"]("torch"), *case["args"])
        for f in ("B", "H", "Q_LEN", "KV_LEN", "Q_BLOCK_SIZE", "KV_BLOCK_SIZE"):
            out[f"block_mask/{name}/{f}"] = np.asarray(int(getattr(bm, f)), dtype=np.int64)
        for f in rc.BLOCK_MASK_FIELDS:
            if getattr(bm, f) is not None:          # from_kv_blocks (behind full_mask) leaves the q-side lists unset
                out[f"block_mask/{name}/{f}"] = getattr(bm, f).numpy().astype(np.int32)
        dense = bm.materialize_mask().numpy().astype(np.uint8)
        out[f"block_mask/{name}/dense_packed"] = np.packbits(dense.reshape(-1))
        print("block_mask", name, int(dense.sum()))

    for name, case in rc.FLEX.items():
        q, k, v, do = (torch.from_numpy(x) for x in rc.flex_inputs(name))
        q, k, v = (x.requires_grad_(True) for x in (q, k, v))
        kw = {key: case[key] for key in ("scale", "enable_gqa", "score_mod") if key in case}
        if "block_mask" in case:
            mask, b, h, block = case["block_mask"]
            L, S = case["shape"][3], case["shape"][4]
            kw["block_mask"] = ref_block_mask.create_block_mask(mask("torch"), b, h, L, S, block)
        o = ref_attention.flex_attention(q, k, v, **kw)
        o.backward(do)
        for key, x in (("O", o), ("dQ", q.grad), ("dK", k.grad), ("dV", v.grad)):
            rc.pack(f"flex/{name}/{key}", x.detach().numpy(), out)
        print("flex", name, tuple(o.shape))

    path = HERE / "reference_vectors.npz"
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
