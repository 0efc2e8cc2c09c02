"""Writes tests/golden/block_mask_known_answers.json.

The reference (acutkosky/jaxmodules) cannot be imported on these machines (JAX is not
installed), so the fixtures are the literal known-answer arrays that the reference's own test
file states inline, transcribed with their location.  Each case names the lines of
tests/test_block_mask.py it was read from.  Run from the repository root:

    python tests/golden/make_block_mask_known_answers.py
"""
import json
from pathlib import Path

CAUSAL_8 = [[1 if q >= k else 0 for k in range(8)] for q in range(8)]

CASES = {
    # tests/test_block_mask.py:15-51 — create_block_mask(q>=k, B=2,H=2,L=8, BLOCK=4).materialize_mask()
    "create_causal_8x8_block4": {
        "source": "tests/test_block_mask.py:15-51",
        "B": 2, "H": 2, "Q_LEN": 8, "KV_LEN": 8, "BLOCK_SIZE": 4, "mask": "causal",
        "dense_mask_bh": CAUSAL_8,
    },
    # tests/test_block_mask.py:54-72 — (q+k)%3==0, B=H=1, L=8, BLOCK=4; dense mask equals the predicate
    "create_mod3_8x8_block4": {
        "source": "tests/test_block_mask.py:54-72",
        "B": 1, "H": 1, "Q_LEN": 8, "KV_LEN": 8, "BLOCK_SIZE": 4, "mask": "mod3",
        "dense_mask_bh": [[1 if (q + k) % 3 == 0 else 0 for k in range(8)] for q in range(8)],
    },
    # tests/test_block_mask.py:75-113 — from_kv_blocks with explicit seq_lengths
    "from_kv_blocks_banded": {
        "source": "tests/test_block_mask.py:75-113",
        "BLOCK_SIZE": 2, "seq_lengths": [8, 8],
        "kv_num_blocks": [[[2, 2, 2, 2]]],
        "kv_indices": [[[[0, 1], [1, 2], [2, 3], [3, 4]]]],
        "full_kv_num_blocks": [[[0, 0]]],
        "full_kv_indices": [[[[0, 0], [0, 0]]]],
        "mask": "block_band2",
        "dense_mask_bh": [[1 if (k // 2 >= q // 2) and (k // 2 < q // 2 + 2) else 0 for k in range(8)] for q in range(8)],
    },
    # tests/test_block_mask.py:116-169 — from_kv_blocks without seq_lengths: inferred lengths
    "from_kv_blocks_inferred": {
        "source": "tests/test_block_mask.py:116-169",
        "BLOCK_SIZE": 2,
        "kv_num_blocks": [[[1, 2, 1]]],
        "kv_indices": [[[[0, 3], [1, 2], [3, 3]]]],
        "full_kv_num_blocks": [[[1, 0, 1]]],
        "full_kv_indices": [[[[2, 0], [0, 0], [1, 0]]]],
        "mask": "parity",
        "expected_Q_LEN": 6, "expected_KV_LEN": 8,
    },
    # tests/test_block_mask.py:172-185 — get_partial_block((q+k)%2==0, block (0,0), 4x4)
    "get_partial_block_checkerboard": {
        "source": "tests/test_block_mask.py:172-185",
        "mask": "parity", "Q_BLOCK_SIZE": 4, "KV_BLOCK_SIZE": 4,
        "expected": [[1, 0, 1, 0], [0, 1, 0, 1], [1, 0, 1, 0], [0, 1, 0, 1]],
    },
    # tests/test_block_mask.py:188-228 — get_sparse_kv_data_from_blocks; indices compared on the valid prefix only
    "sparse_kv": {
        "source": "tests/test_block_mask.py:188-228",
        "blocks": [[[[1, 0], [1, 1]]]],
        "expected_num_blocks": [[[1, 2]]],
        "expected_indices": [[[[0, 2], [0, 1]]]],
        "relevant": [[True, False], [True, True]],
    },
    # tests/test_block_mask.py:231-252 — get_sparse_q_data_from_blocks
    "sparse_q": {
        "source": "tests/test_block_mask.py:231-252",
        "blocks": [[[[1, 0], [1, 1]]]],
        "expected_num_blocks": [[[2, 1]]],
        "expected_indices": [[[[0, 1], [1, 2]]]],
        "relevant": [[True, True], [True, False]],
    },
    # tests/test_block_mask.py:255-272 — get_dense_from_kv_blocks
    "dense_from_kv": {
        "source": "tests/test_block_mask.py:255-272",
        "NUM_Q_BLOCKS": 2, "NUM_KV_BLOCKS": 2,
        "kv_num_blocks": [[[1, 2]]],
        "kv_indices": [[[[0, 0], [0, 1]]]],
        "expected": [[[[1, 0], [1, 1]]]],
    },
    # tests/test_block_mask.py:275-303 — BlockMask.causal_mask(2,2,8,8,4).materialize_mask()
    "classmethod_causal": {
        "source": "tests/test_block_mask.py:275-303",
        "B": 2, "H": 2, "Q_LEN": 8, "KV_LEN": 8, "BLOCK_SIZE": 4, "dense_mask_bh": CAUSAL_8,
    },
    # tests/test_block_mask.py:306-323 — BlockMask.full_mask(2,2,8,8,4).materialize_mask() is all ones
    "classmethod_full": {
        "source": "tests/test_block_mask.py:306-323",
        "B": 2, "H": 2, "Q_LEN": 8, "KV_LEN": 8, "BLOCK_SIZE": 4,
        "dense_mask_bh": [[1] * 8 for _ in range(8)],
    },
}

if __name__ == "__main__":
    out = Path(__file__).with_name("block_mask_known_answers.json")
    out.write_text(json.dumps(CASES, indent=1))
    print("wrote", out)
