"""B200-native blockwise masked attention: a drop-in for the hot path of acutkosky/jaxmodules
(``masked_attention_via_map``, ``flex_attention`` and ``create_block_mask``) on hand-written sm_100a CUDA kernels.

The compute library (libbma.so) must be built first: ``python -m jaxmodules_b200.build``.
"""
from .attention import default_kernel, masked_attention_via_map, threshold_kernel
from .block_mask import (BlockMask, create_block_mask, extract_block_size, get_dense_from_kv_blocks,
                         get_partial_block, get_sparse_kv_data_from_blocks, get_sparse_q_data_from_blocks)
from .flex import flex_attention
from .masks import and_masks, causal_mask, document_mask, full_mask, sliding_window_mask

__all__ = [
    "masked_attention_via_map", "flex_attention", "default_kernel", "threshold_kernel",
    "BlockMask", "create_block_mask", "extract_block_size", "get_partial_block",
    "get_sparse_kv_data_from_blocks", "get_sparse_q_data_from_blocks", "get_dense_from_kv_blocks",
    "causal_mask", "full_mask", "sliding_window_mask", "document_mask", "and_masks",
]
