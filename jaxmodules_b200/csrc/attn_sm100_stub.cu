// Placeholder until the tcgen05 backward kernel lands: the backward runs on the SIMT kernels.
#include "common.cuh"
namespace bma {
bool sm100_bwd_supported(const bma_attn_args&) { return false; }
int sm100_bwd(const bma_attn_args&, const bma_mask_spec&, const bma_block_lists&, void*, size_t, cudaStream_t) { return BMA_ERR_UNSUPPORTED; }
size_t sm100_bwd_workspace_bytes(const bma_attn_args&) { return 0; }
}
