// Placeholder until the tensor-core GEMM lands: large batches run through the
// small-M kernel in groups of tokens.
#include "common.cuh"

namespace dwim {
bool gemm_available() { return false; }
int gemm_large(dwim_b200_ctx *ctx, const WeightView &, const __half *, size_t, float *, const float *, int) {
    return fail(ctx, DWIM_B200_EINVAL, "the tensor-core GEMM is not built");
}
void gemm_release(dwim_b200_ctx *) {}
}  // namespace dwim
