// Prefill-regime multiply (M > 8): int8 tensor-core GEMM with per-block rescale.
#include "jq_common.cuh"

namespace jq {

int launch_gemm_mma(cudaStream_t, const void *, const void *, float *, int64_t, int64_t, int64_t M, int) {
    return set_error(JQ_ERR_UNSUPPORTED, "tensor-core GEMM not built yet (M = %lld)", (long long)M);
}

}  // namespace jq
