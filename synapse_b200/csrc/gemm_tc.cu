// Prompt-run product on the tensor cores (placeholder until the tcgen05 kernel lands): reports UNAVAILABLE so
// that no caller can mistake a missing kernel for a result.
#include "common.cuh"

namespace syn {

uint64_t gemm_scratch_bytes(uint64_t tokens, uint64_t columns) { return align_up(tokens * columns * 2, 256); }

int32_t launch_gemm(const syn_b200_matrix *, const float *, uint64_t, uint64_t, float *, uint64_t, uint32_t, void *, uint64_t,
                    cudaStream_t)
{
    return fail(SYN_B200_UNAVAILABLE, "the tensor-core product is not part of this build");
}

}  // namespace syn
