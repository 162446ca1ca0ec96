// XQ8 matrix-vector kernels for Q4_K weights (file layout; its 144-byte blocks are 16-byte aligned).
#include "matvec_xq8.cuh"

namespace syn {
namespace mv {
cudaError_t launch_xq8_q4_k(const MatvecArgs &a, const WeightView *views, cudaStream_t stream)
{
    const uint64_t K = a.matrix->columns;
    return launch_format<Q4KXq8>(a, views, K / 128, K / 32, stream);
}
}  // namespace mv
}  // namespace syn
