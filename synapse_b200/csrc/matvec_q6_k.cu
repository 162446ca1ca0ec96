// XQ8 matrix-vector kernels for Q6_K weights (planar repack and file layout).
#include "matvec_xq8.cuh"

namespace syn {
namespace mv {
cudaError_t launch_xq8_q6_k(const MatvecArgs &a, const WeightView *views, cudaStream_t stream)
{
    const uint64_t K = a.matrix->columns;
    return a.matrix->layout == Layout::Planar ? launch_format<Q6KPlanarXq8>(a, views, K / 64, K / 16, stream)
                                              : launch_format<Q6KNaturalXq8>(a, views, K / 64, K / 16, stream);
}
}  // namespace mv
}  // namespace syn
