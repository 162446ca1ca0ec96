// XQ8 matrix-vector kernels for Q8_0 weights (planar repack and file layout).
#include "matvec_xq8.cuh"

namespace syn {
namespace mv {
cudaError_t launch_xq8_q8_0(const MatvecArgs &a, const WeightView *views, cudaStream_t stream)
{
    const uint64_t K = a.matrix->columns;
    return a.matrix->layout == Layout::Planar ? launch_format<Q8PlanarXq8>(a, views, K / 16, K / 32, stream)
                                              : launch_format<Q8NaturalXq8>(a, views, K / 32, K / 32, stream);
}
}  // namespace mv
}  // namespace syn
