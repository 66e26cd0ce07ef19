// C[M,N] = A[K,M]^T B[K,N]: the weight gradient of a linear map (gW = g^T x), a small output with a
// reduction over every node.  Both operands are contiguous along M / N.  The K range is split over
// the SMs by the stream-K scheduler (partial tiles are combined through the workspace in a fixed
// order, so the result does not depend on timing).  128x128 tiles, 32-deep K steps:
// 2.8 ms for 256x256 over K = 2.4e6 against 6.7 ms for the fp32 SIMT kernel.
#include "gemm_bf16x9.cuh"

namespace sgnn {

template <int kBands>
static int run_tn(const GemmCall &c, size_t *query)
{
    using G = Bf16x9Gemm<cutlass::layout::ColumnMajor, cutlass::layout::RowMajor, cutlass::gemm::StreamKScheduler,
                         cute::Shape<cute::_128, cute::_128, cute::_32>,
                         cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100,
                         cutlass::epilogue::FastF32NoSmemWarpSpecialized1Sm, kBands>;
    return G::run(c, query, "sgnn_gemm_f32(TN)");
}

int gemm_bf16x9_tn(const GemmCall &c, size_t *query) { return run_tn<5>(c, query); }
int gemm_bf16x6_tn(const GemmCall &c, size_t *query) { return run_tn<3>(c, query); }

}  // namespace sgnn
