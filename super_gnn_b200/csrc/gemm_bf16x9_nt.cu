// C[M,N] = A[M,K] B[N,K]^T: the forward of a linear map (y = x W^T) and, with the transposed weight,
// its input gradient.  Both operands are contiguous along K.  64x128 output tiles, 32-deep K steps,
// split operands staged in shared memory, result tiles written (and, for beta != 0, read) by TMA
// through shared memory: the fastest of the tile shapes and epilogues tried at M = 2.4e6, N = 256,
// K in {96, 100, 256} (3.6 ms at K = 256 against 5.6 ms for the fp32 SIMT kernel; beta = 1 costs
// 0.1 ms more, where the epilogue that stores straight from registers took three times as long).
#include "gemm_bf16x9.cuh"

namespace sgnn {

template <int kBands>
static int run_nt(const GemmCall &c, size_t *query)
{
    using G = Bf16x9Gemm<cutlass::layout::RowMajor, cutlass::layout::ColumnMajor, void,
                         cute::Shape<cute::_64, cute::_128, cute::_32>,
                         cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32SmemSm100,
                         cutlass::epilogue::TmaWarpSpecialized1Sm, kBands>;
    return G::run(c, query, "sgnn_gemm_f32(NT)");
}

int gemm_bf16x9_nt(const GemmCall &c, size_t *query) { return run_nt<5>(c, query); }
int gemm_bf16x6_nt(const GemmCall &c, size_t *query) { return run_nt<3>(c, query); }

}  // namespace sgnn
