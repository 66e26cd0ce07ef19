// fp32 GEMM on the sm_100a tensor cores with fp32 accuracy ("BF16x9"): every fp32 operand is split
// into three bf16 terms (a = a0 + 2^-8 a1 + 2^-16 a2) inside the kernel, the nine cross products run
// as tcgen05 bf16 MMAs with TMEM accumulators, and the partial sums are promoted into fp32 registers.
// The mainloop, TMA pipelines and epilogue are the CUTLASS 3.x sm100 "FastFP32" collectives
// (cutlass/gemm/collective/sm100_mma_warpspecialized_emulated.hpp); this header only fixes the tile
// shapes, the layouts and the leading dimensions the C ABI exposes.  Cluster shape is 1x1x1: one CTA
// per tile, plain (non-multicast) TMA loads.
#pragma once
#include "gemm_call.cuh"

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/gemm/kernel/tile_scheduler.hpp"

namespace sgnn {

template <class LayoutA, class LayoutB, class Scheduler, class MmaTile, class KernelSchedule, class EpilogueSchedule>
struct Bf16x9Gemm {
    using LayoutC = cutlass::layout::RowMajor;
    using Cluster = cute::Shape<cute::_1, cute::_1, cute::_1>;
    static constexpr int kAlign = 4;  // 16-byte rows for TMA
    using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTile, Cluster,
        cutlass::epilogue::collective::EpilogueTileAuto, float, float, float, LayoutC, kAlign, float, LayoutC, kAlign,
        EpilogueSchedule>::CollectiveOp;
    using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, float, LayoutA, kAlign, float, LayoutB, kAlign, float,
        MmaTile, Cluster,
        cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
        KernelSchedule>::CollectiveOp;
    using Kernel = cutlass::gemm::kernel::GemmUniversal<cute::Shape<int, int, int, int>, Mainloop, Epilogue, Scheduler>;
    using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;

    // Sets the one run-time entry of a (ld, 1, batch) or (1, ld, batch) stride.
    template <class Stride>
    static Stride with_ld(int64_t ld)
    {
        Stride s{};
        if constexpr (cute::is_static<decltype(cute::get<0>(s))>::value) {
            cute::get<1>(s) = ld;
        } else {
            cute::get<0>(s) = ld;
        }
        cute::get<2>(s) = 0;  // one matrix, no batch
        return s;
    }

    static int run(const GemmCall &c, size_t *query, const char *what)
    {
        using SA = typename Kernel::StrideA;
        using SB = typename Kernel::StrideB;
        using SC = typename Kernel::StrideC;
        using SD = typename Kernel::StrideD;
        cutlass::KernelHardwareInfo hw;
        int dev = 0;
        SGNN_CUDA_OK(cudaGetDevice(&dev));
        hw.device_id = dev;
        hw.sm_count = sm_count();
        typename Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                                      {c.M, c.N, c.K, 1},
                                      {c.A, with_ld<SA>(c.lda), c.B, with_ld<SB>(c.ldb)},
                                      {{1.0f, c.beta}, c.C, with_ld<SC>(c.ldc), c.C, with_ld<SD>(c.ldc)},
                                      hw};
        const size_t need = Gemm::get_workspace_size(args);
        if (query) {
            *query = need;
            return SGNN_OK;
        }
        Gemm gemm;
        SGNN_REQUIRE(gemm.can_implement(args) == cutlass::Status::kSuccess, SGNN_ERR_UNSUPPORTED,
                     "%s: shape M=%d N=%d K=%d (lda=%lld ldb=%lld ldc=%lld) is outside what the kernel implements "
                     "(extents along the contiguous dimensions must be multiples of 4)",
                     what, c.M, c.N, c.K, (long long)c.lda, (long long)c.ldb, (long long)c.ldc);
        SGNN_REQUIRE(need == 0 || (c.workspace != nullptr && c.workspace_bytes >= need), SGNN_ERR_WORKSPACE,
                     "%s: workspace of %zu bytes needed, %zu given", what, need, c.workspace_bytes);
        cutlass::Status st = gemm.initialize(args, c.workspace, c.stream);
        SGNN_REQUIRE(st == cutlass::Status::kSuccess, SGNN_ERR_CUDA, "%s: initialize failed: %s", what,
                     cutlassGetStatusString(st));
        st = gemm.run(c.stream);
        SGNN_REQUIRE(st == cutlass::Status::kSuccess, SGNN_ERR_CUDA, "%s: launch failed: %s", what,
                     cutlassGetStatusString(st));
        return SGNN_OK;
    }
};

}  // namespace sgnn
