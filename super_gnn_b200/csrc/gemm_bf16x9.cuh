// fp32 GEMM on the sm_100a tensor cores with fp32 accuracy ("BF16x9"): every fp32 operand is split
// into three bf16 terms (a = a0 + 2^-8 a1 + 2^-16 a2) inside the kernel, the nine cross products run
// as tcgen05 bf16 MMAs with TMEM accumulators, and the partial sums are promoted into fp32 registers.
// The mainloop, TMA pipelines and epilogue are the CUTLASS 3.x sm100 "FastFP32" collectives
// (cutlass/gemm/collective/sm100_mma_warpspecialized_emulated.hpp); this header only fixes the tile
// shapes, the layouts, the leading dimensions the C ABI exposes and how many of the nine cross products
// are computed.  Cluster shape is 1x1x1: one CTA per tile, plain (non-multicast) TMA loads.
//
// The nine products a_i b_j fall into five bands by weight 2^-8(i+j).  kBands = 5 computes all nine;
// kBands = 3 leaves out a1 b2, a2 b1 (2^-24 of the leading product) and a2 b2 (2^-32): six MMAs per
// K step, a per-product error of at most 2^-23 relative, the same order as the rounding of one fp32
// multiply-add.
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

// The mainloop collective `Op` the CUTLASS builder produced, with another number of bands (the builder
// fixes it at five).
template <class Op, int kBands>
struct WithBands;
template <int L2T, int T2M, int SCH, int ACC, int NB, int SF, int API, class Cl, class AccAtom, class Arch, class Tile,
          class SA, class SB, class TM, class GA, class SLA, class CA, class TA, class GB, class SLB, class CB, class TB,
          int kBands>
struct WithBands<cutlass::gemm::collective::CollectiveMma<
                     cutlass::gemm::MainloopSm100TmaUmmaWarpSpecializedFastF32<L2T, T2M, SCH, ACC, NB, SF, API, Cl, AccAtom, Arch>,
                     Tile, float, SA, float, SB, TM, GA, SLA, CA, TA, GB, SLB, CB, TB>,
                 kBands> {
    using type = cutlass::gemm::collective::CollectiveMma<
        cutlass::gemm::MainloopSm100TmaUmmaWarpSpecializedFastF32<L2T, T2M, SCH, ACC, kBands, SF, API, Cl, AccAtom, Arch>, Tile,
        float, SA, float, SB, TM, GA, SLA, CA, TA, GB, SLB, CB, TB>;
};

template <class LayoutA, class LayoutB, class Scheduler, class MmaTile, class KernelSchedule, class EpilogueSchedule,
          int kBands = 5>
struct Bf16x9Gemm {
    using LayoutC = cutlass::layout::RowMajor;
    using Cluster = cute::Shape<cute::_1, cute::_1, cute::_1>;
    static constexpr int kAlign = 4;  // 16-byte rows for TMA
    using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTile, Cluster,
        cutlass::epilogue::collective::EpilogueTileAuto, float, float, float, LayoutC, kAlign, float, LayoutC, kAlign,
        EpilogueSchedule>::CollectiveOp;
    using BuilderMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, float, LayoutA, kAlign, float, LayoutB, kAlign, float,
        MmaTile, Cluster,
        cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
        KernelSchedule>::CollectiveOp;
    using Mainloop = typename WithBands<BuilderMainloop, kBands>::type;
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
