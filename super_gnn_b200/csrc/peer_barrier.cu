// Barrier among the ranks of the one-sided boundary exchange, with a bounded wait that ends in a status
// word instead of a trap.
//
// Every rank owns an array of `world` 32-bit flags that all peers map; rank r announces that it reached
// barrier number `epoch` by storing `epoch` into flag r of every peer's array and then waits until each
// of its own flags holds `epoch` or a later number.  Epochs only grow, so a flag never has to be reset
// and a peer that runs ahead into the next barrier cannot be missed.  A wait that lasts longer than the
// limit gives up: the kernel writes the epoch into status[p] for the peer p it waited for and returns, so
// the context stays usable and the host learns from the status words (pinned host memory that the device
// writes directly) which peer did not arrive.  Plain loads and stores on peer memory only.
#include "common.cuh"

namespace sgnn {

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__global__ void peer_barrier_kernel(const int64_t *__restrict__ flag_ptrs, int rank, int world, uint32_t epoch,
                                    unsigned long long limit_ns, uint32_t *status)
{
    const int p = threadIdx.x;
    if (p >= world || p == rank) return;
    // Release: what this GPU wrote before the barrier (earlier kernels of the stream, stores into peer
    // memory included) is visible system-wide before the flag is.
    __threadfence_system();
    uint32_t *theirs = reinterpret_cast<uint32_t *>(flag_ptrs[p]) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const uint32_t *mine = reinterpret_cast<const uint32_t *>(flag_ptrs[rank]) + p;
    const unsigned long long t0 = global_ns();
    // Two bounds: elapsed time, and an iteration count (every iteration sleeps about 100 ns) in case the
    // timer does not advance.
    const unsigned long long max_iterations = limit_ns / 50 + 1024;
    for (unsigned long long it = 0; it < max_iterations; ++it) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - epoch) >= 0) return;
        if (global_ns() - t0 > limit_ns) break;
        __nanosleep(100);
    }
    status[p] = epoch;  // gave up on peer p at this barrier
    __threadfence_system();
}

}  // namespace sgnn

using namespace sgnn;

extern "C" SGNN_API int sgnn_peer_barrier(const int64_t *d_flag_ptrs, int rank, int world, uint32_t epoch,
                                          int64_t timeout_us, uint32_t *status, void *stream)
{
    SGNN_REQUIRE(d_flag_ptrs != nullptr && status != nullptr, SGNN_ERR_INVALID_ARGUMENT, "sgnn_peer_barrier: null pointer");
    SGNN_REQUIRE(world >= 1 && world <= SGNN_PEER_BARRIER_MAX_RANKS, SGNN_ERR_TOO_LARGE,
                 "sgnn_peer_barrier: world must be in [1, %d]", SGNN_PEER_BARRIER_MAX_RANKS);
    SGNN_REQUIRE(rank >= 0 && rank < world, SGNN_ERR_INVALID_ARGUMENT, "sgnn_peer_barrier: rank outside [0, world)");
    SGNN_REQUIRE(epoch != 0, SGNN_ERR_INVALID_ARGUMENT, "sgnn_peer_barrier: epoch 0 is the initial value of the flags");
    SGNN_REQUIRE(timeout_us > 0 && timeout_us <= 600ll * 1000 * 1000, SGNN_ERR_INVALID_ARGUMENT,
                 "sgnn_peer_barrier: the wait limit must be in (0, 600 s]");
    if (world == 1) return SGNN_OK;
    peer_barrier_kernel<<<1, SGNN_PEER_BARRIER_MAX_RANKS, 0, (cudaStream_t)stream>>>(
        d_flag_ptrs, rank, world, epoch, (unsigned long long)timeout_us * 1000ull, status);
    SGNN_LAUNCH_OK("peer_barrier_kernel");
    return SGNN_OK;
}
