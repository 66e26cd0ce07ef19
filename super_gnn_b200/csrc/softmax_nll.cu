// Training loss of the node classifier and its gradient in one pass over the logits (sm_100a):
//
//     logp = log_softmax(logits + bias, dim=1)
//     loss = - sum_{r: mask[r]} logp[r, labels[r]] * inv_count
//     grad[r, c] = mask[r] * inv_count * (exp(logp[r, c]) - [c == labels[r]])
//
// The reference runs F.log_softmax inside the model (examples/graphsage/sage.py:211) and
// F.nll_loss(out[mask], labels[mask], reduction="sum") / num_train in the driver
// (examples/graphsage/train.py:41-44) and lets autograd walk back through both: a boolean
// gather, four framework kernels forward and four backward over [n, classes].  Here a warp owns a
// row; the row is read once, the gradient row written once, and the loss is summed per block and
// then over the blocks in a fixed order (bit-reproducible).
#include "common.cuh"

namespace sgnn {

constexpr int kLossThreads = 256;
constexpr int kLossMaxSlots = 8;  // columns per lane: C <= 256

__device__ __forceinline__ float warp_max_f(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum_f(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    return v;
}

template <int SLOTS>
__global__ void __launch_bounds__(kLossThreads)
softmax_nll_kernel(const float *__restrict__ logits, int64_t ld, const float *__restrict__ bias,
                   const int64_t *__restrict__ labels, const uint8_t *__restrict__ mask, float inv_count, int64_t n,
                   int C, float *__restrict__ grad, int64_t ldg, int Cg, float *__restrict__ partials)
{
    __shared__ float sred[kLossThreads / 32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t warps_total = (int64_t)gridDim.x * (kLossThreads / 32);
    float b[SLOTS];
#pragma unroll
    for (int k = 0; k < SLOTS; ++k) {
        const int c = lane + 32 * k;
        b[k] = (bias != nullptr && c < C) ? __ldg(bias + c) : 0.f;
    }
    float loss = 0.f;  // lane 0 carries the warp's sum
    for (int64_t r = (int64_t)blockIdx.x * (kLossThreads / 32) + warp; r < n; r += warps_total) {
        bool on = mask == nullptr || mask[r] != 0;
        if (on) {  // a label outside [0, C) (-1 marks an unlabelled node in the partition files; F.nll_loss skips its
                   // ignore_index the same way) takes the row out of the loss: no contribution, zero gradient
            const int64_t lab = labels[r];
            on = lab >= 0 && lab < (int64_t)C;
        }
        float *grow = grad + r * ldg;
        if (!on) {  // uniform over the warp: rows outside the mask contribute nothing
#pragma unroll
            for (int k = 0; k < SLOTS; ++k) {
                const int c = lane + 32 * k;
                if (c < Cg) grow[c] = 0.f;
            }
            continue;
        }
        float z[SLOTS];
        float mx = -INFINITY;
#pragma unroll
        for (int k = 0; k < SLOTS; ++k) {
            const int c = lane + 32 * k;
            z[k] = c < C ? ld_stream(logits + r * ld + c) + b[k] : -INFINITY;
            mx = fmaxf(mx, z[k]);
        }
        mx = warp_max_f(mx);
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < SLOTS; ++k) {
            z[k] -= mx;                                   // shifted logit (-inf beyond C)
            s += (lane + 32 * k < C) ? expf(z[k]) : 0.f;
        }
        const float lse = logf(warp_sum_f(s));
        const int label = (int)labels[r];
        float picked = 0.f;
#pragma unroll
        for (int k = 0; k < SLOTS; ++k) {
            const int c = lane + 32 * k;
            if (c < Cg) {
                float g = 0.f;
                if (c < C) {
                    const float logp = z[k] - lse;
                    g = expf(logp);
                    if (c == label) {
                        g -= 1.0f;
                        picked = logp;
                    }
                    g *= inv_count;
                }
                grow[c] = g;  // columns in [C, Cg) are padding: zero
            }
        }
        picked = warp_sum_f(picked);  // exactly one lane holds a non-zero value
        loss -= picked * inv_count;
    }
    if (lane == 0) sred[warp] = loss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float acc = 0.f;
        for (int w = 0; w < kLossThreads / 32; ++w) acc += sred[w];
        partials[blockIdx.x] = acc;
    }
}

__global__ void softmax_nll_reduce_kernel(const float *__restrict__ partials, int blocks, float *__restrict__ out)
{
    // one warp, fixed order: lane l sums partials l, l+32, ... then a shuffle tree
    float acc = 0.f;
    for (int i = threadIdx.x; i < blocks; i += 32) acc += partials[i];
    acc = warp_sum_f(acc);
    if (threadIdx.x == 0) out[0] = acc;
}

static int loss_grid() { return sm_count() * 8; }

}  // namespace sgnn

using namespace sgnn;

extern "C" SGNN_API int sgnn_softmax_nll_blocks(void) { return loss_grid(); }

extern "C" SGNN_API int sgnn_softmax_nll_loss(const float *d_logits, int64_t ld, const float *d_bias,
                                              const int64_t *d_labels, const uint8_t *d_mask, float inv_count,
                                              int64_t n, int64_t C, float *d_grad, int64_t ldg, int64_t Cg,
                                              float *d_partials, float *d_loss, void *stream)
{
    SGNN_REQUIRE(n >= 0 && C > 0, SGNN_ERR_INVALID_ARGUMENT, "softmax_nll_loss: bad size");
    SGNN_REQUIRE(C <= 32 * kLossMaxSlots, SGNN_ERR_UNSUPPORTED, "softmax_nll_loss: at most %d classes (got %lld)",
                 32 * kLossMaxSlots, (long long)C);
    SGNN_REQUIRE(Cg >= C && Cg <= 32 * kLossMaxSlots, SGNN_ERR_INVALID_ARGUMENT,
                 "softmax_nll_loss: the gradient width must be in [C, %d]", 32 * kLossMaxSlots);
    SGNN_REQUIRE(n <= (1LL << 40), SGNN_ERR_TOO_LARGE, "softmax_nll_loss: too many rows");
    SGNN_REQUIRE(d_loss != nullptr && d_partials != nullptr, SGNN_ERR_INVALID_ARGUMENT, "softmax_nll_loss: null output");
    SGNN_REQUIRE(inv_count == inv_count, SGNN_ERR_INVALID_ARGUMENT, "softmax_nll_loss: inv_count is NaN");
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        SGNN_CUDA_OK(cudaMemsetAsync(d_loss, 0, sizeof(float), s));
        return SGNN_OK;
    }
    SGNN_REQUIRE(d_logits && d_labels && d_grad, SGNN_ERR_INVALID_ARGUMENT, "softmax_nll_loss: null pointer");
    SGNN_REQUIRE(ld >= C && ldg >= Cg, SGNN_ERR_INVALID_ARGUMENT, "softmax_nll_loss: leading dimension shorter than a row");
    const int g = loss_grid();
    const int slots = (int)((Cg + 31) / 32);
#define SGNN_LOSS(SL)                                                                                                   \
    softmax_nll_kernel<SL><<<g, kLossThreads, 0, s>>>(d_logits, ld, d_bias, d_labels, d_mask, inv_count, n, (int)C,      \
                                                      d_grad, ldg, (int)Cg, d_partials)
    if (slots <= 1) SGNN_LOSS(1); else if (slots <= 2) SGNN_LOSS(2); else if (slots <= 4) SGNN_LOSS(4); else SGNN_LOSS(8);
#undef SGNN_LOSS
    SGNN_LAUNCH_OK("softmax_nll_kernel");
    softmax_nll_reduce_kernel<<<1, 32, 0, s>>>(d_partials, g, d_loss);
    SGNN_LAUNCH_OK("softmax_nll_reduce_kernel");
    return SGNN_OK;
}
