// Row softmax over a materialised (B*H*T, T) score matrix with the causal mask and the scale
// folded in, and its backward: the non-tiled branch of the reference model
// (src/kernels/attention.cu:147-306 of sarimahsan/transformer-cuda). HBM-bound: one warp owns one
// row, reads only the causal prefix j <= i, and finishes the row maximum, the row sum and the
// dp.p dot product with warp-shuffle reductions. Elements above the diagonal are written as zeros.
#include <cfloat>

#include "kernels.cuh"

namespace b200attn {
namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) causal_softmax_fwd_kernel(const float* __restrict__ scores,
                                                                               float* __restrict__ probs,
                                                                               long long rows, int T, float scale) {
    const int lane = threadIdx.x & 31;
    long long row = blockIdx.x * (long long)kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int i = int(row % T);  // query position: keys 0..i are visible
    const float* s = scores + row * T;
    float* p = probs + row * T;

    float mx = -FLT_MAX;
    for (int j = lane; j <= i; j += 32) mx = fmaxf(mx, s[j] * scale);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int j = lane; j <= i; j += 32) {
        float e = expf(s[j] * scale - mx);
        p[j] = e;  // same lane rewrites it below
        sum += e;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int j = lane; j <= i; j += 32) p[j] *= inv;
    for (int j = i + 1 + lane; j < T; j += 32) p[j] = 0.f;
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) causal_softmax_bwd_kernel(const float* __restrict__ dprobs,
                                                                               const float* __restrict__ probs,
                                                                               float* __restrict__ dscores,
                                                                               long long rows, int T, float scale) {
    const int lane = threadIdx.x & 31;
    long long row = blockIdx.x * (long long)kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int i = int(row % T);
    const float* dp = dprobs + row * T;
    const float* p = probs + row * T;
    float* ds = dscores + row * T;
    float dot = 0.f;
    for (int j = lane; j <= i; j += 32) dot += dp[j] * p[j];
    dot = warp_sum(dot);
    for (int j = lane; j <= i; j += 32) ds[j] = scale * p[j] * (dp[j] - dot);
    for (int j = i + 1 + lane; j < T; j += 32) ds[j] = 0.f;
}

}  // namespace

cudaError_t launch_causal_softmax_fwd(const float* scores, float* probs, long long rows, int T, float scale,
                                      cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    unsigned int blocks = (unsigned int)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    causal_softmax_fwd_kernel<<<blocks, kWarpsPerBlock * 32, 0, stream>>>(scores, probs, rows, T, scale);
    return cudaGetLastError();
}

cudaError_t launch_causal_softmax_bwd(const float* dprobs, const float* probs, float* dscores, long long rows, int T,
                                      float scale, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    unsigned int blocks = (unsigned int)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    causal_softmax_bwd_kernel<<<blocks, kWarpsPerBlock * 32, 0, stream>>>(dprobs, probs, dscores, rows, T, scale);
    return cudaGetLastError();
}

}  // namespace b200attn
