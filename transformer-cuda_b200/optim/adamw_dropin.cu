// AdamW of the reference model (class AdamW, include/optimizer.h of sarimahsan/transformer-cuda; definitions
// src/optimizer.cu:166-249) with the same members and arithmetic and HBM-bound kernels behind it. Compiled against
// the reference's own optimizer.h and config.h (the class layout is theirs), in place of src/optimizer.cu.
//
// fused_step is the step the data-parallel harness runs after the gradient all-reduce: global L2 norm of the
// gradient, clip factor, AdamW update, gradient zeroed. The traffic that cannot be avoided is one read of the
// gradient for the norm (the clip factor is needed before the first update) and one pass that reads p, g, m, v and
// writes p, m, v, g: 32 bytes per parameter, 5.2 GB for the 163 M parameters of the GPT-2-small step. Differences
// from the reference's three launches (src/optimizer.cu:239-248):
//   * the norm is one launch: a fixed grid of 16-byte loads, per-CTA partial sums in double precision, and the last
//     CTA to finish (atomic ticket) adds the partials in index order - the reference writes 637 k block sums and
//     reduces them with ONE 256-thread block, a latency-bound walk over 2.5 MB;
//   * the update pass moves 16 bytes per thread per stream instead of 4;
//   * both are deterministic (no floating-point atomics), as the reference's are.
// The update keeps the reference's expression order (src/optimizer.cu:131-152), so results agree to rounding.
//
// When the GEMM drop-in of this repository is in the same link and its BF16 twins are on, the update pass also writes
// the new parameters as BF16 into a twin of the whole parameter buffer (2 more bytes per parameter), and the GEMMs read
// the layer weights from there instead of converting each of them twice per step.
#include "optimizer.h"

#include <cuda_bf16.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

// Resolved only when the GEMM drop-in is linked in as well (declared in its kernels/matmul.cuh); NULL result: twins off.
extern "C" void* b200gemm_bf16_twin_range(const void* fp32, long long count) __attribute__((weak));
extern "C" void b200gemm_drop_twin_range(const void* fp32) __attribute__((weak));

namespace {

__nv_bfloat16* parameter_twin(const float* params, size_t n) {
    return b200gemm_bf16_twin_range ? static_cast<__nv_bfloat16*>(b200gemm_bf16_twin_range(params, (long long)n)) : nullptr;
}

constexpr int kThreads = 256;
constexpr int kNormCtasPerSm = 8;

#define B200OPT_CHECK(call)                                                                                  \
    do {                                                                                                     \
        cudaError_t e_ = (call);                                                                             \
        if (e_ != cudaSuccess) {                                                                             \
            fprintf(stderr, "[b200opt] %s failed: %s (%s:%d)\n", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            exit(1);                                                                                         \
        }                                                                                                    \
    } while (0)

// Scratch behind AdamW::d_norm_buffer: [0] total norm (float), [1] ticket (uint), from byte 16 the per-CTA partials.
struct NormScratch {
    float* total;
    unsigned int* ticket;
    double* partials;
};
__host__ __device__ inline NormScratch norm_scratch(float* buffer) {
    return {buffer, reinterpret_cast<unsigned int*>(buffer) + 1, reinterpret_cast<double*>(buffer + 4)};
}

int norm_grid() {
    static const int sms = [] {
        int dev = 0, n = 0;
        B200OPT_CHECK(cudaGetDevice(&dev));
        B200OPT_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        return n;
    }();
    return sms * kNormCtasPerSm;
}

__device__ __forceinline__ double block_sum(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double total = 0.0;
    if (threadIdx.x == 0)
        for (int w = 0; w < kThreads / 32; ++w) total += red[w];
    return total;  // valid in thread 0
}

__global__ void __launch_bounds__(kThreads) grad_norm_kernel(const float* __restrict__ grads, size_t n, float* buffer) {
    __shared__ double red[kThreads / 32];
    __shared__ unsigned int is_last;
    const NormScratch s = norm_scratch(buffer);
    const size_t n4 = n / 4, stride = (size_t)gridDim.x * kThreads;
    const float4* g4 = reinterpret_cast<const float4*>(grads);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride) {
        const float4 g = __ldg(g4 + i);
        acc.x = fmaf(g.x, g.x, acc.x), acc.y = fmaf(g.y, g.y, acc.y);
        acc.z = fmaf(g.z, g.z, acc.z), acc.w = fmaf(g.w, g.w, acc.w);
    }
    double mine = ((double)acc.x + (double)acc.y) + ((double)acc.z + (double)acc.w);
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
        const float g = grads[n4 * 4 + threadIdx.x];
        mine += (double)g * (double)g;
    }
    const double cta = block_sum(mine, red);
    if (threadIdx.x == 0) {
        s.partials[blockIdx.x] = cta;
        __threadfence();
        is_last = atomicAdd(s.ticket, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    double part = 0.0;
    for (unsigned int i = threadIdx.x; i < gridDim.x; i += kThreads) part += __ldcg(s.partials + i);
    __syncthreads();  // red is reused
    const double total = block_sum(part, red);
    if (threadIdx.x == 0) {
        *s.total = sqrtf((float)total);
        *s.ticket = 0u;
    }
}

struct AdamArgs {
    float lr, beta1, beta2, eps, weight_decay, max_norm, bias_correction1, bias_correction2;
};

// src/optimizer.cu:131-152, same order of operations
template <bool kClip>
__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, float clip, const AdamArgs& a) {
    if (kClip) g *= clip;
    const float m_t = a.beta1 * m + (1.0f - a.beta1) * g;
    const float v_t = a.beta2 * v + (1.0f - a.beta2) * g * g;
    m = m_t, v = v_t;
    const float m_hat = m_t / a.bias_correction1, v_hat = v_t / a.bias_correction2;
    p = p - a.lr * (m_hat / (sqrtf(v_hat) + a.eps) + a.weight_decay * p);
}

// kClip: multiply the gradient by max_norm / norm when the norm exceeds max_norm (src/optimizer.cu:134-137);
// kZero: clear the gradient behind the update (src/optimizer.cu:153).
template <bool kClip, bool kZero>
__global__ void __launch_bounds__(kThreads) adamw_kernel(float* __restrict__ params, float* __restrict__ grads,
                                                         float* __restrict__ m, float* __restrict__ v,
                                                         const float* __restrict__ total_norm, size_t n, AdamArgs a,
                                                         __nv_bfloat16* __restrict__ twin) {
    float clip = 1.0f;
    if (kClip) {
        const float norm = *total_norm;
        if (norm > a.max_norm && norm > 1e-6f) clip = a.max_norm / norm;
    }
    const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x, n4 = n / 4;
    if (i < n4) {
        float4 p = reinterpret_cast<float4*>(params)[i];
        const float4 g = reinterpret_cast<const float4*>(grads)[i];
        float4 mm = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
        adam_one<kClip>(p.x, g.x, mm.x, vv.x, clip, a);
        adam_one<kClip>(p.y, g.y, mm.y, vv.y, clip, a);
        adam_one<kClip>(p.z, g.z, mm.z, vv.z, clip, a);
        adam_one<kClip>(p.w, g.w, mm.w, vv.w, clip, a);
        reinterpret_cast<float4*>(params)[i] = p;
        if (twin) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
            uint2 w;
            w.x = *reinterpret_cast<const unsigned int*>(&lo), w.y = *reinterpret_cast<const unsigned int*>(&hi);
            reinterpret_cast<uint2*>(twin)[i] = w;
        }
        reinterpret_cast<float4*>(m)[i] = mm;
        reinterpret_cast<float4*>(v)[i] = vv;
        if (kZero) reinterpret_cast<float4*>(grads)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    } else if (i - n4 < (n & 3)) {  // the last n % 4 parameters, one thread each
        const size_t j = n4 * 4 + (i - n4);
        float p = params[j], mm = m[j], vv = v[j];
        adam_one<kClip>(p, grads[j], mm, vv, clip, a);
        params[j] = p, m[j] = mm, v[j] = vv;
        if (twin) twin[j] = __float2bfloat16_rn(p);
        if (kZero) grads[j] = 0.f;
    }
}

// grads *= max_norm / norm when the norm exceeds max_norm (src/optimizer.cu:101-115)
__global__ void __launch_bounds__(kThreads) scale_grads_kernel(float* __restrict__ grads, const float* __restrict__ total_norm,
                                                               float max_norm, size_t n) {
    const float norm = *total_norm;
    if (norm <= max_norm || norm <= 1e-6f) return;
    const float scale = max_norm / norm;
    const size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x, n4 = n / 4;
    if (i < n4) {
        float4 g = reinterpret_cast<float4*>(grads)[i];
        g.x *= scale, g.y *= scale, g.z *= scale, g.w *= scale;
        reinterpret_cast<float4*>(grads)[i] = g;
    } else if (i - n4 < (n & 3)) {
        grads[n4 * 4 + (i - n4)] *= scale;
    }
}

unsigned int update_grid(size_t n) { return (unsigned int)((n / 4 + (n & 3) + kThreads - 1) / kThreads); }

}  // namespace

AdamW::AdamW(float* params, float* grads, size_t num_params, const TransformerConfig& config)
    : d_params(params), d_grads(grads), num_params(num_params), step_count(0), beta1(config.beta1), beta2(config.beta2),
      eps(config.adam_eps), weight_decay(config.weight_decay) {
    if ((reinterpret_cast<uintptr_t>(params) | reinterpret_cast<uintptr_t>(grads)) & 15u) {
        fprintf(stderr, "[b200opt] parameter and gradient buffers must be 16-byte aligned\n");
        exit(1);
    }
    B200OPT_CHECK(cudaMalloc(&d_m, num_params * sizeof(float)));
    B200OPT_CHECK(cudaMalloc(&d_v, num_params * sizeof(float)));
    const size_t scratch = 16 + sizeof(double) * (size_t)norm_grid();
    B200OPT_CHECK(cudaMalloc(&d_norm_buffer, scratch));
    B200OPT_CHECK(cudaMemset(d_norm_buffer, 0, scratch));
    reset();
}

AdamW::~AdamW() {
    // the parameters may be freed or rewritten by others once their optimizer is gone: no twin of them may outlive it
    if (b200gemm_drop_twin_range) b200gemm_drop_twin_range(d_params);
    cudaFree(d_m);
    cudaFree(d_v);
    cudaFree(d_norm_buffer);
}

void AdamW::reset() {
    B200OPT_CHECK(cudaMemset(d_m, 0, num_params * sizeof(float)));
    B200OPT_CHECK(cudaMemset(d_v, 0, num_params * sizeof(float)));
    step_count = 0;
}

void AdamW::zero_grad(cudaStream_t stream) { B200OPT_CHECK(cudaMemsetAsync(d_grads, 0, num_params * sizeof(float), stream)); }

// Returns 0 like the reference (src/optimizer.cu:193-205): the norm stays on the device.
float AdamW::clip_grad_norm(float max_norm, cudaStream_t stream) {
    grad_norm_kernel<<<norm_grid(), kThreads, 0, stream>>>(d_grads, num_params, d_norm_buffer);
    scale_grads_kernel<<<update_grid(num_params), kThreads, 0, stream>>>(d_grads, norm_scratch(d_norm_buffer).total, max_norm,
                                                                         num_params);
    B200OPT_CHECK(cudaGetLastError());
    return 0.0f;
}

void AdamW::step(float lr, cudaStream_t stream) {
    step_count++;
    const AdamArgs a{lr, beta1, beta2, eps, weight_decay, 0.f, 1.0f - powf(beta1, (float)step_count),
                     1.0f - powf(beta2, (float)step_count)};
    adamw_kernel<false, false><<<update_grid(num_params), kThreads, 0, stream>>>(d_params, d_grads, d_m, d_v, nullptr, num_params, a,
                                                                                 parameter_twin(d_params, num_params));
    B200OPT_CHECK(cudaGetLastError());
}

void AdamW::fused_step(float lr, float max_norm, cudaStream_t stream) {
    step_count++;
    const AdamArgs a{lr, beta1, beta2, eps, weight_decay, max_norm, 1.0f - powf(beta1, (float)step_count),
                     1.0f - powf(beta2, (float)step_count)};
    grad_norm_kernel<<<norm_grid(), kThreads, 0, stream>>>(d_grads, num_params, d_norm_buffer);
    adamw_kernel<true, true><<<update_grid(num_params), kThreads, 0, stream>>>(d_params, d_grads, d_m, d_v,
                                                                              norm_scratch(d_norm_buffer).total, num_params, a,
                                                                              parameter_twin(d_params, num_params));
    B200OPT_CHECK(cudaGetLastError());
}
