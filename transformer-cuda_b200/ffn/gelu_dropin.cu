// GELU launchers of the reference model (src/kernels/ffn.cu of sarimahsan/transformer-cuda) with the same arithmetic
// (gelu_compute / gelu_bwd_compute, ffn.cu:8-21, restated below) and one addition: the activations these kernels write
// are operands of the next GEMM - gelu(x + b) feeds the second FFN product and its weight gradient, dx feeds the
// backward of the first - and the GEMM drop-in multiplies in BF16. So, when that drop-in is linked into the same
// program and B200GEMM_TWINS=1, each kernel also writes a BF16 twin of its result (2 bytes per element more) and the
// GEMM side converts nothing (6 bytes per element less, twice for the forward activation). HBM-bound: 8 / 12 bytes
// per element (+2 with a twin), 16-byte accesses, one thread per four elements.
#include "kernels/ffn.cuh"

#include <cuda_bf16.h>

#include <cstdint>
#include <cstdio>

// Defined by the GEMM drop-in (libb200gemm.a) when linked into the same program, else NULL.
extern "C" void* b200gemm_bf16_twin(const void* fp32, int rows, int cols) __attribute__((weak));
extern "C" void* b200gemm_bf16_twin_flat(const void* fp32, long long count) __attribute__((weak));

namespace {

constexpr float kSqrt2OverPi = 0.7978845608028654f;
constexpr float kCoeff = 0.044715f;
constexpr int kThreads = 256;

__device__ __forceinline__ float gelu(float v) {  // ffn.cu:8-12
    const float u = kSqrt2OverPi * (v + kCoeff * v * v * v);
    const float t = tanhf(u);
    return 0.5f * v * (1.0f + t);
}
__device__ __forceinline__ float gelu_grad(float v, float dy) {  // ffn.cu:14-21
    const float u = kSqrt2OverPi * (v + kCoeff * v * v * v);
    const float t = tanhf(u);
    const float dt = 1.0f - t * t;
    const float du = kSqrt2OverPi * (1.0f + 3.0f * kCoeff * v * v);
    const float dgelu = 0.5f * (1.0f + t) + 0.5f * v * dt * du;
    return dy * dgelu;
}
__device__ __forceinline__ void store_twin4(__nv_bfloat16* twin, long long i4, const float4& r) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
    reinterpret_cast<uint2*>(twin)[i4] = make_uint2(*reinterpret_cast<const unsigned int*>(&lo), *reinterpret_cast<const unsigned int*>(&hi));
}

// y = gelu(x + bias[col]); bias may be NULL. n4 float4 groups, n_vec4 groups per row.
__global__ void __launch_bounds__(kThreads) gelu_forward_vec4_kernel(const float4* __restrict__ x, const float4* __restrict__ bias,
                                                                      float4* __restrict__ y, long long n4, int n_vec4,
                                                                      __nv_bfloat16* __restrict__ twin) {
    const long long i = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (i >= n4) return;
    float4 v = __ldcs(x + i);
    if (bias) {
        const float4 b = __ldg(bias + (i % n_vec4));
        v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
    }
    const float4 r = make_float4(gelu(v.x), gelu(v.y), gelu(v.z), gelu(v.w));
    y[i] = r;
    if (twin) store_twin4(twin, i, r);
}
__global__ void __launch_bounds__(kThreads) gelu_forward_scalar_kernel(const float* __restrict__ x, const float* __restrict__ bias,
                                                                        float* __restrict__ y, long long n, int N) {
    const long long i = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (i < n) y[i] = gelu(x[i] + (bias ? bias[i % N] : 0.f));
}

__global__ void __launch_bounds__(kThreads) gelu_backward_vec4_kernel(const float4* __restrict__ dy, const float4* __restrict__ x,
                                                                       float4* __restrict__ dx, long long n4,
                                                                       __nv_bfloat16* __restrict__ twin) {
    const long long i = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (i >= n4) return;
    const float4 g = __ldcs(dy + i), v = __ldcs(x + i);
    const float4 r = make_float4(gelu_grad(v.x, g.x), gelu_grad(v.y, g.y), gelu_grad(v.z, g.z), gelu_grad(v.w, g.w));
    dx[i] = r;
    if (twin) store_twin4(twin, i, r);
}
__global__ void __launch_bounds__(kThreads) gelu_backward_scalar_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                         float* __restrict__ dx, long long n) {
    const long long i = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (i < n) dx[i] = gelu_grad(x[i], dy[i]);
}

bool aligned16(std::initializer_list<const void*> ptrs) {
    uintptr_t bits = 0;
    for (const void* p : ptrs) bits |= reinterpret_cast<uintptr_t>(p);
    return (bits & 15u) == 0;
}
unsigned int blocks(long long n) { return (unsigned int)((n + kThreads - 1) / kThreads); }
void report(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) fprintf(stderr, "[b200ffn] %s: %s\n", what, cudaGetErrorString(e));
}

}  // namespace

void gelu_forward(const float* x, float* y, int N, cudaStream_t stream) {
    if (N <= 0) return;
    if (N % 4 == 0 && aligned16({x, y})) {
        // a twin without a row structure: usable by a GEMM whose rows and columns are multiples of 8
        __nv_bfloat16* twin = b200gemm_bf16_twin_flat ? static_cast<__nv_bfloat16*>(b200gemm_bf16_twin_flat(y, N)) : nullptr;
        gelu_forward_vec4_kernel<<<blocks(N / 4), kThreads, 0, stream>>>(reinterpret_cast<const float4*>(x), nullptr,
                                                                         reinterpret_cast<float4*>(y), N / 4, 1, twin);
    } else {
        gelu_forward_scalar_kernel<<<blocks(N), kThreads, 0, stream>>>(x, nullptr, y, N, 1);
    }
    report("gelu_forward");
}

void add_bias_gelu_forward(const float* x, const float* bias, float* y, int M, int N, cudaStream_t stream) {
    const long long total = (long long)M * N;
    if (total <= 0) return;
    if (N % 4 == 0 && aligned16({x, bias, y})) {
        // the twin's rows are N elements long only when N is a multiple of 8 (the GEMM side rounds leading dimensions up)
        __nv_bfloat16* twin = (N % 8 == 0 && b200gemm_bf16_twin) ? static_cast<__nv_bfloat16*>(b200gemm_bf16_twin(y, M, N)) : nullptr;
        gelu_forward_vec4_kernel<<<blocks(total / 4), kThreads, 0, stream>>>(reinterpret_cast<const float4*>(x),
                                                                             reinterpret_cast<const float4*>(bias),
                                                                             reinterpret_cast<float4*>(y), total / 4, N / 4, twin);
    } else {
        gelu_forward_scalar_kernel<<<blocks(total), kThreads, 0, stream>>>(x, bias, y, total, N);
    }
    report("add_bias_gelu_forward");
}

void gelu_backward(const float* dy, const float* x, float* dx, int N, cudaStream_t stream) {
    if (N <= 0) return;
    if (N % 4 == 0 && aligned16({dy, x, dx})) {
        __nv_bfloat16* twin = b200gemm_bf16_twin_flat ? static_cast<__nv_bfloat16*>(b200gemm_bf16_twin_flat(dx, N)) : nullptr;
        gelu_backward_vec4_kernel<<<blocks(N / 4), kThreads, 0, stream>>>(reinterpret_cast<const float4*>(dy),
                                                                          reinterpret_cast<const float4*>(x),
                                                                          reinterpret_cast<float4*>(dx), N / 4, twin);
    } else {
        gelu_backward_scalar_kernel<<<blocks(N), kThreads, 0, stream>>>(dy, x, dx, N);
    }
    report("gelu_backward");
}
