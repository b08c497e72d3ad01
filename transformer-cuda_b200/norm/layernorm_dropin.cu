// LayerNorm forward and backward of the reference model (src/kernels/layernorm.cu of sarimahsan/transformer-cuda) as
// HBM-bound kernels for sm_100a. Same arithmetic (mean, then the variance of the centred values, rsqrtf; the
// backward's two row sums and its dx expression, layernorm.cu:52-94 and :176-207), different data movement:
//
//   * One WARP per row, the row in registers (C = 128 * k floats, k <= 8: each lane holds k float4 of x and of dout).
//     A row is read from HBM once per pass; the row sums are warp shuffles, no shared memory and no block barrier.
//     The reference gives a row a 512-thread block that reads it three times (forward) or twice plus a second
//     kernel (backward) and synchronises the block four times.
//   * The backward is ONE kernel: while a warp walks its rows (a persistent grid) every lane also accumulates
//     dgamma / dbeta of its own columns in registers; the eight warps of a CTA add their partials in a fixed order
//     through shared memory and the CTA adds the result to dgamma / dbeta with one atomic per column. The reference
//     reads dout and x a second time in a 48-CTA kernel for those sums (226 us per call at 16384 x 768, against 23 us
//     for the whole 150 MB at the HBM rate) and also finishes with atomics, so the order of the last additions is
//     as undetermined as there.
//   * Other shapes (C not a multiple of 128, C > 1024, buffers not 16-byte aligned) take generic kernels: one warp
//     per row, strided scalar accesses, the row re-read from cache for the second pass, column sums through
//     shared-memory atomics.
#include "kernels/layernorm.cuh"

#include <cuda_bf16.h>

#include <cstdint>
#include <cstdio>

// Defined by the GEMM drop-in (libb200gemm.a) when it is linked into the same program, else NULL: a BF16 twin of an FP32
// matrix the GEMMs will read, written here beside the FP32 values so that the GEMM side converts nothing (B200GEMM_TWINS=1).
extern "C" void* b200gemm_bf16_twin(const void* fp32, int rows, int cols) __attribute__((weak));

namespace {

__device__ __forceinline__ void store_twin4(__nv_bfloat16* twin_row, int i, const float4& r) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
    uint2 w;
    w.x = *reinterpret_cast<const unsigned int*>(&lo), w.y = *reinterpret_cast<const unsigned int*>(&hi);
    reinterpret_cast<uint2*>(twin_row)[i] = w;
}
__nv_bfloat16* twin_of(const float* fp32, int rows, int cols) {
    return b200gemm_bf16_twin ? static_cast<__nv_bfloat16*>(b200gemm_bf16_twin(fp32, rows, cols)) : nullptr;
}

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxVec = 8;               // register path: C = 128 * kVec, kVec <= 8
constexpr int kGenericMaxC = 12 * 1024;  // generic backward: 2 * C floats of shared memory

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float sum4(const float4& a) { return (a.x + a.y) + (a.z + a.w); }

// ------------------------------------------------------------------ forward
template <int kVec>
__global__ void __launch_bounds__(kThreads) ln_forward_reg_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                   const float* __restrict__ beta, float* __restrict__ out,
                                                                   float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                   int N, float eps, __nv_bfloat16* __restrict__ twin) {
    constexpr int C = 128 * kVec;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (row >= N) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * C);
    float4 v[kVec];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        v[j] = __ldcs(xr + lane + 32 * j);
        s += sum4(v[j]);
    }
    const float mean = warp_sum(s) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
        q += (a * a + b * b) + (c * c + d * d);
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)C + eps);
    if (lane == 0) mean_out[row] = mean, rstd_out[row] = rstd;
    float4* orow = reinterpret_cast<float4*>(out + (size_t)row * C);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = lane + 32 * j;
        const float4 g = gamma ? __ldg(reinterpret_cast<const float4*>(gamma) + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 b = beta ? __ldg(reinterpret_cast<const float4*>(beta) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 r;
        r.x = ((v[j].x - mean) * rstd) * g.x + b.x;
        r.y = ((v[j].y - mean) * rstd) * g.y + b.y;
        r.z = ((v[j].z - mean) * rstd) * g.z + b.z;
        r.w = ((v[j].w - mean) * rstd) * g.w + b.w;
        orow[i] = r;
        if (twin) store_twin4(twin + (size_t)row * C, i, r);
    }
}

__global__ void __launch_bounds__(kThreads) ln_forward_generic_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                       const float* __restrict__ beta, float* __restrict__ out,
                                                                       float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                       int N, int C, float eps) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (row >= N) return;
    const float* xr = x + (size_t)row * C;
    float s = 0.f;
    for (int i = lane; i < C; i += 32) s += xr[i];
    const float mean = warp_sum(s) / (float)C;
    float q = 0.f;
    for (int i = lane; i < C; i += 32) {
        const float a = xr[i] - mean;
        q += a * a;
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)C + eps);
    if (lane == 0) mean_out[row] = mean, rstd_out[row] = rstd;
    float* orow = out + (size_t)row * C;
    for (int i = lane; i < C; i += 32) orow[i] = ((xr[i] - mean) * rstd) * (gamma ? gamma[i] : 1.f) + (beta ? beta[i] : 0.f);
}

// ------------------------------------------------------------------ backward
// Adds the eight warps' column partials in warp order and the CTA's totals to the global sums.
template <int kVec>
__device__ __forceinline__ void flush_column_sums(const float4 (&acc)[kVec], float* smem, float* __restrict__ global_sum) {
    constexpr int C = 128 * kVec;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kVec; ++j) reinterpret_cast<float4*>(smem + warp * C)[lane + 32 * j] = acc[j];
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += kThreads) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) t += smem[w * C + c];
        atomicAdd(global_sum + c, t);
    }
}

template <int kVec>
__global__ void __launch_bounds__(kThreads, 2)
    ln_backward_reg_kernel(const float* __restrict__ dout, const float* __restrict__ x, const float* __restrict__ gamma,
                           const float* __restrict__ mean_in, const float* __restrict__ rstd_in, float* __restrict__ dx,
                           float* __restrict__ dgamma, float* __restrict__ dbeta, int N, const float* __restrict__ residual,
                           int accumulate, __nv_bfloat16* __restrict__ twin) {
    constexpr int C = 128 * kVec;
    extern __shared__ __align__(16) float smem[];  // kWarps * C floats
    const int lane = threadIdx.x & 31;
    float4 dg[kVec], db[kVec];
#pragma unroll
    for (int j = 0; j < kVec; ++j) dg[j] = db[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float inv_c = 1.0f / (float)C;

    for (int row = blockIdx.x * kWarps + (threadIdx.x >> 5); row < N; row += gridDim.x * kWarps) {
        const float4* dyr = reinterpret_cast<const float4*>(dout + (size_t)row * C);
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * C);
        float4 dy[kVec], xc[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) dy[j] = __ldcs(dyr + lane + 32 * j), xc[j] = __ldcs(xr + lane + 32 * j);
        const float mean = mean_in[row], rstd = rstd_in[row];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            const float4 g = gamma ? __ldg(reinterpret_cast<const float4*>(gamma) + lane + 32 * j) : make_float4(1.f, 1.f, 1.f, 1.f);
            xc[j].x -= mean, xc[j].y -= mean, xc[j].z -= mean, xc[j].w -= mean;  // x - mean
            db[j].x += dy[j].x, db[j].y += dy[j].y, db[j].z += dy[j].z, db[j].w += dy[j].w;
            dg[j].x += dy[j].x * (xc[j].x * rstd), dg[j].y += dy[j].y * (xc[j].y * rstd);
            dg[j].z += dy[j].z * (xc[j].z * rstd), dg[j].w += dy[j].w * (xc[j].w * rstd);
            dy[j].x *= g.x, dy[j].y *= g.y, dy[j].z *= g.z, dy[j].w *= g.w;      // dout * gamma
            s1 += sum4(dy[j]);
            s2 += (dy[j].x * xc[j].x + dy[j].y * xc[j].y) + (dy[j].z * xc[j].z + dy[j].w * xc[j].w);
        }
        s1 = warp_sum(s1), s2 = warp_sum(s2);
        const float a = inv_c * s1, b = inv_c * s2 * rstd;
        float4* dxr = reinterpret_cast<float4*>(dx + (size_t)row * C);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            const int i = lane + 32 * j;
            float4 r;
            r.x = rstd * (dy[j].x - a - (xc[j].x * rstd) * b);
            r.y = rstd * (dy[j].y - a - (xc[j].y * rstd) * b);
            r.z = rstd * (dy[j].z - a - (xc[j].z * rstd) * b);
            r.w = rstd * (dy[j].w - a - (xc[j].w * rstd) * b);
            if (residual) {
                const float4 e = __ldcs(reinterpret_cast<const float4*>(residual + (size_t)row * C) + i);
                r.x += e.x, r.y += e.y, r.z += e.z, r.w += e.w;
            }
            if (accumulate) {
                const float4 o = dxr[i];
                r.x += o.x, r.y += o.y, r.z += o.z, r.w += o.w;
            }
            dxr[i] = r;
            if (twin) store_twin4(twin + (size_t)row * C, i, r);
        }
    }
    if (dgamma) flush_column_sums<kVec>(dg, smem, dgamma);
    if (dbeta) flush_column_sums<kVec>(db, smem, dbeta);
}

__global__ void __launch_bounds__(kThreads)
    ln_backward_generic_kernel(const float* __restrict__ dout, const float* __restrict__ x, const float* __restrict__ gamma,
                               const float* __restrict__ mean_in, const float* __restrict__ rstd_in, float* __restrict__ dx,
                               float* __restrict__ dgamma, float* __restrict__ dbeta, int N, int C,
                               const float* __restrict__ residual, int accumulate) {
    extern __shared__ __align__(16) float smem[];  // column sums of this CTA: dgamma [0, C), dbeta [C, 2C)
    const int lane = threadIdx.x & 31;
    for (int c = threadIdx.x; c < 2 * C; c += kThreads) smem[c] = 0.f;
    __syncthreads();
    const float inv_c = 1.0f / (float)C;
    for (int row = blockIdx.x * kWarps + (threadIdx.x >> 5); row < N; row += gridDim.x * kWarps) {
        const float* dyr = dout + (size_t)row * C;
        const float* xr = x + (size_t)row * C;
        const float mean = mean_in[row], rstd = rstd_in[row];
        float s1 = 0.f, s2 = 0.f;
        for (int i = lane; i < C; i += 32) {
            const float dy = dyr[i], xm = xr[i] - mean, dyg = dy * (gamma ? gamma[i] : 1.f);
            s1 += dyg, s2 += dyg * xm;
            atomicAdd(smem + i, dy * (xm * rstd));
            atomicAdd(smem + C + i, dy);
        }
        s1 = warp_sum(s1), s2 = warp_sum(s2);
        const float a = inv_c * s1, b = inv_c * s2 * rstd;
        float* dxr = dx + (size_t)row * C;
        for (int i = lane; i < C; i += 32) {
            float r = rstd * (dyr[i] * (gamma ? gamma[i] : 1.f) - a - ((xr[i] - mean) * rstd) * b);
            if (residual) r += residual[(size_t)row * C + i];
            if (accumulate) r += dxr[i];
            dxr[i] = r;
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += kThreads) {
        if (dgamma) atomicAdd(dgamma + c, smem[c]);
        if (dbeta) atomicAdd(dbeta + c, smem[C + c]);
    }
}

int sm_count() {
    static const int n = [] {
        int dev = 0, v = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v;
    }();
    return n;
}

bool aligned16(std::initializer_list<const void*> ptrs) {
    uintptr_t bits = 0;
    for (const void* p : ptrs) bits |= reinterpret_cast<uintptr_t>(p);
    return (bits & 15u) == 0;
}

void report(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) fprintf(stderr, "[b200norm] %s: %s\n", what, cudaGetErrorString(e));
}

// Called after every layernorm_backward with the number of such calls since the last reset. In the reference model's
// backward pass the k-th LayerNorm backward marks the point where the gradients of another part of the model are final
// (src/model.cu:478-700: the final LayerNorm after the head, then LN2 and LN1 of each layer, last layer first), which is
// what a data-parallel trainer needs to know to start reducing them while the rest of the pass still runs.
void (*g_backward_hook)(int, cudaStream_t, void*) = nullptr;
void* g_backward_hook_user = nullptr;
int g_backward_calls = 0;
void after_backward(cudaStream_t stream) {
    const int index = ++g_backward_calls;
    if (g_backward_hook) g_backward_hook(index, stream, g_backward_hook_user);
}

template <int kVec>
void launch_backward_reg(const float* dout, const float* x, const float* gamma, const float* mean, const float* rstd, float* dx,
                         float* dgamma, float* dbeta, int N, const float* residual, bool accumulate, cudaStream_t stream) {
    constexpr int smem = kWarps * 128 * kVec * (int)sizeof(float);
    static bool attr_set = false;
    if (smem > 48 * 1024 && !attr_set) {
        cudaFuncSetAttribute(ln_backward_reg_kernel<kVec>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        attr_set = true;
    }
    const int ctas_needed = (N + kWarps - 1) / kWarps, persistent = 2 * sm_count();
    ln_backward_reg_kernel<kVec><<<ctas_needed < persistent ? ctas_needed : persistent, kThreads, smem, stream>>>(
        dout, x, gamma, mean, rstd, dx, dgamma, dbeta, N, residual, accumulate ? 1 : 0, twin_of(dx, N, 128 * kVec));
}

}  // namespace

void layernorm_forward(const float* x, const float* gamma, const float* beta, float* out, float* mean, float* rstd, int N, int C,
                       float eps, cudaStream_t stream) {
    if (N <= 0 || C <= 0) return;
    const int grid = (N + kWarps - 1) / kWarps;
    const bool reg = C % 128 == 0 && C <= 128 * kMaxVec && aligned16({x, gamma, beta, out});
    __nv_bfloat16* twin = reg ? twin_of(out, N, C) : nullptr;  // (the generic kernels write no twin: the GEMMs convert)
#define B200NORM_FWD(K) \
    case K: ln_forward_reg_kernel<K><<<grid, kThreads, 0, stream>>>(x, gamma, beta, out, mean, rstd, N, eps, twin); break;
    if (reg) {
        switch (C / 128) {
            B200NORM_FWD(1) B200NORM_FWD(2) B200NORM_FWD(3) B200NORM_FWD(4) B200NORM_FWD(5) B200NORM_FWD(6) B200NORM_FWD(7)
            B200NORM_FWD(8)
        }
    } else {
        ln_forward_generic_kernel<<<grid, kThreads, 0, stream>>>(x, gamma, beta, out, mean, rstd, N, C, eps);
    }
#undef B200NORM_FWD
    report("layernorm_forward");
}

void layernorm_backward(const float* dout, const float* x, const float* gamma, const float* mean, const float* rstd, float* dx,
                        float* dgamma, float* dbeta, int N, int C, const float* residual_add, bool accumulate,
                        cudaStream_t stream) {
    if (N <= 0 || C <= 0) return;
    const bool reg = C % 128 == 0 && C <= 128 * kMaxVec && aligned16({dout, x, gamma, dx, residual_add});
#define B200NORM_BWD(K) \
    case K: launch_backward_reg<K>(dout, x, gamma, mean, rstd, dx, dgamma, dbeta, N, residual_add, accumulate, stream); break;
    if (reg) {
        switch (C / 128) {
            B200NORM_BWD(1) B200NORM_BWD(2) B200NORM_BWD(3) B200NORM_BWD(4) B200NORM_BWD(5) B200NORM_BWD(6) B200NORM_BWD(7)
            B200NORM_BWD(8)
        }
    } else if (C <= kGenericMaxC) {
        const int smem = 2 * C * (int)sizeof(float);
        static bool attr_set = false;
        if (smem > 48 * 1024 && !attr_set) {
            cudaFuncSetAttribute(ln_backward_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kGenericMaxC * (int)sizeof(float));
            attr_set = true;
        }
        const int ctas_needed = (N + kWarps - 1) / kWarps, persistent = 2 * sm_count();
        ln_backward_generic_kernel<<<ctas_needed < persistent ? ctas_needed : persistent, kThreads, smem, stream>>>(
            dout, x, gamma, mean, rstd, dx, dgamma, dbeta, N, C, residual_add, accumulate ? 1 : 0);
    } else {
        fprintf(stderr, "[b200norm] layernorm_backward: C = %d exceeds the %d columns the generic kernel holds in shared memory\n", C,
                kGenericMaxC);
        return;
    }
#undef B200NORM_BWD
    report("layernorm_backward");
    after_backward(stream);
}

extern "C" void b200norm_set_backward_hook(void (*fn)(int, cudaStream_t, void*), void* user) {
    g_backward_hook = fn, g_backward_hook_user = user, g_backward_calls = 0;
}
extern "C" void b200norm_reset_backward_count(void) { g_backward_calls = 0; }
