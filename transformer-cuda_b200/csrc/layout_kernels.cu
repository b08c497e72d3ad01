// HBM-bound data movement around the attention core: QKV split-transpose and its inverse,
// head merge and its inverse (each optionally fused with the FP32<->BF16 conversion), the
// FP32->BF16 staging copy, and the counter-based N(0,1) generator used for synthetic inputs.
//
// All vector paths move 16 bytes per thread per access and keep a warp's accesses contiguous on
// the side that is contiguous in memory (the (B,T,C)-shaped tensor), with >= d*sizeof(T)-byte runs
// on the head-major side. They replace the kernels of src/kernels/attention.cu:24-143 and :308-379
// of sarimahsan/transformer-cuda (same index maps, new code).
#include "kernels.cuh"

namespace b200attn {
namespace {

constexpr int kThreads = 256;

template <typename T, int VEC>
struct Pack;
template <>
struct Pack<float, 4> {
    using type = float4;
};
template <>
struct Pack<float, 1> {
    using type = float;
};
template <>
struct Pack<__nv_bfloat16, 8> {
    using type = uint4;
};
template <>
struct Pack<__nv_bfloat16, 1> {
    using type = __nv_bfloat16;
};

// Load VEC consecutive elements as FP32.
template <int VEC>
__device__ __forceinline__ void load_as_f32(const float* p, float (&r)[VEC]) {
    if constexpr (VEC == 1) {
        r[0] = __ldg(p);
    } else {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            float4 v = __ldg(reinterpret_cast<const float4*>(p + i));
            r[i] = v.x, r[i + 1] = v.y, r[i + 2] = v.z, r[i + 3] = v.w;
        }
    }
}
template <int VEC>
__device__ __forceinline__ void load_as_f32(const __nv_bfloat16* p, float (&r)[VEC]) {
    if constexpr (VEC == 1) {
        r[0] = __bfloat162float(*p);
    } else {
#pragma unroll
        for (int i = 0; i < VEC; i += 8) {
            uint4 v = __ldg(reinterpret_cast<const uint4*>(p + i));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                r[i + 2 * j] = __uint_as_float(w[j] << 16);
                r[i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
        }
    }
}
template <int VEC>
__device__ __forceinline__ void store_from_f32(float* p, const float (&r)[VEC]) {
    if constexpr (VEC == 1) {
        *p = r[0];
    } else {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    }
}
template <int VEC>
__device__ __forceinline__ void store_from_f32(__nv_bfloat16* p, const float (&r)[VEC]) {
    if constexpr (VEC == 1) {
        *p = __float2bfloat16_rn(r[0]);
    } else if constexpr (VEC == 4) {  // one 8-byte store (p is 8-byte aligned)
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    } else {
        static_assert(VEC % 8 == 0, "BF16 stores move 1, 4 or a multiple of 8 elements");
#pragma unroll
        for (int i = 0; i < VEC; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(r[i + 2 * j], r[i + 2 * j + 1]);
                w[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(p + i) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

// One thread moves VEC elements of each of q, k, v. Thread order follows the (B,T,C) side.
template <typename TOut, int VEC>
__global__ void __launch_bounds__(kThreads) qkv_split_kernel(const float* __restrict__ qkv, TOut* __restrict__ q,
                                                            TOut* __restrict__ k, TOut* __restrict__ v, int T, int H,
                                                            int d, long long groups) {
    long long g = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (g >= groups) return;
    const int dv = d / VEC;
    int e = int(g % dv) * VEC;
    long long r = g / dv;
    int h = int(r % H);
    r /= H;
    int t = int(r % T);
    long long b = r / T;
    const long long C = (long long)H * d;
    const float* src = qkv + (b * T + t) * 3 * C + (long long)h * d + e;
    long long dst = ((b * H + h) * T + t) * d + e;
    float a[VEC];
    load_as_f32<VEC>(src, a);
    store_from_f32<VEC>(q + dst, a);
    load_as_f32<VEC>(src + C, a);
    store_from_f32<VEC>(k + dst, a);
    load_as_f32<VEC>(src + 2 * C, a);
    store_from_f32<VEC>(v + dst, a);
}

// The FP32 split with BF16 copies of q, k, v written in the same pass (8 elements per thread and tensor): what the
// FP32 launch API in BF16 math mode would otherwise produce with three separate conversion passes.
__global__ void __launch_bounds__(kThreads) qkv_split_dual_kernel(const float* __restrict__ qkv, float* __restrict__ q,
                                                                 float* __restrict__ k, float* __restrict__ v,
                                                                 __nv_bfloat16* __restrict__ qb, __nv_bfloat16* __restrict__ kb,
                                                                 __nv_bfloat16* __restrict__ vb, int T, int H, int d,
                                                                 long long groups) {
    long long g = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (g >= groups) return;
    const int dv = d / 8;
    int e = int(g % dv) * 8;
    long long r = g / dv;
    int h = int(r % H);
    r /= H;
    int t = int(r % T);
    long long b = r / T;
    const long long C = (long long)H * d;
    const float* src = qkv + (b * T + t) * 3 * C + (long long)h * d + e;
    long long dst = ((b * H + h) * T + t) * d + e;
    float a[8];
    load_as_f32<8>(src, a);
    store_from_f32<8>(q + dst, a);
    store_from_f32<8>(qb + dst, a);
    load_as_f32<8>(src + C, a);
    store_from_f32<8>(k + dst, a);
    store_from_f32<8>(kb + dst, a);
    load_as_f32<8>(src + 2 * C, a);
    store_from_f32<8>(v + dst, a);
    store_from_f32<8>(vb + dst, a);
}
// (B,T,H*d) FP32 -> (B,H,T,d) FP32 and BF16 in one pass.
__global__ void __launch_bounds__(kThreads) split_heads_dual_kernel(const float* __restrict__ merged_in, float* __restrict__ head_out,
                                                                   __nv_bfloat16* __restrict__ head_out_bf16, int T, int H, int d,
                                                                   long long groups) {
    long long g = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (g >= groups) return;
    const int dv = d / 8;
    int e = int(g % dv) * 8;
    long long r = g / dv;
    int h = int(r % H);
    r /= H;
    int t = int(r % T);
    long long b = r / T;
    float a[8];
    load_as_f32<8>(merged_in + ((b * T + t) * H + h) * d + e, a);
    const long long head = ((b * H + h) * T + t) * d + e;
    store_from_f32<8>(head_out + head, a);
    store_from_f32<8>(head_out_bf16 + head, a);
}

template <typename TIn, int VEC>
__global__ void __launch_bounds__(kThreads) qkv_merge_grad_kernel(const TIn* __restrict__ dq, const TIn* __restrict__ dk,
                                                                 const TIn* __restrict__ dv, float* __restrict__ dqkv,
                                                                 int T, int H, int d, long long groups,
                                                                 __nv_bfloat16* __restrict__ twin, int twin_ld) {
    long long g = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (g >= groups) return;
    const int dvv = d / VEC;
    int e = int(g % dvv) * VEC;
    long long r = g / dvv;
    int h = int(r % H);
    r /= H;
    int t = int(r % T);
    long long b = r / T;
    const long long C = (long long)H * d;
    float* dst = dqkv + (b * T + t) * 3 * C + (long long)h * d + e;
    long long src = ((b * H + h) * T + t) * d + e;
    // optional BF16 twin of dqkv (rows of twin_ld elements) for the GEMMs that read it next
    __nv_bfloat16* tw = twin ? twin + (b * T + t) * twin_ld + (long long)h * d + e : nullptr;
    float a[VEC];
    load_as_f32<VEC>(dq + src, a);
    store_from_f32<VEC>(dst, a);
    if (tw) store_from_f32<VEC>(tw, a);
    load_as_f32<VEC>(dk + src, a);
    store_from_f32<VEC>(dst + C, a);
    if (tw) store_from_f32<VEC>(tw + C, a);
    load_as_f32<VEC>(dv + src, a);
    store_from_f32<VEC>(dst + 2 * C, a);
    if (tw) store_from_f32<VEC>(tw + 2 * C, a);
}

// (B,H,T,d) <-> (B,T,H*d); TO_MERGED selects the direction. Thread order follows (B,T,H*d).
template <typename THead, int VEC, bool TO_MERGED>
__global__ void __launch_bounds__(kThreads) head_transpose_kernel(const THead* __restrict__ head_in,
                                                                 THead* __restrict__ head_out,
                                                                 const float* __restrict__ merged_in,
                                                                 float* __restrict__ merged_out, int T, int H, int d,
                                                                 long long groups, __nv_bfloat16* __restrict__ twin = nullptr,
                                                                 int twin_ld = 0) {
    long long g = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (g >= groups) return;
    const int dv = d / VEC;
    int e = int(g % dv) * VEC;
    long long r = g / dv;
    int h = int(r % H);
    r /= H;
    int t = int(r % T);
    long long b = r / T;
    long long merged = ((b * T + t) * H + h) * d + e;
    long long head = ((b * H + h) * T + t) * d + e;
    float a[VEC];
    if constexpr (TO_MERGED) {
        load_as_f32<VEC>(head_in + head, a);
        store_from_f32<VEC>(merged_out + merged, a);
        if (twin) store_from_f32<VEC>(twin + (b * T + t) * twin_ld + (long long)h * d + e, a);  // BF16 twin of the merged rows
    } else {
        load_as_f32<VEC>(merged_in + merged, a);
        store_from_f32<VEC>(head_out + head, a);
    }
}

__global__ void __launch_bounds__(kThreads) f32_to_bf16_kernel(const float* __restrict__ src,
                                                              __nv_bfloat16* __restrict__ dst, long long n8,
                                                              long long n, float scale) {
    // the last kernel of the BF16 backward chain: launched with programmatic serialisation (see launch_pdl)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    long long g = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (g < n8) {
        float a[8];
        load_as_f32<8>(src + g * 8, a);
#pragma unroll
        for (int x = 0; x < 8; ++x) a[x] *= scale;  // exact no-op for scale = 1
        store_from_f32<8>(dst + g * 8, a);
    } else {
        long long i = n8 * 8 + (g - n8);
        if (i < n) dst[i] = __float2bfloat16_rn(src[i] * scale);
    }
}

// splitmix64 finaliser: a bijective mix of the 64-bit counter.
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// Sample number `idx` of stream `seed`: Box-Muller on two 24-bit uniforms cut from one 64-bit hash.
__device__ __forceinline__ float normal_at(unsigned long long seed, unsigned long long idx) {
    unsigned long long h = mix64(seed * 0xD1342543DE82EF95ull + idx);
    float u1 = (float((h >> 40) & 0xFFFFFFull) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
    float u2 = float((h >> 8) & 0xFFFFFFull) * (1.0f / 16777216.0f);           // [0, 1)
    float rad = sqrtf(-2.0f * logf(u1));
    return rad * cospif(2.0f * u2);
}
template <typename T>
__global__ void __launch_bounds__(kThreads) fill_normal_kernel(T* __restrict__ dst, long long n,
                                                              unsigned long long seed, long long offset) {
    long long i = blockIdx.x * (long long)kThreads + threadIdx.x;
    if (i >= n) return;
    float x = normal_at(seed, (unsigned long long)(offset + i));
    if constexpr (sizeof(T) == 2) {
        dst[i] = __float2bfloat16_rn(x);
    } else {
        dst[i] = x;
    }
}

inline unsigned int blocks_for(long long work) { return (unsigned int)((work + kThreads - 1) / kThreads); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

template <typename TOut>
cudaError_t launch_qkv_split(const float* qkv, TOut* q, TOut* k, TOut* v, int B, int T, int H, int d,
                             cudaStream_t stream) {
    constexpr int VEC = sizeof(TOut) == 2 ? 8 : 4;
    long long n = (long long)B * T * H * d;
    if (n == 0) return cudaSuccess;
    bool vec_ok = (d % VEC == 0) && aligned16(qkv) && aligned16(q) && aligned16(k) && aligned16(v);
    if (vec_ok) {
        long long groups = n / VEC;
        qkv_split_kernel<TOut, VEC><<<blocks_for(groups), kThreads, 0, stream>>>(qkv, q, k, v, T, H, d, groups);
    } else {
        qkv_split_kernel<TOut, 1><<<blocks_for(n), kThreads, 0, stream>>>(qkv, q, k, v, T, H, d, n);
    }
    return cudaGetLastError();
}
template cudaError_t launch_qkv_split<float>(const float*, float*, float*, float*, int, int, int, int, cudaStream_t);
template cudaError_t launch_qkv_split<__nv_bfloat16>(const float*, __nv_bfloat16*, __nv_bfloat16*, __nv_bfloat16*, int,
                                                    int, int, int, cudaStream_t);

template <typename TIn>
cudaError_t launch_qkv_merge_grad(const TIn* dq, const TIn* dk, const TIn* dv, float* dqkv, int B, int T, int H, int d,
                                  cudaStream_t stream, __nv_bfloat16* twin) {
    constexpr int VEC = sizeof(TIn) == 2 ? 8 : 4;
    long long n = (long long)B * T * H * d;
    if (n == 0) return cudaSuccess;
    bool vec_ok = (d % VEC == 0) && aligned16(dqkv) && aligned16(dq) && aligned16(dk) && aligned16(dv);
    const int twin_ld = (3 * H * d + 7) / 8 * 8;  // the layout the GEMM side expects: leading dimension rounded up to 8
    if (vec_ok) {
        long long groups = n / VEC;
        qkv_merge_grad_kernel<TIn, VEC><<<blocks_for(groups), kThreads, 0, stream>>>(dq, dk, dv, dqkv, T, H, d, groups, twin, twin_ld);
    } else {
        qkv_merge_grad_kernel<TIn, 1><<<blocks_for(n), kThreads, 0, stream>>>(dq, dk, dv, dqkv, T, H, d, n, twin, twin_ld);
    }
    return cudaGetLastError();
}
template cudaError_t launch_qkv_merge_grad<float>(const float*, const float*, const float*, float*, int, int, int, int,
                                                 cudaStream_t, __nv_bfloat16*);
template cudaError_t launch_qkv_merge_grad<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*,
                                                         const __nv_bfloat16*, float*, int, int, int, int, cudaStream_t,
                                                         __nv_bfloat16*);

template <typename TIn>
cudaError_t launch_merge_heads(const TIn* in, float* out, int B, int H, int T, int d, cudaStream_t stream, __nv_bfloat16* twin) {
    constexpr int VEC = sizeof(TIn) == 2 ? 8 : 4;
    long long n = (long long)B * T * H * d;
    if (n == 0) return cudaSuccess;
    bool vec_ok = (d % VEC == 0) && aligned16(in) && aligned16(out);
    const int twin_ld = (H * d + 7) / 8 * 8;
    if (vec_ok) {
        long long groups = n / VEC;
        head_transpose_kernel<TIn, VEC, true><<<blocks_for(groups), kThreads, 0, stream>>>(in, nullptr, nullptr, out, T, H, d, groups, twin, twin_ld);
    } else {
        head_transpose_kernel<TIn, 1, true><<<blocks_for(n), kThreads, 0, stream>>>(in, nullptr, nullptr, out, T, H, d, n, twin, twin_ld);
    }
    return cudaGetLastError();
}
template cudaError_t launch_merge_heads<float>(const float*, float*, int, int, int, int, cudaStream_t, __nv_bfloat16*);
template cudaError_t launch_merge_heads<__nv_bfloat16>(const __nv_bfloat16*, float*, int, int, int, int, cudaStream_t, __nv_bfloat16*);

template <typename TOut>
cudaError_t launch_split_heads(const float* dout, TOut* din, int B, int H, int T, int d, cudaStream_t stream) {
    constexpr int VEC = sizeof(TOut) == 2 ? 8 : 4;
    long long n = (long long)B * T * H * d;
    if (n == 0) return cudaSuccess;
    bool vec_ok = (d % VEC == 0) && aligned16(dout) && aligned16(din);
    if (vec_ok) {
        long long groups = n / VEC;
        head_transpose_kernel<TOut, VEC, false><<<blocks_for(groups), kThreads, 0, stream>>>(nullptr, din, dout, nullptr, T, H, d, groups);
    } else {
        head_transpose_kernel<TOut, 1, false><<<blocks_for(n), kThreads, 0, stream>>>(nullptr, din, dout, nullptr, T, H, d, n);
    }
    return cudaGetLastError();
}
template cudaError_t launch_split_heads<float>(const float*, float*, int, int, int, int, cudaStream_t);
template cudaError_t launch_split_heads<__nv_bfloat16>(const float*, __nv_bfloat16*, int, int, int, int, cudaStream_t);

bool dual_layout_supported(int d, const void* a, const void* b, const void* c, const void* e) {
    return d % 8 == 0 && aligned16(a) && aligned16(b) && aligned16(c) && aligned16(e);
}
cudaError_t launch_qkv_split_dual(const float* qkv, float* q, float* k, float* v, __nv_bfloat16* qb, __nv_bfloat16* kb,
                                  __nv_bfloat16* vb, int B, int T, int H, int d, cudaStream_t stream) {
    const long long n = (long long)B * T * H * d;
    if (n == 0) return cudaSuccess;
    const long long groups = n / 8;
    qkv_split_dual_kernel<<<blocks_for(groups), kThreads, 0, stream>>>(qkv, q, k, v, qb, kb, vb, T, H, d, groups);
    return cudaGetLastError();
}
cudaError_t launch_split_heads_dual(const float* dout, float* din, __nv_bfloat16* din_bf16, int B, int H, int T, int d,
                                    cudaStream_t stream) {
    const long long n = (long long)B * T * H * d;
    if (n == 0) return cudaSuccess;
    const long long groups = n / 8;
    split_heads_dual_kernel<<<blocks_for(groups), kThreads, 0, stream>>>(dout, din, din_bf16, T, H, d, groups);
    return cudaGetLastError();
}

cudaError_t launch_f32_to_bf16(const float* src, __nv_bfloat16* dst, long long n, cudaStream_t stream, float scale) {
    if (n == 0) return cudaSuccess;
    bool vec_ok = aligned16(src) && aligned16(dst);
    long long n8 = vec_ok ? n / 8 : 0;
    long long work = n8 + (n - n8 * 8);
    return launch_pdl(f32_to_bf16_kernel, dim3(blocks_for(work)), dim3(kThreads), 0, stream, src, dst, n8, n, scale);
}

cudaError_t launch_fill_normal_f32(float* dst, long long n, unsigned long long seed, long long offset,
                                   cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    fill_normal_kernel<float><<<blocks_for(n), kThreads, 0, stream>>>(dst, n, seed, offset);
    return cudaGetLastError();
}
cudaError_t launch_fill_normal_bf16(__nv_bfloat16* dst, long long n, unsigned long long seed, long long offset,
                                    cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    fill_normal_kernel<__nv_bfloat16><<<blocks_for(n), kThreads, 0, stream>>>(dst, n, seed, offset);
    return cudaGetLastError();
}

}  // namespace b200attn
