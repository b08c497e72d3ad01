// FP32 parity mode of the causal attention core: SIMT arithmetic, exact expf, FP32 everywhere.
// This is the path that meets the max-abs <= 1e-5 gate against the PyTorch oracle; the tensor-core
// path in attn_tc_*.cu is the fast one. It computes what src/kernels/attention.cu:518-1011 of
// sarimahsan/transformer-cuda computes (forward with exported m/l statistics, D pre-pass, dQ and
// dK/dV passes) with a different decomposition:
//
//   * one warp owns one query row (forward, dQ) or one key row (dK/dV);
//   * the 32 lanes take 32 consecutive keys (queries) for the score / dP dot products, so the
//     row maximum and row sum are finished with warp-shuffle reductions;
//   * for the P.V / dS.K / P^T.dO / dS^T.Q products the lanes switch to owning head-dim columns
//     and the per-key weight is broadcast with a shuffle, so V / K / dO / Q rows are read coalesced;
//   * any head dim d <= 256 works in both directions (the reference backward handles 32 and 64 only).
//
// Nothing here is accumulated with atomics, so results are bit-reproducible run to run.
#include <cfloat>

#include "kernels.cuh"

namespace b200attn {
namespace {

constexpr int kWarps = 4;
constexpr int kMaxD = 256;
constexpr int kMaxE = kMaxD / 32;  // head-dim columns owned by one lane

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
// dot(a_smem[0..d), b_global[0..d)); a is a per-warp shared copy (broadcast reads).
__device__ __forceinline__ float dot_row(const float* __restrict__ a, const float* __restrict__ b, int d, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int e = 0; e < d; e += 4) {
            float4 x = *reinterpret_cast<const float4*>(a + e);
            float4 y = __ldg(reinterpret_cast<const float4*>(b + e));
            acc = fmaf(x.x, y.x, acc);
            acc = fmaf(x.y, y.y, acc);
            acc = fmaf(x.z, y.z, acc);
            acc = fmaf(x.w, y.w, acc);
        }
    } else {
        for (int e = 0; e < d; ++e) acc = fmaf(a[e], __ldg(b + e), acc);
    }
    return acc;
}

// ------------------------------------------------------------------ forward
__global__ void __launch_bounds__(kWarps * 32) attn_fwd_f32_kernel(const float* __restrict__ q,
                                                                  const float* __restrict__ k,
                                                                  const float* __restrict__ v, float* __restrict__ out,
                                                                  float* __restrict__ m_out, float* __restrict__ l_out,
                                                                  int T, int d, float scale, bool vec) {
    __shared__ __align__(16) float sq[kWarps][kMaxD];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    // late (long) rows are scheduled first
    const int i = T - 1 - (blockIdx.x * kWarps + w);
    if (i < 0) return;
    const long long slab = (long long)blockIdx.y * T * d;
    const float* qh = q + slab;
    const float* kh = k + slab;
    const float* vh = v + slab;
    for (int e = lane; e < d; e += 32) sq[w][e] = qh[(long long)i * d + e];
    __syncwarp();

    float o[kMaxE];
#pragma unroll
    for (int r = 0; r < kMaxE; ++r) o[r] = 0.f;
    float m = -FLT_MAX, l = 0.f;
    for (int j0 = 0; j0 <= i; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= i;
        float s = valid ? scale * dot_row(sq[w], kh + (long long)j * d, d, vec) : -FLT_MAX;
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);  // 0 on the first chunk
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int r = 0; r < kMaxE; ++r) o[r] *= alpha;
        const int cnt = min(32, i - j0 + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float* vr = vh + (long long)(j0 + jj) * d;
#pragma unroll
            for (int r = 0; r < kMaxE; ++r) {
                const int e = lane + 32 * r;
                if (e < d) o[r] = fmaf(pj, __ldg(vr + e), o[r]);
            }
        }
        m = m_new;
    }
    const float inv = 1.0f / l;
    float* orow = out + slab + (long long)i * d;
#pragma unroll
    for (int r = 0; r < kMaxE; ++r) {
        const int e = lane + 32 * r;
        if (e < d) orow[e] = o[r] * inv;
    }
    if (lane == 0) {
        const long long row = (long long)blockIdx.y * T + i;
        if (m_out) m_out[row] = m;
        if (l_out) l_out[row] = l;
    }
}

// ------------------------------------------------------------------ D = rowsum(dO * O)
__global__ void __launch_bounds__(kWarps * 32) dot_do_o_f32_kernel(const float* __restrict__ dO,
                                                                  const float* __restrict__ O, float* __restrict__ D,
                                                                  long long rows, int d) {
    const int lane = threadIdx.x & 31;
    long long row = blockIdx.x * (long long)kWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* a = dO + row * d;
    const float* b = O + row * d;
    float acc = 0.f;
    for (int e = lane; e < d; e += 32) acc = fmaf(a[e], b[e], acc);
    acc = warp_sum(acc);
    if (lane == 0) D[row] = acc;
}

// ------------------------------------------------------------------ dQ: one warp per query row
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_dq_f32_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ dO, const float* __restrict__ m, const float* __restrict__ l, const float* __restrict__ D,
    float* __restrict__ dq, int T, int d, float scale, bool vec) {
    __shared__ __align__(16) float sq[kWarps][kMaxD];
    __shared__ __align__(16) float sdo[kWarps][kMaxD];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int i = T - 1 - (blockIdx.x * kWarps + w);
    if (i < 0) return;
    const long long slab = (long long)blockIdx.y * T * d;
    const long long row = (long long)blockIdx.y * T + i;
    const float* kh = k + slab;
    const float* vh = v + slab;
    for (int e = lane; e < d; e += 32) {
        sq[w][e] = q[slab + (long long)i * d + e];
        sdo[w][e] = dO[slab + (long long)i * d + e];
    }
    __syncwarp();
    const float mi = m[row], inv_l = 1.0f / l[row], Di = D[row];
    float acc[kMaxE];
#pragma unroll
    for (int r = 0; r < kMaxE; ++r) acc[r] = 0.f;
    for (int j0 = 0; j0 <= i; j0 += 32) {
        const int j = j0 + lane;
        float ds = 0.f;
        if (j <= i) {
            const float s = scale * dot_row(sq[w], kh + (long long)j * d, d, vec);
            const float p = expf(s - mi) * inv_l;
            const float dp = dot_row(sdo[w], vh + (long long)j * d, d, vec);
            ds = scale * p * (dp - Di);
        }
        const int cnt = min(32, i - j0 + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float dsj = __shfl_sync(0xffffffffu, ds, jj);
            const float* kr = kh + (long long)(j0 + jj) * d;
#pragma unroll
            for (int r = 0; r < kMaxE; ++r) {
                const int e = lane + 32 * r;
                if (e < d) acc[r] = fmaf(dsj, __ldg(kr + e), acc[r]);
            }
        }
    }
    float* dst = dq + slab + (long long)i * d;
#pragma unroll
    for (int r = 0; r < kMaxE; ++r) {
        const int e = lane + 32 * r;
        if (e < d) dst[e] = acc[r];
    }
}

// ------------------------------------------------------------------ dK, dV: one warp per key row
__global__ void __launch_bounds__(kWarps * 32) attn_bwd_dkv_f32_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ dO, const float* __restrict__ m, const float* __restrict__ l, const float* __restrict__ D,
    float* __restrict__ dk, float* __restrict__ dv, int T, int d, float scale, bool vec) {
    __shared__ __align__(16) float sk[kWarps][kMaxD];
    __shared__ __align__(16) float sv[kWarps][kMaxD];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int j = blockIdx.x * kWarps + w;  // early keys see the most queries and go first
    if (j >= T) return;
    const long long slab = (long long)blockIdx.y * T * d;
    const long long row0 = (long long)blockIdx.y * T;
    const float* qh = q + slab;
    const float* doh = dO + slab;
    for (int e = lane; e < d; e += 32) {
        sk[w][e] = k[slab + (long long)j * d + e];
        sv[w][e] = v[slab + (long long)j * d + e];
    }
    __syncwarp();
    float acc_k[kMaxE], acc_v[kMaxE];
#pragma unroll
    for (int r = 0; r < kMaxE; ++r) acc_k[r] = acc_v[r] = 0.f;
    for (int i0 = j; i0 < T; i0 += 32) {
        const int i = i0 + lane;
        float p = 0.f, ds = 0.f;
        if (i < T) {
            const float s = scale * dot_row(sk[w], qh + (long long)i * d, d, vec);
            p = expf(s - m[row0 + i]) / l[row0 + i];
            const float dp = dot_row(sv[w], doh + (long long)i * d, d, vec);
            ds = scale * p * (dp - D[row0 + i]);
        }
        const int cnt = min(32, T - i0);
        for (int ii = 0; ii < cnt; ++ii) {
            const float pi = __shfl_sync(0xffffffffu, p, ii);
            const float dsi = __shfl_sync(0xffffffffu, ds, ii);
            const float* dor = doh + (long long)(i0 + ii) * d;
            const float* qr = qh + (long long)(i0 + ii) * d;
#pragma unroll
            for (int r = 0; r < kMaxE; ++r) {
                const int e = lane + 32 * r;
                if (e < d) {
                    acc_v[r] = fmaf(pi, __ldg(dor + e), acc_v[r]);
                    acc_k[r] = fmaf(dsi, __ldg(qr + e), acc_k[r]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kMaxE; ++r) {
        const int e = lane + 32 * r;
        if (e < d) {
            dk[slab + (long long)j * d + e] = acc_k[r];
            dv[slab + (long long)j * d + e] = acc_v[r];
        }
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

cudaError_t launch_attn_fwd_f32(const float* q, const float* k, const float* v, float* out, float* m_out, float* l_out,
                                int BH, int T, int d, float scale, cudaStream_t stream) {
    if (BH == 0 || T == 0) return cudaSuccess;
    if (attn_f32_tiled_supported(d, q, k, v, q))
        return launch_attn_fwd_f32_tiled(q, k, v, out, m_out, l_out, BH, T, d, scale, stream);
    bool vec = (d % 4 == 0) && aligned16(q) && aligned16(k);
    dim3 grid((T + kWarps - 1) / kWarps, BH);
    attn_fwd_f32_kernel<<<grid, kWarps * 32, 0, stream>>>(q, k, v, out, m_out, l_out, T, d, scale, vec);
    return cudaGetLastError();
}

cudaError_t launch_dot_do_o_f32(const float* dO, const float* O, float* D, long long rows, int d, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    unsigned int blocks = (unsigned int)((rows + kWarps - 1) / kWarps);
    dot_do_o_f32_kernel<<<blocks, kWarps * 32, 0, stream>>>(dO, O, D, rows, d);
    return cudaGetLastError();
}

cudaError_t launch_attn_bwd_f32(const float* q, const float* k, const float* v, const float* dO, const float* m,
                                const float* l, const float* D, float* dq, float* dk, float* dv, int BH, int T, int d,
                                float scale, cudaStream_t stream) {
    if (BH == 0 || T == 0) return cudaSuccess;
    if (attn_f32_tiled_supported(d, q, k, v, dO))
        return launch_attn_bwd_f32_tiled(q, k, v, dO, m, l, D, dq, dk, dv, BH, T, d, scale, stream);
    bool vec = (d % 4 == 0) && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(dO);
    dim3 grid((T + kWarps - 1) / kWarps, BH);
    attn_bwd_dq_f32_kernel<<<grid, kWarps * 32, 0, stream>>>(q, k, v, dO, m, l, D, dq, T, d, scale, vec);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    attn_bwd_dkv_f32_kernel<<<grid, kWarps * 32, 0, stream>>>(q, k, v, dO, m, l, D, dk, dv, T, d, scale, vec);
    return cudaGetLastError();
}

}  // namespace b200attn
