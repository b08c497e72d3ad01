// FP32 parity mode, tiled: the same arithmetic as attn_f32.cu (SIMT FP32, exact expf, no atomics,
// bit-reproducible) organised as small register-blocked GEMMs over shared-memory tiles, for the head
// dims the models use (32, 64, 128). attn_f32.cu keeps the generic one-warp-per-row kernels for any
// other head dim. Replaces the reference's tiled kernels (src/kernels/attention.cu:518-1011) in the
// default (FP32) math mode of the float* launch API.
//
// Decomposition. A CTA of 8 warps owns 32 consecutive "block rows" (queries in the forward and dQ
// kernels, keys in the dK/dV kernel), 4 per warp, and walks the other sequence in tiles of 64
// positions staged in shared memory with rows padded to D+4 floats. Two primitives do all the work:
//
//   tile_dot    s[r][c] = <A_row r, B_tile row (lane + 32c)>, r < 4, c < 2: each lane reads its two
//               tile rows with 16-byte shared loads (conflict-free thanks to the padding) and the four
//               block rows with broadcast 16-byte loads: 6 loads feed 32 FMAs.
//   tile_accum  acc[r][0..CW) += sum_j w[r][j] * V_tile[j][lane*CW ..], CW = D/32 consecutive head-dim
//               columns per lane: the weights w (probabilities or dS) are exchanged through a per-warp
//               shared buffer and read back as broadcast 16-byte loads.
//
// Row maxima / sums over a tile are finished with warp-shuffle reductions. Tiles wholly on the masked
// side of the causal diagonal are skipped; the mask is applied per element only on diagonal tiles.
#include <cfloat>

#include "kernels.cuh"

namespace b200attn {
namespace {

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 4;
constexpr int kBlockRows = kWarps * kRowsPerWarp;  // 32
constexpr int kTile = 64;                          // positions of the other sequence per tile
constexpr int kThreads = kWarps * 32;

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

template <int D>
struct Smem {
    static constexpr int kPitch = D + 4;  // floats per staged row: keeps 16-byte alignment, spreads banks
};

// Stage `rows` rows (row index row0 .. row0+rows-1 of a (T, D) slab, zero beyond T) into shared memory.
template <int D>
__device__ __forceinline__ void stage_rows(float* __restrict__ dst, const float* __restrict__ slab, int row0, int rows,
                                           int T) {
    constexpr int kVecPerRow = D / 4;
    for (int idx = threadIdx.x; idx < rows * kVecPerRow; idx += kThreads) {
        const int r = idx / kVecPerRow, c = (idx % kVecPerRow) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < T) v = __ldg(reinterpret_cast<const float4*>(slab + (long long)(row0 + r) * D + c));
        *reinterpret_cast<float4*>(dst + r * Smem<D>::kPitch + c) = v;
    }
}

// s[r][c] = dot(a_rows[r], tile[lane + 32 c]) over D.
template <int D>
__device__ __forceinline__ void tile_dot(const float* __restrict__ a_rows, const float* __restrict__ tile, int lane,
                                         float (&s)[kRowsPerWarp][2]) {
    constexpr int P = Smem<D>::kPitch;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) s[r][0] = s[r][1] = 0.f;
    const float* b0 = tile + lane * P;
    const float* b1 = tile + (lane + 32) * P;
#pragma unroll 4
    for (int e = 0; e < D; e += 4) {
        const float4 k0 = *reinterpret_cast<const float4*>(b0 + e);
        const float4 k1 = *reinterpret_cast<const float4*>(b1 + e);
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const float4 a = *reinterpret_cast<const float4*>(a_rows + r * P + e);  // broadcast
            s[r][0] = fmaf(a.x, k0.x, fmaf(a.y, k0.y, fmaf(a.z, k0.z, fmaf(a.w, k0.w, s[r][0]))));
            s[r][1] = fmaf(a.x, k1.x, fmaf(a.y, k1.y, fmaf(a.z, k1.z, fmaf(a.w, k1.w, s[r][1]))));
        }
    }
}

// acc[r][x] += sum_{j < kTile} w[r][j] * tile[j][lane*CW + x]; w is a per-warp (4 x kTile) shared buffer.
template <int D>
__device__ __forceinline__ void tile_accum(const float* __restrict__ w, const float* __restrict__ tile, int lane,
                                           float (&acc)[kRowsPerWarp][D / 32]) {
    constexpr int P = Smem<D>::kPitch;
    constexpr int CW = D / 32;
    const float* col = tile + lane * CW;
#pragma unroll 2
    for (int j = 0; j < kTile; j += 4) {
        float4 wr[kRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) wr[r] = *reinterpret_cast<const float4*>(w + r * kTile + j);  // broadcast
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            float vv[CW];
            if constexpr (CW == 4) {
                const float4 t = *reinterpret_cast<const float4*>(col + (j + jj) * P);
                vv[0] = t.x, vv[1] = t.y, vv[2] = t.z, vv[3] = t.w;
            } else if constexpr (CW == 2) {
                const float2 t = *reinterpret_cast<const float2*>(col + (j + jj) * P);
                vv[0] = t.x, vv[1] = t.y;
            } else {
                vv[0] = col[(j + jj) * P];
            }
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                const float wj = jj == 0 ? wr[r].x : jj == 1 ? wr[r].y : jj == 2 ? wr[r].z : wr[r].w;
#pragma unroll
                for (int x = 0; x < CW; ++x) acc[r][x] = fmaf(wj, vv[x], acc[r][x]);
            }
        }
    }
}

template <int D>
__device__ __forceinline__ void store_rows(float* __restrict__ slab, int row0, int T, int lane,
                                           const float (&acc)[kRowsPerWarp][D / 32], const float (&mul)[kRowsPerWarp]) {
    constexpr int CW = D / 32;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        if (row0 + r >= T) continue;
        float* dst = slab + (long long)(row0 + r) * D + lane * CW;
#pragma unroll
        for (int x = 0; x < CW; ++x) dst[x] = acc[r][x] * mul[r];
    }
}

// ------------------------------------------------------------------ forward
template <int D>
__global__ void __launch_bounds__(kThreads) attn_fwd_f32_tiled_kernel(const float* __restrict__ q,
                                                                     const float* __restrict__ k,
                                                                     const float* __restrict__ v, float* __restrict__ out,
                                                                     float* __restrict__ m_out, float* __restrict__ l_out,
                                                                     int T, float scale) {
    extern __shared__ __align__(16) float smem_f[];
    constexpr int P = Smem<D>::kPitch;
    float* sQ = smem_f;                    // kBlockRows x P
    float* sK = sQ + kBlockRows * P;       // kTile x P
    float* sV = sK + kTile * P;            // kTile x P
    float* sW = sV + kTile * P;            // kWarps x 4 x kTile
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int n_blocks = (T + kBlockRows - 1) / kBlockRows;
    const int blk = n_blocks - 1 - blockIdx.x;  // late (long) blocks first
    const int row0 = blk * kBlockRows;
    const long long slab = (long long)blockIdx.y * T * D;
    stage_rows<D>(sQ, q + slab, row0, kBlockRows, T);

    const int my_row0 = row0 + w * kRowsPerWarp;
    float acc[kRowsPerWarp][D / 32];
    float m[kRowsPerWarp], l[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        m[r] = -FLT_MAX, l[r] = 0.f;
#pragma unroll
        for (int x = 0; x < D / 32; ++x) acc[r][x] = 0.f;
    }
    const int last_row = min(T, row0 + kBlockRows) - 1;
    float* wbuf = sW + w * kRowsPerWarp * kTile;
    for (int j0 = 0; j0 <= last_row; j0 += kTile) {
        __syncthreads();  // previous tile fully consumed (and sQ staged, first time)
        stage_rows<D>(sK, k + slab, j0, kTile, T);
        stage_rows<D>(sV, v + slab, j0, kTile, T);
        __syncthreads();
        if (j0 > my_row0 + kRowsPerWarp - 1) continue;  // tile wholly above this warp's rows (barriers stay aligned)
        float s[kRowsPerWarp][2];
        tile_dot<D>(sQ + w * kRowsPerWarp * P, sK, lane, s);
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int i = my_row0 + r;
            float s0 = (j0 + lane <= i) ? s[r][0] * scale : -FLT_MAX;
            float s1 = (j0 + lane + 32 <= i) ? s[r][1] * scale : -FLT_MAX;
            const float m_new = fmaxf(m[r], warp_max(fmaxf(s0, s1)));
            const float alpha = expf(m[r] - m_new);  // 0 on the first tile; 1 for rows with nothing visible yet
            const float p0 = (j0 + lane <= i) ? expf(s0 - m_new) : 0.f;
            const float p1 = (j0 + lane + 32 <= i) ? expf(s1 - m_new) : 0.f;
            l[r] = l[r] * alpha + warp_sum(p0 + p1);
            m[r] = m_new;
#pragma unroll
            for (int x = 0; x < D / 32; ++x) acc[r][x] *= alpha;
            wbuf[r * kTile + lane] = p0;
            wbuf[r * kTile + lane + 32] = p1;
        }
        __syncwarp();
        tile_accum<D>(wbuf, sV, lane, acc);
        __syncwarp();
    }
    float inv[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) inv[r] = 1.0f / l[r];
    store_rows<D>(out + slab, my_row0, T, lane, acc, inv);
    if (lane < kRowsPerWarp && my_row0 + lane < T) {
        const long long row = (long long)blockIdx.y * T + my_row0 + lane;
        float mm = m[0], ll = l[0];
#pragma unroll
        for (int r = 1; r < kRowsPerWarp; ++r)
            if (lane == r) mm = m[r], ll = l[r];
        if (m_out) m_out[row] = mm;
        if (l_out) l_out[row] = ll;
    }
}

// ------------------------------------------------------------------ dQ: block rows are queries
template <int D>
__global__ void __launch_bounds__(kThreads) attn_bwd_dq_f32_tiled_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ dO, const float* __restrict__ m, const float* __restrict__ l, const float* __restrict__ Dv,
    float* __restrict__ dq, int T, float scale) {
    extern __shared__ __align__(16) float smem_f[];
    constexpr int P = Smem<D>::kPitch;
    float* sQ = smem_f;
    float* sDO = sQ + kBlockRows * P;
    float* sK = sDO + kBlockRows * P;
    float* sV = sK + kTile * P;
    float* sW = sV + kTile * P;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int n_blocks = (T + kBlockRows - 1) / kBlockRows;
    const int row0 = (n_blocks - 1 - blockIdx.x) * kBlockRows;
    const long long slab = (long long)blockIdx.y * T * D;
    const long long stat0 = (long long)blockIdx.y * T;
    stage_rows<D>(sQ, q + slab, row0, kBlockRows, T);
    stage_rows<D>(sDO, dO + slab, row0, kBlockRows, T);
    const int my_row0 = row0 + w * kRowsPerWarp;
    float acc[kRowsPerWarp][D / 32];
    float mi[kRowsPerWarp], il[kRowsPerWarp], Di[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int i = my_row0 + r;
        mi[r] = i < T ? m[stat0 + i] : 0.f;
        il[r] = i < T ? 1.0f / l[stat0 + i] : 0.f;
        Di[r] = i < T ? Dv[stat0 + i] : 0.f;
#pragma unroll
        for (int x = 0; x < D / 32; ++x) acc[r][x] = 0.f;
    }
    const int last_row = min(T, row0 + kBlockRows) - 1;
    float* wbuf = sW + w * kRowsPerWarp * kTile;
    for (int j0 = 0; j0 <= last_row; j0 += kTile) {
        __syncthreads();
        stage_rows<D>(sK, k + slab, j0, kTile, T);
        stage_rows<D>(sV, v + slab, j0, kTile, T);
        __syncthreads();
        if (j0 > my_row0 + kRowsPerWarp - 1) continue;
        float s[kRowsPerWarp][2], dp[kRowsPerWarp][2];
        tile_dot<D>(sQ + w * kRowsPerWarp * P, sK, lane, s);
        tile_dot<D>(sDO + w * kRowsPerWarp * P, sV, lane, dp);
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int i = my_row0 + r;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int j = j0 + lane + 32 * c;
                float ds = 0.f;
                if (j <= i && i < T) {
                    const float p = expf(s[r][c] * scale - mi[r]) * il[r];
                    ds = scale * p * (dp[r][c] - Di[r]);
                }
                wbuf[r * kTile + lane + 32 * c] = ds;
            }
        }
        __syncwarp();
        tile_accum<D>(wbuf, sK, lane, acc);
        __syncwarp();
    }
    const float one[kRowsPerWarp] = {1.f, 1.f, 1.f, 1.f};
    store_rows<D>(dq + slab, my_row0, T, lane, acc, one);
}

// ------------------------------------------------------------------ dK, dV: block rows are keys
template <int D>
__global__ void __launch_bounds__(kThreads) attn_bwd_dkv_f32_tiled_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ dO, const float* __restrict__ m, const float* __restrict__ l, const float* __restrict__ Dv,
    float* __restrict__ dk, float* __restrict__ dv, int T, float scale) {
    extern __shared__ __align__(16) float smem_f[];
    constexpr int P = Smem<D>::kPitch;
    float* sK = smem_f;                     // block rows: keys
    float* sV = sK + kBlockRows * P;
    float* sQ = sV + kBlockRows * P;        // tiles: queries
    float* sDO = sQ + kTile * P;
    float* sW = sDO + kTile * P;            // kWarps x 2 x (4 x kTile): p and ds
    float* sStat = sW + kWarps * 2 * kRowsPerWarp * kTile;  // 3 x kTile: m, 1/l, D of the query tile
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int row0 = blockIdx.x * kBlockRows;  // early keys see the most queries and go first
    const long long slab = (long long)blockIdx.y * T * D;
    const long long stat0 = (long long)blockIdx.y * T;
    stage_rows<D>(sK, k + slab, row0, kBlockRows, T);
    stage_rows<D>(sV, v + slab, row0, kBlockRows, T);
    const int my_row0 = row0 + w * kRowsPerWarp;
    float acc_k[kRowsPerWarp][D / 32], acc_v[kRowsPerWarp][D / 32];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
        for (int x = 0; x < D / 32; ++x) acc_k[r][x] = acc_v[r][x] = 0.f;
    float* pbuf = sW + w * 2 * kRowsPerWarp * kTile;
    float* dsbuf = pbuf + kRowsPerWarp * kTile;
    // query tiles from the one containing this block's first key to the end of the sequence
    for (int i0 = (row0 / kTile) * kTile; i0 < T; i0 += kTile) {
        __syncthreads();
        stage_rows<D>(sQ, q + slab, i0, kTile, T);
        stage_rows<D>(sDO, dO + slab, i0, kTile, T);
        if (threadIdx.x < kTile) {
            const int i = i0 + threadIdx.x;
            sStat[threadIdx.x] = i < T ? m[stat0 + i] : 0.f;
            sStat[kTile + threadIdx.x] = i < T ? 1.0f / l[stat0 + i] : 0.f;
            sStat[2 * kTile + threadIdx.x] = i < T ? Dv[stat0 + i] : 0.f;
        }
        __syncthreads();
        float s[kRowsPerWarp][2], dp[kRowsPerWarp][2];
        tile_dot<D>(sK + w * kRowsPerWarp * P, sQ, lane, s);    // s[r][c] = <k_r, q_(i0 + lane + 32c)>
        tile_dot<D>(sV + w * kRowsPerWarp * P, sDO, lane, dp);  // <v_r, dO_i>
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int j = my_row0 + r;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int ii = lane + 32 * c, i = i0 + ii;
                float p = 0.f, ds = 0.f;
                if (i >= j && i < T && j < T) {
                    p = expf(s[r][c] * scale - sStat[ii]) * sStat[kTile + ii];
                    ds = scale * p * (dp[r][c] - sStat[2 * kTile + ii]);
                }
                pbuf[r * kTile + ii] = p;
                dsbuf[r * kTile + ii] = ds;
            }
        }
        __syncwarp();
        tile_accum<D>(pbuf, sDO, lane, acc_v);
        tile_accum<D>(dsbuf, sQ, lane, acc_k);
        __syncwarp();
    }
    const float one[kRowsPerWarp] = {1.f, 1.f, 1.f, 1.f};
    store_rows<D>(dk + slab, my_row0, T, lane, acc_k, one);
    store_rows<D>(dv + slab, my_row0, T, lane, acc_v, one);
}

template <int D>
size_t fwd_smem() { return sizeof(float) * ((kBlockRows + 2 * kTile) * Smem<D>::kPitch + kWarps * kRowsPerWarp * kTile); }
template <int D>
size_t dq_smem() { return sizeof(float) * ((2 * kBlockRows + 2 * kTile) * Smem<D>::kPitch + kWarps * kRowsPerWarp * kTile); }
template <int D>
size_t dkv_smem() {
    return sizeof(float) * ((2 * kBlockRows + 2 * kTile) * Smem<D>::kPitch + kWarps * 2 * kRowsPerWarp * kTile + 3 * kTile);
}

template <int D>
cudaError_t launch_fwd(const float* q, const float* k, const float* v, float* out, float* m_out, float* l_out, int BH,
                       int T, float scale, cudaStream_t stream) {
    auto kern = attn_fwd_f32_tiled_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem<D>());
    if (e != cudaSuccess) return e;
    dim3 grid((T + kBlockRows - 1) / kBlockRows, BH);
    kern<<<grid, kThreads, fwd_smem<D>(), stream>>>(q, k, v, out, m_out, l_out, T, scale);
    return cudaGetLastError();
}
template <int D>
cudaError_t launch_bwd(const float* q, const float* k, const float* v, const float* dO, const float* m, const float* l,
                       const float* Dv, float* dq, float* dk, float* dv, int BH, int T, float scale, cudaStream_t stream) {
    auto kq = attn_bwd_dq_f32_tiled_kernel<D>;
    auto kkv = attn_bwd_dkv_f32_tiled_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dq_smem<D>());
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dkv_smem<D>());
    if (e != cudaSuccess) return e;
    dim3 grid((T + kBlockRows - 1) / kBlockRows, BH);
    kq<<<grid, kThreads, dq_smem<D>(), stream>>>(q, k, v, dO, m, l, Dv, dq, T, scale);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    kkv<<<grid, kThreads, dkv_smem<D>(), stream>>>(q, k, v, dO, m, l, Dv, dk, dv, T, scale);
    return cudaGetLastError();
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

bool attn_f32_tiled_supported(int d, const void* a, const void* b, const void* c, const void* e) {
    return (d == 32 || d == 64 || d == 128) && aligned16(a) && aligned16(b) && aligned16(c) && aligned16(e);
}

cudaError_t launch_attn_fwd_f32_tiled(const float* q, const float* k, const float* v, float* out, float* m_out,
                                      float* l_out, int BH, int T, int d, float scale, cudaStream_t stream) {
    if (BH == 0 || T == 0) return cudaSuccess;
    if (d == 32) return launch_fwd<32>(q, k, v, out, m_out, l_out, BH, T, scale, stream);
    if (d == 64) return launch_fwd<64>(q, k, v, out, m_out, l_out, BH, T, scale, stream);
    if (d == 128) return launch_fwd<128>(q, k, v, out, m_out, l_out, BH, T, scale, stream);
    return cudaErrorInvalidValue;
}

cudaError_t launch_attn_bwd_f32_tiled(const float* q, const float* k, const float* v, const float* dO, const float* m,
                                      const float* l, const float* D, float* dq, float* dk, float* dv, int BH, int T,
                                      int d, float scale, cudaStream_t stream) {
    if (BH == 0 || T == 0) return cudaSuccess;
    if (d == 32) return launch_bwd<32>(q, k, v, dO, m, l, D, dq, dk, dv, BH, T, scale, stream);
    if (d == 64) return launch_bwd<64>(q, k, v, dO, m, l, D, dq, dk, dv, BH, T, scale, stream);
    if (d == 128) return launch_bwd<128>(q, k, v, dO, m, l, D, dq, dk, dv, BH, T, scale, stream);
    return cudaErrorInvalidValue;
}

}  // namespace b200attn
