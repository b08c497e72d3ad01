// BF16 x BF16 -> FP32 GEMM on the sm_100a tensor cores, hand-written: C (M x N, FP32, row-major, ANY leading dimension)
// = alpha * op(A) * op(B) from BF16 operands in the layouts the staging pass of matmul_dropin.cu leaves them in (A stored
// M x K or K x M, B stored K x N or N x K, leading dimensions multiples of 8). Used by the staged path of the GEMM drop-in
// in place of the library call when B200GEMM_KERNEL=tcgen05.
//
//   * One persistent CTA per SM walks 256 x 256 output tiles (M fastest, so the CTAs running together share one
//     256-column panel of B in L2). 320 threads in three roles: warp 8 issues TMA loads (cp.async.bulk.tensor, 128-byte
//     swizzle, no multicast) into a three-stage ring of 64 KB (A 256 x 64, B 256 x 64); one thread of warp 9 issues
//     tcgen05.mma (M = 128, N = 256, K = 16; two per K step, one for each half of the tile's rows, both reading the same
//     B tile); warps 0-7 are the epilogue.
//   * Why 256 x 256: what paces a one-CTA GEMM on this part is the L2 -> SM path, not the tensor pipe. With 128 x 256
//     tiles (and a double-buffered accumulator) this kernel moved 48 KB per 512 cycles of MMA and ran at 41 % of the MMA
//     rate with 9.8 TB/s of L2 reads (measured on the K = 50257 product of the head: about 38 B/clk per SM); a 256 x 256
//     tile needs 64 KB per 1024 cycles, a third less per FLOP. The price is TMEM: two 128 x 256 FP32 accumulators fill
//     all 512 columns, so the epilogue of a tile does not overlap the MMAs of the next (its loads do: the producer runs
//     ahead into the ring).
//   * Transposed operands cost nothing: an operand whose M / N index is the contiguous one is loaded as 64 x 64 boxes and
//     described to the MMA as MN-major (descriptor LBO = distance between 64-wide atoms, K step = 16 rows = 2 KB); a
//     K-contiguous operand is one box and K-major (K step = 32 bytes inside the swizzle atom).
//   * Epilogue: tcgen05.ld gives thread = row, 32 columns; a padded shared-memory transpose turns that into lane = column,
//     so every global store instruction writes 128 contiguous bytes of one row whatever the row's alignment. That is
//     what lets the language-model-head products (leading dimension V = 50257) be written in place, without the padded
//     result tile and copy-back the library path needs.
//   * Tiles beyond M, N or K are zero-filled by TMA; rows and columns beyond M and N are masked in the epilogue.
// Every mbarrier wait is bounded (tc_common.cuh); a wait that runs out is recorded in a fault word, the kernel runs to its
// end and frees its TMEM.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "gemm_tc.h"
#include "tc_common.cuh"

namespace b200gemm {
namespace {

using namespace b200attn;

constexpr int kBM = 256, kBN = 256, kBK = 64;
constexpr int kStages = 3;
constexpr int kABytes = kBM * kBK * 2;      // 32 KB
constexpr int kBBytes = kBN * kBK * 2;      // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kAtom64Bytes = 64 * 128;      // a 64-row x 64-element box: 8 KB
constexpr int kEpiWarps = 8;                // two per scheduler: a lone warp cannot hide its own load -> store latency
constexpr int kEpiPitch = 33;               // floats per staged row: conflict-free transposition
constexpr int kEpiBytes = kEpiWarps * 32 * kEpiPitch * 4;
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr int kThreads = 320;
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024;  // + slack for the 1024-byte alignment of the ring

__device__ unsigned int g_fault_word;

struct Args {
    CUtensorMap map_a, map_b;
    float* C;
    long long ldc;
    int M, N, K;
    float alpha;
};

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const __grid_constant__ Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* epi = reinterpret_cast<float*>(ring + kStages * kStageBytes);
    __shared__ uint64_t full[kStages], empty[kStages], acc_full, acc_empty;
    __shared__ uint32_t tmem_base_sh, abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], 1);
        mbar_init(&acc_full, 1), mbar_init(&acc_empty, kEpiWarps * 32);
        abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&a.map_a);
        tma_prefetch_desc(&a.map_b);
    }
    if (warp == kProducerWarp) {
        tmem_alloc(&tmem_base_sh, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_sh;
    unsigned int* fault = &g_fault_word;

    const int m_tiles = (a.M + kBM - 1) / kBM, n_tiles = (a.N + kBN - 1) / kBN, k_blocks = (a.K + kBK - 1) / kBK;
    const int total = m_tiles * n_tiles;

    if (warp == kProducerWarp) {
        if (elect_one()) {
            int g = 0;  // k-blocks loaded so far by this CTA
            for (int t = blockIdx.x; t < total; t += gridDim.x) {
                const int m0 = (t % m_tiles) * kBM, n0 = (t / m_tiles) * kBN;
                for (int kb = 0; kb < k_blocks; ++kb, ++g) {
                    const int s = g % kStages, k0 = kb * kBK;
                    if (g >= kStages) mbar_wait(&empty[s], ((g / kStages) - 1) & 1, &abort_flag, fault, 0x60);
                    mbar_expect_tx(&full[s], kStageBytes);
                    uint8_t* sA = ring + s * kStageBytes;
                    uint8_t* sB = sA + kABytes;
                    if (A_MN) {  // stored K x M: four boxes of 64 (M) x 64 (K rows)
#pragma unroll
                        for (int q = 0; q < 4; ++q) tma_load_2d(sA + q * kAtom64Bytes, &a.map_a, &full[s], m0 + 64 * q, k0);
                    } else {     // stored M x K: one box of 64 (K) x 256 (M rows)
                        tma_load_2d(sA, &a.map_a, &full[s], k0, m0);
                    }
                    if (B_MN) {  // stored K x N: four boxes of 64 (N) x 64 (K rows)
#pragma unroll
                        for (int q = 0; q < 4; ++q) tma_load_2d(sB + q * kAtom64Bytes, &a.map_b, &full[s], n0 + 64 * q, k0);
                    } else {     // stored N x K: one box of 64 (K) x 256 (N rows)
                        tma_load_2d(sB, &a.map_b, &full[s], k0, n0);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        constexpr uint32_t idesc = make_idesc_bf16(128, kBN, A_MN, B_MN);
        // rows [128, 256) of the A tile: 128 rows of 128 bytes further on (K-major), or two 64-wide atoms further (MN-major)
        constexpr uint32_t a_hi = A_MN ? 2 * kAtom64Bytes : 128 * 128;
        int g = 0, lt = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++lt) {
            if (lt >= 1) mbar_wait(&acc_empty, (lt - 1) & 1, &abort_flag, fault, 0x61);
            tc_fence_after();
            for (int kb = 0; kb < k_blocks; ++kb, ++g) {
                const int s = g % kStages;
                mbar_wait(&full[s], (g / kStages) & 1, &abort_flag, fault, 0x62);
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t sA = smem_u32(ring + s * kStageBytes), sB = sA + kABytes;
                    const uint64_t a_desc = make_smem_desc_sw128(sA, A_MN ? kAtom64Bytes : 0, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(sB, B_MN ? kAtom64Bytes : 0, 1024);
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk) {
                        const uint64_t ad = desc_advance(a_desc, A_MN ? kk * 2048 : kk * 32);
                        const uint64_t bd = desc_advance(b_desc, B_MN ? kk * 2048 : kk * 32);
                        tc_mma_ss(tmem, ad, bd, idesc, (kb > 0) || (kk > 0));
                        tc_mma_ss(tmem + kBN, desc_advance(ad, a_hi), bd, idesc, (kb > 0) || (kk > 0));
                    }
                    tc_commit(&empty[s]);
                    if (kb == k_blocks - 1) tc_commit(&acc_full);
                }
                __syncwarp();
            }
        }
    } else {
        // epilogue: warp w reads TMEM lanes [32 (w % 4), +32) (the quadrant a warp may access) = rows 32 (w % 4) ... of either
        // half of the tile, and takes every other 32-column chunk (w / 4 selects which)
        float* stage = epi + warp * 32 * kEpiPitch;
        const int quad = warp & 3, phase = warp >> 2;
        int lt = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++lt) {
            const int n0 = (t / m_tiles) * kBN;
            mbar_wait(&acc_full, lt & 1, &abort_flag, fault, 0x63);
            tc_fence_after();
#pragma unroll 1
            for (int c = phase; c < 2 * (kBN / 32); c += 2) {
                const int half = c / (kBN / 32), cc = c % (kBN / 32);  // accumulator (row half), 32-column chunk
                const int m0 = (t % m_tiles) * kBM + half * 128 + quad * 32;
                uint32_t v[32];
                tmem_ld32(tmem_addr(tmem, quad * 32, half * kBN + cc * 32), v);
                tmem_wait_ld();
                if (c + 2 >= 2 * (kBN / 32)) {  // this warp has read its share of both accumulators
                    tc_fence_before();
                    mbar_arrive(&acc_empty);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) stage[lane * kEpiPitch + j] = __uint_as_float(v[j]) * a.alpha;
                __syncwarp();
                float o[32];
#pragma unroll
                for (int r = 0; r < 32; ++r) o[r] = stage[r * kEpiPitch + lane];
                const int col = n0 + cc * 32 + lane;
                const int rows = col < a.N ? a.M - m0 : 0;  // rows of this warp's strip that exist (may exceed 32)
                float* dst = a.C + (long long)m0 * a.ldc + col;
#pragma unroll
                for (int r = 0; r < 32; ++r)
                    if (r < rows) dst[(long long)r * a.ldc] = o[r];
                __syncwarp();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kProducerWarp) tmem_dealloc(tmem, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
long long g_launches = 0;

// BF16 row-major matrix of `rows` rows of `cols` elements (leading dimension ld) as a 2-D map with boxes of 64 x box_rows.
bool make_map(CUtensorMap* m, const void* base, int cols, int rows, int ld, int box_rows) {
    cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
    cuuint32_t box[2] = {64, cuuint32_t(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    return g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One line on stderr the first time a reason occurs; the caller then takes the library path.
bool refuse(const char* why) {
    static const char* last = nullptr;
    if (last != why) fprintf(stderr, "b200gemm: tcgen05 kernel not used (%s: %s)\n", why, cudaGetErrorString(cudaGetLastError()));
    last = why;
    return false;
}

template <int A_MN, int B_MN>
bool launch(const Args& args, int grid, cudaStream_t stream) {
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
            return false;
        attr_set = true;
    }
    gemm_tc_kernel<A_MN, B_MN><<<grid, kThreads, kSmemBytes, stream>>>(args);
    return cudaGetLastError() == cudaSuccess;
}

}  // namespace

int tc_gemm_tiles(int M, int N) { return ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN); }

bool tc_gemm_bf16(const void* A, int rows_a, int lda, bool trans_a, const void* B, int rows_b, int ldb, bool trans_b, float* C,
                  long long ldc, int M, int N, int K, float alpha, cudaStream_t stream) {
    static int sm_count = 0;
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return false;
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        int dev = 0, major = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return false;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (major != 10) sm_count = 0;
    }
    if (sm_count <= 0) return false;  // not an sm_100 device: the caller keeps the library path
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15u || lda % 8 || ldb % 8) return refuse("operand alignment");
    Args args;
    // A: stored M x K (K contiguous: box 64 x 128) or K x M (M contiguous: boxes 64 x 64)
    if (!make_map(&args.map_a, A, trans_a ? M : K, rows_a, lda, trans_a ? 64 : kBM)) return refuse("tensor map of A");
    // B: stored N x K (K contiguous: box 64 x 256) or K x N (N contiguous: boxes 64 x 64)
    if (!make_map(&args.map_b, B, trans_b ? K : N, rows_b, ldb, trans_b ? kBN : 64)) return refuse("tensor map of B");
    args.C = C, args.ldc = ldc, args.M = M, args.N = N, args.K = K, args.alpha = alpha;
    const int tiles = tc_gemm_tiles(M, N), grid = tiles < sm_count ? tiles : sm_count;
    const bool a_mn = trans_a, b_mn = !trans_b;
    const bool ok = a_mn ? (b_mn ? launch<1, 1>(args, grid, stream) : launch<1, 0>(args, grid, stream))
                         : (b_mn ? launch<0, 1>(args, grid, stream) : launch<0, 0>(args, grid, stream));
    if (ok) ++g_launches;
    return ok ? true : refuse("kernel launch");
}

long long tc_gemm_launches() { return g_launches; }

unsigned int tc_gemm_take_fault() {
    unsigned int word = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&word, g_fault_word, sizeof(word)) != cudaSuccess) return 0xffffffffu;
    if (word) cudaMemcpyToSymbol(g_fault_word, &zero, sizeof(zero));
    return word;
}

}  // namespace b200gemm
