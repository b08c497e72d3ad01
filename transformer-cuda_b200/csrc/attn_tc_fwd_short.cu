// TWO-CTAS-PER-SM variant of the causal attention forward (used for d = 64 at every T and for d = 128 up to
// T = 4096; attn_tc_fwd.cu has the one-large-CTA variant for longer d = 128 sequences and the dispatch). Same math, same TMEM/TMA/MMA
// idioms, different occupancy trade: a CTA here is small enough (256 TMEM columns, <= 96 KB of shared
// memory, 192 threads) for TWO to be resident per SM, so that the prologue and epilogue of one CTA -
// a large share of a CTA's life when it only walks a handful of key tiles - overlap the main loop of
// the other, and one CTA's MMAs run while the other's softmax warps work.
//
// Causal attention forward on the sm_100a tensor cores (tcgen05), BF16 operands, FP32
// accumulation and FP32 softmax statistics. Computes what tiled_causal_attention_forward of
// sarimahsan/transformer-cuda computes (src/kernels/attention.cu:518-657): O = softmax(scale*QK^T
// + causal mask) V with the row maximum m and the un-normalised row sum l exported.
//
// One CTA owns one 128-row query tile of one (batch, head) slab and walks the key/value tiles
// 0..diagonal (tiles above the diagonal are never loaded). Six warps, three roles:
//
//   warps 0-3  softmax: thread r owns query row r. S_j is read from TMEM with tcgen05.ld (one row
//              per thread, so row max / row sum need no cross-thread traffic), turned into
//              P_j = exp2(S_j*scale*log2e - m) in BF16 and written back over S_j in TMEM, where the
//              P.V MMA reads it as its A operand. The same threads rescale the O accumulator in
//              TMEM when the running maximum has moved by more than 2^8, and run the epilogue.
//   warp 4     TMA producer: Q once, then a ring of K and V tiles (cp.async.bulk.tensor, 128-byte
//              swizzle, no multicast), each signalled through an mbarrier with expect_tx.
//   warp 5     MMA issuer: S_j = Q K_j^T (both operands K-major in shared memory) into the TMEM
//              score buffer, and O += P_j V_j (A from TMEM, V as an MN-major shared-memory
//              operand, so no transpose is materialised).
//
// A CTA uses 256 TMEM columns and at most 96 KB of shared memory, so two CTAs are resident per SM:
// while one CTA's softmax warps work on a tile, the other CTA's MMAs and loads run, and the
// prologue / epilogue of one overlaps the main loop of the other.
//   D = 128: [0,128) S with P written over it, [128,256) O. S_{j+1} can only be issued behind P_j V_j.
//   D = 64:  [0,128) S, [128,192) O, [192,256) P. The softmax threads pull a whole score row into
//            registers and release the score buffer at once (s_free), so S_{j+1} = Q K_{j+1}^T runs
//            under the exponentials of tile j and the softmax threads never wait for the tensor
//            pipe in steady state; P_j V_j runs under the exponentials of tile j+1.
// Every mbarrier wait has an iteration limit (tc_common.cuh); a wait that gives up sets the fault
// word and the kernel still runs to its end and frees its TMEM.
#include "kernels.cuh"
#include "tc_common.cuh"


namespace b200attn {
namespace {

constexpr int kBM = 128;                 // query rows per CTA
constexpr int kBN = 128;                 // key/value rows per tile
constexpr int kAtomBytes = 128 * 128;    // one TMA box: 128 rows x 64 bf16, 128-byte swizzled
constexpr int kSoftmaxThreads = 128;
constexpr int kThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int D>
struct FwdCfg {
    static constexpr int kAtoms = D / 64;
    static constexpr int kTileBytes = kAtoms * kAtomBytes;
    static constexpr int kStages = (D == 64) ? 2 : 1;
    static constexpr int kSmemBytes = kTileBytes * (1 + 2 * kStages);  // dynamic buffer is declared 1024-aligned
    static constexpr uint32_t kTmemCols = 256;
    static constexpr bool kSeparateP = (D == 64);  // P in its own columns: the score buffer is free once loaded
    static constexpr uint32_t kColS = 0, kColO = 128;
    static constexpr uint32_t kColP = kSeparateP ? 192 : 0;
};

struct FwdBarriers {
    uint64_t q_full;
    uint64_t k_full[3], v_full[3], k_empty[3], v_empty[3];
    uint64_t s_full, p_full, s_free;
    uint64_t o_done;
};

template <int D, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 2) attn_fwd_tc_short_kernel(const __grid_constant__ TcFwdArgs a) {
    using Cfg = FwdCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = smem + Cfg::kTileBytes;
    uint8_t* sV = sK + Cfg::kStages * Cfg::kTileBytes;

    __shared__ FwdBarriers bars;
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    pdl_launch_dependents();

    const int n_q_tiles = (a.T + kBM - 1) / kBM;
    // CTA order: the last query tile of a slab is the longest. Longest-first across all slabs when the
    // problem fits in L2 (shortest tail), else slab by slab (resident CTAs share K/V tiles in L2).
    const int bh = a.tile_major_order ? int(blockIdx.x % a.BH) : int(blockIdx.x / n_q_tiles);
    const int qt = n_q_tiles - 1 - (a.tile_major_order ? int(blockIdx.x / a.BH) : int(blockIdx.x % n_q_tiles));
    const int hh = bh % a.H, bb = bh / a.H;  // head and batch coordinates of the 4-D tensor maps
    const int n_kv = qt + 1;                                  // key tiles 0..qt; qt is the diagonal tile

    if (tid == 0) {
        mbar_init(&bars.q_full, 1);
        for (int s = 0; s < 3; ++s) {
            mbar_init(&bars.k_full[s], 1);
            mbar_init(&bars.v_full[s], 1);
            mbar_init(&bars.k_empty[s], 1);
            mbar_init(&bars.v_empty[s], 1);
        }
        mbar_init(&bars.s_full, 1);
        mbar_init(&bars.p_full, kSoftmaxThreads);
        mbar_init(&bars.s_free, kSoftmaxThreads);
        mbar_init(&bars.o_done, 1);
        abort_flag = 0;
        if ((smem_u32(smem) & 1023u) != 0 && a.fault_word) atomicCAS(a.fault_word, 0u, kFaultWaitTimeout | 0xA10u);
        mbar_fence_init();
    }
    if (warp == 4) {
        tmem_alloc(&tmem_base_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_slot;
    // barriers, TMEM and the tensor maps are set up: from here on global memory is touched, so wait for the
    // kernel in front of this one in the stream (returns at once for an ordinary launch)
    pdl_wait();

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&a.map_q);
            tma_prefetch_desc(&a.map_k);
            tma_prefetch_desc(&a.map_v);
            mbar_expect_tx(&bars.q_full, Cfg::kTileBytes);
            for (int at = 0; at < Cfg::kAtoms; ++at)
                tma_load_4d(sQ + at * kAtomBytes, &a.map_q, &bars.q_full, at * 64, qt * kBM, hh, bb);
            for (int j = 0; j < n_kv; ++j) {
                const int s = j % Cfg::kStages;
                const int round = j / Cfg::kStages;
                if (round > 0) mbar_wait(&bars.k_empty[s], (round - 1) & 1, &abort_flag, a.fault_word, 0x10);
                mbar_expect_tx(&bars.k_full[s], Cfg::kTileBytes);
                for (int at = 0; at < Cfg::kAtoms; ++at)
                    tma_load_4d(sK + s * Cfg::kTileBytes + at * kAtomBytes, &a.map_k, &bars.k_full[s], at * 64, j * kBN, hh, bb);
                if (round > 0) mbar_wait(&bars.v_empty[s], (round - 1) & 1, &abort_flag, a.fault_word, 0x11);
                mbar_expect_tx(&bars.v_full[s], Cfg::kTileBytes);
                for (int at = 0; at < Cfg::kAtoms; ++at)
                    tma_load_4d(sV + s * Cfg::kTileBytes + at * kAtomBytes, &a.map_v, &bars.v_full[s], at * 64, j * kBN, hh, bb);
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_qk = make_idesc_bf16(kBM, kBN, 0, 0);
        constexpr uint32_t idesc_pv = make_idesc_bf16(kBM, D, 0, 1);
        const uint64_t q_desc = make_smem_desc_sw128(smem_u32(sQ), 0, 1024);
        mbar_wait(&bars.q_full, 0, &abort_flag, a.fault_word, 0x20);
        auto issue_qk = [&](int j) {  // S = Q K_j^T
            const int s = j % Cfg::kStages;
            mbar_wait(&bars.k_full[s], (j / Cfg::kStages) & 1, &abort_flag, a.fault_word, 0x21);
            tc_fence_after();
            if (elect_one()) {
                const uint64_t k_desc = make_smem_desc_sw128(smem_u32(sK + s * Cfg::kTileBytes), 0, 1024);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kAtomBytes + (kk & 3) * 32;
                    tc_mma_ss(tmem + Cfg::kColS, desc_advance(q_desc, off), desc_advance(k_desc, off), idesc_qk, kk > 0);
                }
                tc_commit(&bars.k_empty[s]);
                tc_commit(&bars.s_full);
            }
            __syncwarp();
        };
        if (Cfg::kSeparateP) issue_qk(0);
        for (int j = 0; j < n_kv; ++j) {
            const int s = j % Cfg::kStages;
            const uint32_t ring_phase = (j / Cfg::kStages) & 1;
            if (Cfg::kSeparateP) {
                // the softmax threads hold S_j in registers: the next scores run under their exponentials
                if (j + 1 < n_kv) {
                    mbar_wait(&bars.s_free, j & 1, &abort_flag, a.fault_word, 0x24);
                    issue_qk(j + 1);
                }
            } else {
                // the score buffer is free: P_{j-1} V_{j-1} was issued before, and MMAs run in order
                issue_qk(j);
            }
            // O += P_j V_j
            mbar_wait(&bars.v_full[s], ring_phase, &abort_flag, a.fault_word, 0x22);
            mbar_wait(&bars.p_full, j & 1, &abort_flag, a.fault_word, 0x23);
            tc_fence_after();
            if (elect_one()) {
                // V tile: rows = key index (the MMA's K), 64-column atoms along the head dim (its N)
                const uint64_t v_desc = make_smem_desc_sw128(smem_u32(sV + s * Cfg::kTileBytes), kAtomBytes, 1024);
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk)
                    tc_mma_ts(tmem + Cfg::kColO, tmem + Cfg::kColP + kk * 8, desc_advance(v_desc, kk * 2048), idesc_pv,
                              (j > 0) || (kk > 0));
                tc_commit(&bars.v_empty[s]);
                tc_commit(&bars.o_done);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ softmax + correction + epilogue
        const int r = tid;                                // query row inside the tile, TMEM lane
        const uint32_t lane_base = uint32_t(warp) * 32u;  // this warp's TMEM lane quadrant
        const float scale_log2 = a.scale * kLog2e;
        // Exponents are taken relative to m_ref, which follows the true running maximum m_true only
        // when that has moved by more than kRescaleThreshold (in log2 units): P stays below
        // 2^threshold, and the O accumulator in TMEM has to be rescaled only on those rare moves.
        constexpr float kRescaleThreshold = 8.0f;
        float m_true = -INFINITY;  // running maximum of scale*log2e*s
        float m_ref = -INFINITY;   // reference the exponentials and l_run are relative to
        float l_run = 0.f;
        for (int j = 0; j < n_kv; ++j) {
            constexpr uint32_t s_col = Cfg::kColS;
            // D = 128: s_full(j) also means P.V of tile j-1 has retired (MMAs run in order), so O is up to date
            mbar_wait(&bars.s_full, j & 1, &abort_flag, a.fault_word, 0x30);
            tc_fence_after();
            uint32_t sv[kBN];
#pragma unroll
            for (int c = 0; c < kBN; c += 32) tmem_ld32(tmem_addr(tmem, lane_base, s_col + c), &sv[c]);
            tmem_wait_ld();
            if (Cfg::kSeparateP) {  // the whole row is in registers: hand the score buffer back
                tc_fence_before();
                mbar_arrive(&bars.s_free);
            }
            if (j == qt) {  // diagonal tile: key c is visible to query r iff c <= r
#pragma unroll
                for (int c = 0; c < kBN; ++c)
                    if (c > r) sv[c] = 0xff800000u;  // -inf
            }
            // four independent chains: a single running maximum is 128 dependent instructions
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < kBN; c += 4) {
#pragma unroll
                for (int y = 0; y < 4; ++y) mx4[y] = fmaxf(mx4[y], __uint_as_float(sv[c + y]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            m_true = fmaxf(m_true, mx * scale_log2);
            const bool move = (j == 0) || (m_true - m_ref > kRescaleThreshold);
            float alpha = 1.0f;
            if (move) {
                alpha = fast_exp2(m_ref - m_true);  // 0 on the first tile
                m_ref = m_true;
            }
            // scale-and-shift and row sums on packed pairs (fma2 / add2): five instructions per pair of scores instead of seven
            float2 sum2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
            uint32_t pk[kBN / 2];
            const float neg_ref = -m_ref;
#pragma unroll
            for (int c = 0; c < kBN; c += 2) {
                const float2 arg = fma2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), scale_log2, neg_ref);
                const float p0 = mixed_exp2(arg.x, c);
                const float p1 = mixed_exp2(arg.y, c + 1);
                sum2[(c >> 1) & 3] = add2(sum2[(c >> 1) & 3], p0, p1);
                pk[c >> 1] = pack_bf16x2(p0, p1);
            }
            l_run = l_run * alpha + (((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y)) + ((sum2[2].x + sum2[2].y) + (sum2[3].x + sum2[3].y)));
            if (Cfg::kSeparateP && j > 0) {  // P_{j-1} V_{j-1} must have read the P columns (and updated O)
                mbar_wait(&bars.o_done, (j - 1) & 1, &abort_flag, a.fault_word, 0x31);
                tc_fence_after();
            }
#pragma unroll
            for (int c = 0; c < kBN / 2; c += 32) tmem_st32(tmem_addr(tmem, lane_base, Cfg::kColP + c), &pk[c]);
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                // bring the O accumulator to the new reference (rows that did not move use alpha = 1)
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem_addr(tmem, lane_base, Cfg::kColO + c), ov);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                    tmem_st32(tmem_addr(tmem, lane_base, Cfg::kColO + c), ov);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars.p_full);
        }
        // ---- epilogue: O / l
        mbar_wait(&bars.o_done, (n_kv - 1) & 1, &abort_flag, a.fault_word, 0x32);
        tc_fence_after();
        const float inv_l = 1.0f / l_run;
        const int row_g = qt * kBM + r;
        const long long stat_idx = (long long)bh * a.T + row_g;
        if (row_g < a.T) {
            // exported statistics are relative to the true row maximum
            if (a.m_out) a.m_out[stat_idx] = m_true * kLn2;
            if (a.l_out) a.l_out[stat_idx] = l_run * exp2f(m_ref - m_true);
            if (a.lse_out) a.lse_out[stat_idx] = (m_ref + log2f(l_run)) * kLn2;
        }
#pragma unroll
        for (int c = 0; c < D; c += 32) {
            uint32_t ov[32];
            tmem_ld32(tmem_addr(tmem, lane_base, Cfg::kColO + c), ov);
            tmem_wait_ld();
            if constexpr (OUT_F32) {
                if (row_g < a.T) {
                    float* dst = reinterpret_cast<float*>(a.out) + ((long long)bh * a.T + row_g) * D + c;
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(dst + i) =
                            make_float4(__uint_as_float(ov[i]) * inv_l, __uint_as_float(ov[i + 1]) * inv_l,
                                        __uint_as_float(ov[i + 2]) * inv_l, __uint_as_float(ov[i + 3]) * inv_l);
                }
            } else {
                // stage BF16 rows in the (now idle) Q buffer, swizzled the way the TMA store expects
                uint8_t* atom = sQ + (c >> 6) * kAtomBytes;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 w;
                    w.x = pack_bf16x2(__uint_as_float(ov[i]) * inv_l, __uint_as_float(ov[i + 1]) * inv_l);
                    w.y = pack_bf16x2(__uint_as_float(ov[i + 2]) * inv_l, __uint_as_float(ov[i + 3]) * inv_l);
                    w.z = pack_bf16x2(__uint_as_float(ov[i + 4]) * inv_l, __uint_as_float(ov[i + 5]) * inv_l);
                    w.w = pack_bf16x2(__uint_as_float(ov[i + 6]) * inv_l, __uint_as_float(ov[i + 7]) * inv_l);
                    *reinterpret_cast<uint4*>(atom + swz128(r, ((c & 63) + i) >> 3)) = w;
                }
            }
        }
        if constexpr (!OUT_F32) {
            fence_proxy_async_smem();
            named_bar_sync(1, kSoftmaxThreads);
            if (tid == 0) {
                for (int at = 0; at < Cfg::kAtoms; ++at) tma_store_4d(&a.map_o, sQ + at * kAtomBytes, at * 64, qt * kBM, hh, bb);
                tma_store_commit();
                tma_store_wait_read();  // the staging tile must outlive the bulk read; the write completes with the grid
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem, Cfg::kTmemCols);
}

template <int D, bool OUT_F32>
cudaError_t launch_fwd_short(const TcFwdArgs& a, cudaStream_t stream) {
    using Cfg = FwdCfg<D>;
    auto kern = attn_fwd_tc_short_kernel<D, OUT_F32>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    const int n_q_tiles = (a.T + kBM - 1) / kBM;
    const long long blocks = (long long)n_q_tiles * a.BH;
    return launch_pdl(kern, dim3((unsigned int)blocks), dim3(kThreads), Cfg::kSmemBytes, stream, a);
}

}  // namespace

cudaError_t launch_attn_fwd_tc_short(const TcFwdArgs& a, cudaStream_t stream) {
    if (a.BH == 0 || a.T == 0) return cudaSuccess;
    if (a.d == 64) return a.out_is_f32 ? launch_fwd_short<64, true>(a, stream) : launch_fwd_short<64, false>(a, stream);
    if (a.d == 128) return a.out_is_f32 ? launch_fwd_short<128, true>(a, stream) : launch_fwd_short<128, false>(a, stream);
    return cudaErrorInvalidValue;
}

}  // namespace b200attn
