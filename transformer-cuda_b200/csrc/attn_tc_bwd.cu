// Causal attention backward on the sm_100a tensor cores (tcgen05): dQ, dK, dV from Q, K, V, dO,
// the log-sum-exp of the forward pass and D = rowsum(dO*O). Computes what
// tiled_causal_attention_backward of sarimahsan/transformer-cuda computes
// (src/kernels/attention.cu:697-1011) with five GEMMs per (key tile, query tile) pair instead of the
// reference's seven dot-product passes, and for head dims 64 and 128.
//
// One CTA owns one 128-row key/value tile j of one (batch, head) slab and walks the query tiles
// i = j .. last (tiles before the diagonal are skipped). Scores are produced TRANSPOSED, so that
// thread r of the compute warps owns key row r (TMEM lane r) and the columns are queries:
//
//   S^T  = K_j Q_i^T                  (SS MMA, both operands K-major)        -> TMEM
//   dP^T = V_j dO_i^T                 (SS MMA)                               -> TMEM
//   P^T  = exp2(S^T*scale*log2e - lse2[q])   written BF16 over S^T in TMEM (queries 0-63 packed in
//                                            columns [0,32), queries 64-127 in columns [64,96))
//   dV  += P^T dO_i                   (TS MMA: A = P^T from TMEM, dO_i MN-major)
//   dS^T = P^T * (dP^T - D[q]) * scale       written BF16 to shared memory, 128B-swizzled
//   dK  += dS^T Q_i                   (SS MMA: A = dS^T K-major, Q_i MN-major)
//   dQ_i = dS K_j                     (SS MMA: the same dS^T tile read as an MN-major A, K_j MN-major)
//
// dQ_i is a partial sum over key tiles: the compute warps move it from TMEM through a swizzled
// shared-memory staging tile and add it to an FP32 accumulator in global memory with TMA
// reduce-add operations (cp.reduce.async.bulk.tensor, whole 128-byte lines) that run behind the
// next tile's work. dK and dV stay in TMEM for the whole loop and are written once.
//
// Warps 0-7 compute (warp w and w+4 share TMEM lane quadrant w%4 and split the 128 query columns of
// the transposed tiles, 64 each), warp 8 is the TMA producer (no multicast), warp 9 issues the MMAs.
// TMEM columns, D = 64:  S/P^T [0,128) dP^T [128,256) dV [256,320) dK [320,384) dQ [384,448)
//               D = 128: S/P^T [0,128) dP^T and dQ share [128,256) dV [256,384) dK [384,512)
// Every wait is bounded (tc_common.cuh).
#include "kernels.cuh"
#include "tc_common.cuh"


namespace b200attn {
namespace {

constexpr int kBQ = 128;               // query rows per inner tile
constexpr int kBKV = 128;              // key/value rows per CTA
constexpr int kAtomBytes = 128 * 128;  // 128 rows x 64 bf16, 128-byte swizzled
constexpr int kComputeThreads = 256;
constexpr int kThreads = 320;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct BwdCfg {
    static constexpr int kAtoms = D / 64;
    static constexpr int kTileBytes = kAtoms * kAtomBytes;
    static constexpr int kQStages = 2;
    static constexpr int kDoStages = (D == 64) ? 2 : 1;
    static constexpr int kDsBytes = 2 * kAtomBytes;      // 128 key rows x 128 queries, bf16
    static constexpr int kDqStageBytes = 2 * kAtomBytes;  // two 128 x 32 FP32 blocks of a dQ partial
    static constexpr int kStatBytes = 2 * 2 * kBQ * 4;    // lse2 and D of a query tile, double-buffered
    // The dynamic buffer is declared 1024-byte aligned, so no slack is added (at d = 128 the kernel
    // uses all of the 227 KB a CTA can have).
    static constexpr int kSmemBytes = kTileBytes * (2 + kQStages + kDoStages) + kDsBytes + kDqStageBytes + kStatBytes;
    static constexpr int kDqRounds = D / 64;  // 32-column blocks per thread in a dQ partial
    static constexpr bool kDqAliased = (D == 128);
    static constexpr uint32_t kTmemCols = 512;
    static constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 256 + D;
    static constexpr uint32_t kColDQ = kDqAliased ? kColDP : (256 + 2 * D);
};

struct BwdBarriers {
    uint64_t k_full, v_full;
    uint64_t q_full[2], q_empty[2], do_full[2], do_empty[2];
    uint64_t s_full, dp_full, p_ready, ds_ready, dq_full, dq_empty;
};

template <int D, bool GRADS_F32>
__global__ void __launch_bounds__(kThreads, 1) attn_bwd_tc_kernel(const __grid_constant__ TcBwdArgs a) {
    using Cfg = BwdCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;
    uint8_t* sV = sK + Cfg::kTileBytes;
    uint8_t* sQ = sV + Cfg::kTileBytes;
    uint8_t* sDO = sQ + Cfg::kQStages * Cfg::kTileBytes;
    uint8_t* sDS = sDO + Cfg::kDoStages * Cfg::kTileBytes;
    uint8_t* sDQ = sDS + Cfg::kDsBytes;  // staging of dQ partials for the TMA reduce-add
    float (*s_lse)[kBQ] = reinterpret_cast<float (*)[kBQ]>(sDQ + Cfg::kDqStageBytes);
    float (*s_D)[kBQ] = s_lse + 2;

    __shared__ BwdBarriers bars;
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t abort_flag;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    pdl_launch_dependents();

    const int n_tiles = (a.T + kBKV - 1) / kBKV;
    // CTA order. Key tile 0 sees every query tile and is the longest. When the whole problem fits in
    // L2 the CTAs are issued longest-first across ALL slabs (shortest tail); otherwise slab by slab,
    // so that the CTAs resident at one time share few slabs and their tiles stay in L2.
    const int bh = a.tile_major_order ? int(blockIdx.x % a.BH) : int(blockIdx.x / n_tiles);
    const int jt = a.tile_major_order ? int(blockIdx.x / a.BH) : int(blockIdx.x % n_tiles);
    const int hh = bh % a.H, bb = bh / a.H;  // head and batch coordinates of the 4-D tensor maps
    const int n_it = n_tiles - jt;        // query tiles jt .. n_tiles-1

    if (tid == 0) {
        mbar_init(&bars.k_full, 1);
        mbar_init(&bars.v_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars.q_full[s], 1);
            mbar_init(&bars.q_empty[s], 1);
            mbar_init(&bars.do_full[s], 1);
            mbar_init(&bars.do_empty[s], 1);
        }
        mbar_init(&bars.s_full, 1);
        mbar_init(&bars.dp_full, 1);
        mbar_init(&bars.p_ready, kComputeThreads);
        mbar_init(&bars.ds_ready, kComputeThreads);
        mbar_init(&bars.dq_full, 1);
        mbar_init(&bars.dq_empty, kComputeThreads);
        abort_flag = 0;
        if ((smem_u32(smem) & 1023u) != 0 && a.fault_word) atomicCAS(a.fault_word, 0u, kFaultWaitTimeout | 0xA11u);
        mbar_fence_init();
    }
    if (warp == kProducerWarp) {
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

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&a.map_q);
            tma_prefetch_desc(&a.map_k);
            tma_prefetch_desc(&a.map_v);
            tma_prefetch_desc(&a.map_do);
            mbar_expect_tx(&bars.k_full, Cfg::kTileBytes);
            for (int at = 0; at < Cfg::kAtoms; ++at)
                tma_load_4d(sK + at * kAtomBytes, &a.map_k, &bars.k_full, at * 64, jt * kBKV, hh, bb);
            mbar_expect_tx(&bars.v_full, Cfg::kTileBytes);
            for (int at = 0; at < Cfg::kAtoms; ++at)
                tma_load_4d(sV + at * kAtomBytes, &a.map_v, &bars.v_full, at * 64, jt * kBKV, hh, bb);
            for (int it = 0; it < n_it; ++it) {
                const int i = jt + it;
                const int qs = it % Cfg::kQStages;
                if (it >= Cfg::kQStages)
                    mbar_wait(&bars.q_empty[qs], (it / Cfg::kQStages - 1) & 1, &abort_flag, a.fault_word, 0x40);
                mbar_expect_tx(&bars.q_full[qs], Cfg::kTileBytes);
                for (int at = 0; at < Cfg::kAtoms; ++at)
                    tma_load_4d(sQ + qs * Cfg::kTileBytes + at * kAtomBytes, &a.map_q, &bars.q_full[qs], at * 64, i * kBQ, hh, bb);
                const int os = it % Cfg::kDoStages;
                if (it >= Cfg::kDoStages)
                    mbar_wait(&bars.do_empty[os], (it / Cfg::kDoStages - 1) & 1, &abort_flag, a.fault_word, 0x41);
                mbar_expect_tx(&bars.do_full[os], Cfg::kTileBytes);
                for (int at = 0; at < Cfg::kAtoms; ++at)
                    tma_load_4d(sDO + os * Cfg::kTileBytes + at * kAtomBytes, &a.map_do, &bars.do_full[os], at * 64, i * kBQ, hh, bb);
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_st = make_idesc_bf16(kBKV, kBQ, 0, 0);  // S^T, dP^T
        constexpr uint32_t idesc_kv = make_idesc_bf16(kBKV, D, 0, 1);    // dV, dK: B is MN-major
        constexpr uint32_t idesc_dq = make_idesc_bf16(kBQ, D, 1, 1);     // dQ: A and B MN-major
        const uint64_t k_kmaj = make_smem_desc_sw128(smem_u32(sK), 0, 1024);
        const uint64_t v_kmaj = make_smem_desc_sw128(smem_u32(sV), 0, 1024);
        const uint64_t k_mnmaj = make_smem_desc_sw128(smem_u32(sK), kAtomBytes, 1024);
        const uint64_t ds_kmaj = make_smem_desc_sw128(smem_u32(sDS), 0, 1024);
        const uint64_t ds_mnmaj = make_smem_desc_sw128(smem_u32(sDS), kAtomBytes, 1024);

        auto issue_st = [&](int it) {  // S^T(it) = K_j Q^T
            const int qs = it % Cfg::kQStages;
            mbar_wait(&bars.q_full[qs], (it / Cfg::kQStages) & 1, &abort_flag, a.fault_word, 0x50);
            tc_fence_after();
            if (elect_one()) {
                const uint64_t q_kmaj = make_smem_desc_sw128(smem_u32(sQ + qs * Cfg::kTileBytes), 0, 1024);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kAtomBytes + (kk & 3) * 32;
                    tc_mma_ss(tmem + Cfg::kColS, desc_advance(k_kmaj, off), desc_advance(q_kmaj, off), idesc_st, kk > 0);
                }
                tc_commit(&bars.s_full);
            }
            __syncwarp();
        };
        auto issue_dp = [&](int it) {  // dP^T(it) = V_j dO^T
            const int os = it % Cfg::kDoStages;
            mbar_wait(&bars.do_full[os], (it / Cfg::kDoStages) & 1, &abort_flag, a.fault_word, 0x51);
            if (Cfg::kDqAliased && it > 0)  // the dQ partial of the previous tile sits in these columns
                mbar_wait(&bars.dq_empty, (it - 1) & 1, &abort_flag, a.fault_word, 0x52);
            tc_fence_after();
            if (elect_one()) {
                const uint64_t do_kmaj = make_smem_desc_sw128(smem_u32(sDO + os * Cfg::kTileBytes), 0, 1024);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kAtomBytes + (kk & 3) * 32;
                    tc_mma_ss(tmem + Cfg::kColDP, desc_advance(v_kmaj, off), desc_advance(do_kmaj, off), idesc_st, kk > 0);
                }
                tc_commit(&bars.dp_full);
            }
            __syncwarp();
        };

        mbar_wait(&bars.k_full, 0, &abort_flag, a.fault_word, 0x53);
        mbar_wait(&bars.v_full, 0, &abort_flag, a.fault_word, 0x54);
        issue_st(0);
        issue_dp(0);
        for (int it = 0; it < n_it; ++it) {
            const int qs = it % Cfg::kQStages;
            const int os = it % Cfg::kDoStages;
            // dV += P^T dO
            mbar_wait(&bars.p_ready, it & 1, &abort_flag, a.fault_word, 0x55);
            tc_fence_after();
            if (elect_one()) {
                const uint64_t do_mnmaj = make_smem_desc_sw128(smem_u32(sDO + os * Cfg::kTileBytes), kAtomBytes, 1024);
#pragma unroll
                for (int kk = 0; kk < kBQ / 16; ++kk)
                    tc_mma_ts(tmem + Cfg::kColDV, tmem + Cfg::kColS + (kk >> 2) * 64 + (kk & 3) * 8,
                              desc_advance(do_mnmaj, kk * 2048), idesc_kv, (it > 0) || (kk > 0));
                tc_commit(&bars.do_empty[os]);  // dP^T(it) and dV(it) were the readers of this dO tile
            }
            __syncwarp();
            if (it + 1 < n_it) issue_st(it + 1);  // overlaps the exponentials of the next tile with dK/dQ of this one
            // dK += dS^T Q ; dQ = dS K
            mbar_wait(&bars.ds_ready, it & 1, &abort_flag, a.fault_word, 0x56);
            // dS^T(it) done means dP^T(it) has been consumed: with dQ in its own columns the next dP^T can go first
            if (!Cfg::kDqAliased && it + 1 < n_it) issue_dp(it + 1);
            tc_fence_after();
            if (elect_one()) {
                const uint64_t q_mnmaj = make_smem_desc_sw128(smem_u32(sQ + qs * Cfg::kTileBytes), kAtomBytes, 1024);
#pragma unroll
                for (int kk = 0; kk < kBQ / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kAtomBytes + (kk & 3) * 32;
                    tc_mma_ss(tmem + Cfg::kColDK, desc_advance(ds_kmaj, off), desc_advance(q_mnmaj, kk * 2048), idesc_kv,
                                  (it > 0) || (kk > 0));
                }
                tc_commit(&bars.q_empty[qs]);  // S^T(it) and dK(it) were the readers of this Q tile
            }
            __syncwarp();
            if (!Cfg::kDqAliased && it > 0) {  // previous dQ partial must have been read out of its columns
                mbar_wait(&bars.dq_empty, (it - 1) & 1, &abort_flag, a.fault_word, 0x57);
                tc_fence_after();
            }
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < kBKV / 16; ++kk)
                    tc_mma_ss(tmem + Cfg::kColDQ, desc_advance(ds_mnmaj, kk * 2048), desc_advance(k_mnmaj, kk * 2048),
                              idesc_dq, kk > 0);
                tc_commit(&bars.dq_full);
            }
            __syncwarp();
            if (Cfg::kDqAliased && it + 1 < n_it) issue_dp(it + 1);
        }
    } else {
        // ------------------------------------------------------------ compute warps: thread (r, half) =
        // key row r (TMEM lane r), query columns [64*half, 64*half + 64) of the transposed tiles
        const int r = tid & 127;
        const int half = tid >> 7;
        const int c_begin = half * (kBQ / 2);
        const uint32_t lane_base = uint32_t(warp & 3) * 32u;
        const float scale_log2 = a.scale * kLog2e;
        const long long stat_base = (long long)bh * a.T;

        // A dQ partial (query tile jt+it) travels TMEM -> registers -> a 128-byte-swizzled staging
        // tile -> TMA reduce-add into the FP32 accumulator in global memory (whole 128-byte lines
        // instead of scattered atomics). Here thread (r, half) owns QUERY row r and the head-dim
        // columns of its half; `dqv` holds them between the two steps below.
        // One SM sustains only about 16 bytes/clock of FP32 reductions, so the reduce runs
        // asynchronously behind the next tile's work and is waited for only when the staging tile is
        // needed again; at d = 128 the partial is sent in two rounds of 32 columns per thread.
        uint32_t dqv[D / 2];
        auto dq_fetch = [&](int it) {  // TMEM -> registers; frees the dQ columns for the MMA warp
            mbar_wait(&bars.dq_full, it & 1, &abort_flag, a.fault_word, 0x60);
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < D / 2; c += 32) tmem_ld32(tmem_addr(tmem, lane_base, Cfg::kColDQ + half * (D / 2) + c), &dqv[c]);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&bars.dq_empty);
        };
        auto dq_send = [&](int it, int rd) {  // registers -> staging -> reduce-add, 32 columns per thread
            if (tid == 0) tma_store_wait_read();  // earlier reductions have finished reading the staging tile
            named_bar_sync(2, kComputeThreads);
            uint8_t* stage = sDQ + half * kAtomBytes;
#pragma unroll
            for (int x = 0; x < 32; x += 4)
                *reinterpret_cast<uint4*>(stage + swz128(r, x >> 2)) =
                    make_uint4(dqv[rd * 32 + x], dqv[rd * 32 + x + 1], dqv[rd * 32 + x + 2], dqv[rd * 32 + x + 3]);
            fence_proxy_async_smem();
            named_bar_sync(2, kComputeThreads);
            if (tid == 0) {
                tma_reduce_add_4d(&a.map_dq_acc, sDQ, rd * 32, (jt + it) * kBQ, hh, bb);
                tma_reduce_add_4d(&a.map_dq_acc, sDQ + kAtomBytes, D / 2 + rd * 32, (jt + it) * kBQ, hh, bb);
                tma_store_commit();
            }
        };

        // statistics of the first query tile; later tiles are fetched one iteration ahead
        // Per-query statistics (column c of the transposed tiles is query i*128 + c): half 0 threads carry
        // lse2[q = r], half 1 threads D[q = r], fetched one tile ahead and stored into the other buffer
        // at the END of a step, where the barrier of the dQ drain publishes them; so no barrier of their
        // own stands in front of the exponentials.
        auto load_stat = [&](int i) -> float {
            const int q_g = i * kBQ + r;
            return (half == 0) ? ((q_g < a.T) ? a.lse2[stat_base + q_g] : INFINITY)  // +inf beyond T -> P = 0
                               : ((q_g < a.T) ? a.D[stat_base + q_g] : 0.f);
        };
        auto store_stat = [&](int buf, float v) {
            if (half == 0) s_lse[buf][r] = v;
            else s_D[buf][r] = v;
        };
        store_stat(0, load_stat(jt));
        float stat_next = (n_it > 1) ? load_stat(jt + 1) : 0.f;
        named_bar_sync(1, kComputeThreads);

        for (int it = 0; it < n_it; ++it) {
            const int i = jt + it;
            const int buf = it & 1;

            // ---- P^T
            mbar_wait(&bars.s_full, it & 1, &abort_flag, a.fault_word, 0x61);
            tc_fence_after();
            float p[kBQ / 2];
            const bool diag = (i == jt);
#pragma unroll
            for (int cc = 0; cc < kBQ / 2; cc += 32) {
                const int c = c_begin + cc;
                uint32_t sv[32];
                tmem_ld32(tmem_addr(tmem, lane_base, Cfg::kColS + c), sv);
                tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int x = 0; x < 32; x += 4) {
                    const float4 ls = *reinterpret_cast<const float4*>(&s_lse[buf][c + x]);
                    const float l4[4] = {ls.x, ls.y, ls.z, ls.w};
#pragma unroll
                    for (int y = 0; y < 4; ++y) {
                        float e = mixed_exp2(fmaf(__uint_as_float(sv[x + y]), scale_log2, -l4[y]), y);
                        if (diag && (c + x + y) < r) e = 0.f;  // query before this key: masked
                        p[cc + x + y] = e;
                    }
                    pk[x >> 1] = pack_bf16x2(p[cc + x], p[cc + x + 1]);
                    pk[(x >> 1) + 1] = pack_bf16x2(p[cc + x + 2], p[cc + x + 3]);
                }
                // each half packs its P^T into the first 32 columns of its OWN 64 score columns, so the
                // other half's unread scores are never overwritten
                tmem_st16(tmem_addr(tmem, lane_base, Cfg::kColS + c_begin + (cc >> 1)), pk);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars.p_ready);

            // ---- d = 128: the previous tile's dQ partial sits in the dP^T columns and has to leave before
            // dP^T of this tile can be produced (its MMA ran while the exponentials above were computed)
            if (Cfg::kDqAliased && it > 0) {
                dq_fetch(it - 1);
                dq_send(it - 1, 0);
            }

            // ---- dS^T
            mbar_wait(&bars.dp_full, it & 1, &abort_flag, a.fault_word, 0x62);
            // the dS^T tile in shared memory is still being read by dK / dQ of the previous step until the
            // commit behind that dQ has arrived (at d = 128 the drain above has already waited for it)
            if (!Cfg::kDqAliased && it > 0) mbar_wait(&bars.dq_full, (it - 1) & 1, &abort_flag, a.fault_word, 0x66);
            tc_fence_after();
            {
                // both TMEM loads and the statistics are requested before the single wait: chunk-by-chunk
                // (load, wait, compute, store) exposed the load latency twice and measured 860 cycles
                // for this pass against 490 in this form
                uint32_t dv[kBQ / 2];
#pragma unroll
                for (int cc = 0; cc < kBQ / 2; cc += 32) tmem_ld32(tmem_addr(tmem, lane_base, Cfg::kColDP + c_begin + cc), &dv[cc]);
                float dd[kBQ / 2];
#pragma unroll
                for (int x = 0; x < kBQ / 2; x += 4) {
                    const float4 t = *reinterpret_cast<const float4*>(&s_D[buf][c_begin + x]);
                    dd[x] = t.x, dd[x + 1] = t.y, dd[x + 2] = t.z, dd[x + 3] = t.w;
                }
                tmem_wait_ld();
#pragma unroll
                for (int x = 0; x < kBQ / 2; x += 8) {
                    float ds[8];
#pragma unroll
                    for (int y = 0; y < 8; ++y) ds[y] = (p[x + y] * a.scale) * (__uint_as_float(dv[x + y]) - dd[x + y]);
                    uint4 w;
                    w.x = pack_bf16x2(ds[0], ds[1]);
                    w.y = pack_bf16x2(ds[2], ds[3]);
                    w.z = pack_bf16x2(ds[4], ds[5]);
                    w.w = pack_bf16x2(ds[6], ds[7]);
                    const int qc = c_begin + x;  // first query column of this 16-byte chunk
                    *reinterpret_cast<uint4*>(sDS + (qc >> 6) * kAtomBytes + swz128(r, (qc & 63) >> 3)) = w;
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(&bars.ds_ready);
            // ---- statistics of the next tile, then the (rest of the) previous tile's dQ partial; the
            // barrier inside dq_send (or the explicit one on the first step) publishes the statistics
            if (it + 1 < n_it) {
                store_stat(buf ^ 1, stat_next);
                if (it + 2 < n_it) stat_next = load_stat(i + 2);
            }
            if (it == 0) {
                named_bar_sync(1, kComputeThreads);
            } else if (Cfg::kDqAliased) {
                dq_send(it - 1, 1);  // second half of the previous partial
            } else {
                dq_fetch(it - 1);
                dq_send(it - 1, 0);
            }
        }
        dq_fetch(n_it - 1);  // dq_full of the last tile also means every dV / dK MMA has retired
        dq_send(n_it - 1, 0);
        if (Cfg::kDqRounds == 2) dq_send(n_it - 1, 1);

        // ---- epilogue: dV and dK of this key tile
        const int kv_g = jt * kBKV + r;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const uint32_t col0 = which == 0 ? Cfg::kColDV : Cfg::kColDK;
            void* gout = which == 0 ? a.dv : a.dk;
            uint8_t* stage = sQ + which * Cfg::kTileBytes;  // Q stages are idle now
#pragma unroll
            for (int c = half * (D / 2); c < (half + 1) * (D / 2); c += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_addr(tmem, lane_base, col0 + c), v);
                tmem_wait_ld();
                if constexpr (GRADS_F32) {
                    if (kv_g < a.T) {
                        float* dst = reinterpret_cast<float*>(gout) + (stat_base + kv_g) * D + c;
#pragma unroll
                        for (int x = 0; x < 32; x += 4)
                            *reinterpret_cast<float4*>(dst + x) =
                                make_float4(__uint_as_float(v[x]), __uint_as_float(v[x + 1]), __uint_as_float(v[x + 2]),
                                            __uint_as_float(v[x + 3]));
                    }
                } else {
                    uint8_t* atom = stage + (c >> 6) * kAtomBytes;
#pragma unroll
                    for (int x = 0; x < 32; x += 8) {
                        uint4 w;
                        w.x = pack_bf16x2(__uint_as_float(v[x]), __uint_as_float(v[x + 1]));
                        w.y = pack_bf16x2(__uint_as_float(v[x + 2]), __uint_as_float(v[x + 3]));
                        w.z = pack_bf16x2(__uint_as_float(v[x + 4]), __uint_as_float(v[x + 5]));
                        w.w = pack_bf16x2(__uint_as_float(v[x + 6]), __uint_as_float(v[x + 7]));
                        *reinterpret_cast<uint4*>(atom + swz128(r, ((c & 63) + x) >> 3)) = w;
                    }
                }
            }
        }
        if constexpr (!GRADS_F32) {
            fence_proxy_async_smem();
            named_bar_sync(1, kComputeThreads);
            if (tid == 0) {
                for (int at = 0; at < Cfg::kAtoms; ++at) {
                    tma_store_4d(&a.map_dv, sQ + at * kAtomBytes, at * 64, jt * kBKV, hh, bb);
                    tma_store_4d(&a.map_dk, sQ + Cfg::kTileBytes + at * kAtomBytes, at * 64, jt * kBKV, hh, bb);
                }
                tma_store_commit();
            }
        }
        // shared memory must outlive the bulk reads of every store / reduce issued by this thread;
        // their global writes complete before the grid does
        if (tid == 0) tma_store_wait_read();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kProducerWarp) tmem_dealloc(tmem, Cfg::kTmemCols);
}

// ------------------------------------------------------------------ pre-pass
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}
// -x/2 as three BF16 pieces (24 significant bits), twice: the 32-byte statistics row of BwdStatRows
__device__ __forceinline__ void store_stat_row(__nv_bfloat16* dst_row, float x) {
    const float v = -0.5f * x;
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h);
    const __nv_bfloat16 m = __float2bfloat16_rn(r1);
    const __nv_bfloat16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
    uint4 w;
    w.x = uint32_t(__bfloat16_as_ushort(h)) | (uint32_t(__bfloat16_as_ushort(m)) << 16);
    w.y = uint32_t(__bfloat16_as_ushort(l));
    w.z = 0u, w.w = 0u;
    reinterpret_cast<uint4*>(dst_row)[0] = w;
    reinterpret_cast<uint4*>(dst_row)[1] = w;
}
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

// D[row] = sum_e dO*O and lse2[row] = log-sum-exp in log2 units. A row is shared by d/VEC adjacent
// threads, 16 bytes (VEC elements) each, so a warp's loads are contiguous; the partial sums meet in a
// sub-warp shuffle reduction. When `zero` is given, the same threads clear the FP32 dQ accumulator
// row (4*d bytes) so that no separate memset pass is needed.
template <typename TIn>
__global__ void __launch_bounds__(256) bwd_prepass_kernel(const TIn* __restrict__ o, const TIn* __restrict__ dO,
                                                         const float* __restrict__ m, const float* __restrict__ l,
                                                         const float* __restrict__ lse, float* __restrict__ Dout,
                                                         float* __restrict__ lse2, float* __restrict__ zero,
                                                         long long rows, int d, unsigned int* counter, BwdStatRows ext) {
    constexpr int VEC = 16 / sizeof(TIn);
    pdl_launch_dependents();
    pdl_wait();
    const int tpr = d / VEC;  // threads per row: a power of two <= 32
    const long long gid = blockIdx.x * 256ll + threadIdx.x;
    if (gid == 0 && counter) *counter = 0u;  // the persistent backward that follows hands out work items from it
    const long long row = gid / tpr;
    const int e = int(gid % tpr) * VEC;
    float acc = 0.f;
    if (row < rows) {
        uint4 ua = __ldg(reinterpret_cast<const uint4*>(o + row * d + e));
        uint4 ub = __ldg(reinterpret_cast<const uint4*>(dO + row * d + e));
        const TIn* pa = reinterpret_cast<const TIn*>(&ua);
        const TIn* pb = reinterpret_cast<const TIn*>(&ub);
#pragma unroll
        for (int x = 0; x < VEC; ++x) acc = fmaf(to_f32(pa[x]), to_f32(pb[x]), acc);
        if (zero) {
            float4* z = reinterpret_cast<float4*>(zero + row * d + e);
#pragma unroll
            for (int x = 0; x < VEC / 4; ++x) z[x] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    for (int off = tpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (row < rows && e == 0) {
        Dout[row] = acc;
        if (lse2 || ext.lse_ext) {
            const float lse_nat = lse ? lse[row] : (m[row] + logf(l[row]));
            if (lse2) lse2[row] = lse_nat * kLog2e;
            if (ext.lse_ext) {
                store_stat_row(ext.lse_ext + row * 16, lse_nat * ext.inv_scale);
                store_stat_row(ext.d_ext + row * 16, acc);
            }
        }
    }
}

// Pre-pass on BF16 O / dO whose rows are addressed through strides (merged (B, T, H*d) layout): eight threads per
// 64-wide row (sixteen per 128), 16 bytes each. D, lse2 and the dQ accumulator stay dense (B*H, T[, d]).
__global__ void __launch_bounds__(256) bwd_prepass_strided_kernel(const __nv_bfloat16* __restrict__ o,
                                                                 const __nv_bfloat16* __restrict__ dO,
                                                                 const float* __restrict__ lse, float* __restrict__ Dout,
                                                                 float* __restrict__ lse2, float* __restrict__ zero,
                                                                 long long rows, int d, int T, int H, long long lt,
                                                                 long long lh, long long lb, unsigned int* counter,
                                                                 BwdStatRows ext) {
    pdl_launch_dependents();
    pdl_wait();
    const int tpr = d / 8;
    const long long gid = blockIdx.x * 256ll + threadIdx.x;
    if (gid == 0 && counter) *counter = 0u;
    const long long row = gid / tpr;
    const int e = int(gid % tpr) * 8;
    float acc = 0.f;
    if (row < rows) {
        const long long bh = row / T;
        const int t = int(row - bh * T);
        const long long src = (bh / H) * lb + (bh % H) * lh + (long long)t * lt + e;
        const uint4 ua = __ldg(reinterpret_cast<const uint4*>(o + src));
        const uint4 ub = __ldg(reinterpret_cast<const uint4*>(dO + src));
        const __nv_bfloat16* pa = reinterpret_cast<const __nv_bfloat16*>(&ua);
        const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&ub);
#pragma unroll
        for (int x = 0; x < 8; ++x) acc = fmaf(__bfloat162float(pa[x]), __bfloat162float(pb[x]), acc);
        float4* z = reinterpret_cast<float4*>(zero + row * d + e);
        z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int off = tpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (row < rows && e == 0) {
        Dout[row] = acc;
        lse2[row] = lse[row] * kLog2e;
        if (ext.lse_ext) {
            store_stat_row(ext.lse_ext + row * 16, lse[row] * ext.inv_scale);
            store_stat_row(ext.d_ext + row * 16, acc);
        }
    }
}

// dQ accumulator (dense FP32 rows) -> BF16 rows addressed through strides; one thread per 8 elements.
__global__ void __launch_bounds__(256) dq_convert_strided_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                                                long long rows, int d, int T, int H, long long lt,
                                                                long long lh, long long lb, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int tpr = d / 8;
    const long long gid = blockIdx.x * 256ll + threadIdx.x;
    const long long row = gid / tpr;
    const int e = int(gid % tpr) * 8;
    if (row >= rows) return;
    const long long bh = row / T;
    const int t = int(row - bh * T);
    const float4 a0 = __ldg(reinterpret_cast<const float4*>(acc + row * d + e));
    const float4 a1 = __ldg(reinterpret_cast<const float4*>(acc + row * d + e + 4));
    uint4 w;
    w.x = pack_bf16x2(a0.x * scale, a0.y * scale);
    w.y = pack_bf16x2(a0.z * scale, a0.w * scale);
    w.z = pack_bf16x2(a1.x * scale, a1.y * scale);
    w.w = pack_bf16x2(a1.z * scale, a1.w * scale);
    *reinterpret_cast<uint4*>(dq + (bh / H) * lb + (bh % H) * lh + (long long)t * lt + e) = w;
}

template <int D, bool GRADS_F32>
cudaError_t launch_bwd(const TcBwdArgs& a, cudaStream_t stream) {
    using Cfg = BwdCfg<D>;
    auto kern = attn_bwd_tc_kernel<D, GRADS_F32>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    const int n_tiles = (a.T + kBKV - 1) / kBKV;
    const long long blocks = (long long)n_tiles * a.BH;
    return launch_pdl(kern, dim3((unsigned int)blocks), dim3(kThreads), Cfg::kSmemBytes, stream, a);
}

}  // namespace

cudaError_t launch_attn_bwd_tc(const TcBwdArgs& a, cudaStream_t stream) {
    if (a.BH == 0 || a.T == 0) return cudaSuccess;
    if (a.d == 64 && a.work_counter != nullptr) return launch_attn_bwd_tc64(a, stream);
    if (a.d == 64) return a.grads_are_f32 ? launch_bwd<64, true>(a, stream) : launch_bwd<64, false>(a, stream);
    if (a.d == 128) return a.grads_are_f32 ? launch_bwd<128, true>(a, stream) : launch_bwd<128, false>(a, stream);
    return cudaErrorInvalidValue;
}

template <typename TIn>
cudaError_t launch_bwd_prepass(const TIn* o, const TIn* dO, const float* m, const float* l, const float* lse, float* D,
                               float* lse2, float* zero, long long rows, int d, cudaStream_t stream, unsigned int* counter,
                               BwdStatRows ext) {
    if (rows == 0) return cudaSuccess;
    constexpr int VEC = 16 / sizeof(TIn);
    const int tpr = d / VEC;
    if (d % VEC != 0 || tpr > 32 || (tpr & (tpr - 1)) != 0) return cudaErrorInvalidValue;
    const long long threads = rows * tpr;
    return launch_pdl(bwd_prepass_kernel<TIn>, dim3((unsigned int)((threads + 255) / 256)), dim3(256), 0, stream, o, dO, m, l, lse,
                      D, lse2, zero, rows, d, counter, ext);
}
template cudaError_t launch_bwd_prepass<float>(const float*, const float*, const float*, const float*, const float*,
                                              float*, float*, float*, long long, int, cudaStream_t, unsigned int*, BwdStatRows);
template cudaError_t launch_bwd_prepass<__nv_bfloat16>(const __nv_bfloat16*, const __nv_bfloat16*, const float*,
                                                      const float*, const float*, float*, float*, float*, long long,
                                                      int, cudaStream_t, unsigned int*, BwdStatRows);

cudaError_t launch_bwd_prepass_strided(const __nv_bfloat16* o, const __nv_bfloat16* dO, const float* lse, float* D,
                                       float* lse2, float* zero, long long rows, int d, int T, int H, long long lt,
                                       long long lh, long long lb, cudaStream_t stream, unsigned int* counter, BwdStatRows ext) {
    if (rows == 0) return cudaSuccess;
    const int tpr = d / 8;
    if (d % 8 != 0 || tpr > 32 || (tpr & (tpr - 1)) != 0 || !lse || !lse2 || !zero) return cudaErrorInvalidValue;
    const long long threads = rows * tpr;
    return launch_pdl(bwd_prepass_strided_kernel, dim3((unsigned int)((threads + 255) / 256)), dim3(256), 0, stream, o, dO, lse, D,
                      lse2, zero, rows, d, T, H, lt, lh, lb, counter, ext);
}

cudaError_t launch_dq_convert_strided(const float* dq_acc, __nv_bfloat16* dq, long long rows, int d, int T, int H,
                                      long long lt, long long lh, long long lb, cudaStream_t stream, float scale) {
    if (rows == 0) return cudaSuccess;
    if (d % 8 != 0) return cudaErrorInvalidValue;
    const long long threads = rows * (d / 8);
    return launch_pdl(dq_convert_strided_kernel, dim3((unsigned int)((threads + 255) / 256)), dim3(256), 0, stream, dq_acc, dq, rows,
                      d, T, H, lt, lh, lb, scale);
}

cudaError_t launch_dq_convert(const float* dq_acc, __nv_bfloat16* dq, long long n, cudaStream_t stream, float scale) {
    return launch_f32_to_bf16(dq_acc, dq, n, stream, scale);
}

}  // namespace b200attn
