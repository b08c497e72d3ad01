// Causal attention backward for head dim 64 on the sm_100a tensor cores: a persistent, role-specialised
// variant of the kernel in attn_tc_bwd.cu (which keeps head dim 128). Same arithmetic
// (tiled_causal_attention_backward of sarimahsan/transformer-cuda, src/kernels/attention.cu:697-1011, five
// GEMMs per (key tile, query tile) pair), different schedule:
//
//   * One CTA per SM walks a stream of work items, an item being one 128-row key/value tile of one
//     (batch, head) slab; items are handed out longest-first from an atomic counter, so the per-CTA
//     prologue (barriers, TMEM, first loads) is paid once per SM instead of once per item and the loads,
//     first S^T and first exponentials of the next item run under the tail of the current one.
//   * The 256 compute threads are split by PHASE instead of by columns: group A (warps 0-3) turns S^T into
//     P^T (the exponentials, bound by the 16/clk special-function unit), group B (warps 4-7) turns dP^T and
//     P^T into dS^T, moves the dQ partials out and writes dK / dV of finished items. A works on step g+1 while
//     B works on step g and the tensor pipe on both, so a step no longer costs the SUM of the phases.
//   * Three warps issue MMAs (S^T | dP^T and dV | dK and dQ): one issuing thread spent about 3400 cycles per
//     step inside its issue sequences (clock64 trace), more than twice the 1536 cycles the MMAs execute in.
//   * The per-query statistics never pass through the compute threads: the pre-pass stores -lse/scale and -D
//     of every query row as three BF16 pieces (hi + mid + lo, 24 significant bits), TMA brings the 128 rows of a
//     query tile in beside Q / dO, and one extra K = 16 step of the S^T / dP^T MMAs against a tile of ones
//     adds them to every key row: TMEM then holds S^T - lse/scale and dP^T - D, and the inner loops of both
//     groups are register-only (the broadcast shared-memory loads they replace left a lone warp per scheduler
//     exposed to their latency: 2400 and 3200 cycles per pass instead of 1100 and 700).
//   * Group A reads its score row in chunks of 32 queries inside a rolled loop (the next chunk's TMEM load in flight
//     under the exponentials of this one) and hands the S^T columns back after the last load; P^T has its own 64
//     TMEM columns, so S^T of the next step is produced under the second half of the exponentials of this one.
//   * Code size is part of the design: with six roles running different code on one SM, the first complete version
//     (100 KB of instructions, every loop unrolled, every wait inlined) had an instruction-cache hit rate of 67 % and
//     "no instruction" as its top stall reason; rolled loops, an out-of-line polling loop and an out-of-line item
//     decode brought it to 48 KB, 86 % and 76 -> 62 us at B8 H12 T1024.
//
// Per step (key tile j, query tile i), thread r of either group owns key row r = TMEM lane r:
//   S^T  = K_j Q_i^T - 1 (lse/scale)^T     SS MMA (4 + 1 K-steps) -> TMEM [0,128)
//   P^T  = exp2(S^T * scale*log2e)                     group A -> TMEM [448,512) as packed BF16
//   dV  += P^T dO_i                         TS MMA (A operand = P^T in TMEM)
//   dP^T = V_j dO_i^T - 1 D^T               SS MMA (4 + 1 K-steps) -> TMEM [128,256)
//   dS^T = P^T * dP^T  (FP32 product, rounded once)    group B -> shared memory, 128B-swizzled
//   dK  += dS^T Q_i                         SS MMA (dS^T K-major); multiplied by the softmax scale when stored
//   dQ_i = dS K_j                           SS MMA (the same tile read MN-major) -> TMEM [384,448) -> group B ->
//                                           staging tile -> TMA reduce-add into the FP32 accumulator; the scale is
//                                           applied by the FP32 -> BF16 conversion of dQ (FP32 gradients: here)
// Query rows beyond T need no mask: their Q, dO and statistics rows are zero-filled by TMA, so P^T = 1 there meets
// dO = 0 and dP^T = 0. TMEM columns: S^T [0,128) dP^T [128,256) dV [256,320) dK [320,384) dQ [384,448) P^T [448,512).
// No TMA multicast anywhere; every wait is bounded (tc_common.cuh).
#include <type_traits>

#include "kernels.cuh"
#include "tc_common.cuh"
#include "trace.cuh"

// debug builds: stamps of CTA 0, slot = role * 2048 + step * 16 + point
// (role 0 group A thread 0, 1 group B thread 0, 2 / 3 / 4 the S^T / dP^T+dV / dK+dQ issuing warps)
B200ATTN_TRACE_DEFINE(bwd64, 5 * 2048)
#define T64(role, g, point) B200ATTN_TRACE_POINT(bwd64, blockIdx.x == 0 && (g) < 128, (role) * 2048 + (g) * 16 + (point))

namespace b200attn {
namespace {

constexpr int kBQ = 128;               // query rows per step
constexpr int kBKV = 128;              // key/value rows per work item
constexpr int kD = 64;
constexpr int kTileBytes = 128 * 128;  // 128 rows x 64 bf16, 128-byte swizzled (one "atom")
constexpr int kExtBytes = 128 * 32;    // 128 rows x 16 bf16 (the statistics pieces of a query tile), 32-byte swizzled
constexpr int kGroupThreads = 128;
constexpr int kThreads = 384;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarpS = 9, kMmaWarpV = 10, kMmaWarpK = 11;
constexpr int kKStages = 2, kQStages = 3, kDoStages = 2;
constexpr int kItemRing = 4;
constexpr float kLog2e = 1.4426950408889634f;

constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 320, kColDQ = 384, kColP = 448;
constexpr uint32_t kTmemCols = 512;

// Shared memory: K x2, V x1, Q x3, dO x2 (16 KB each), dS^T (32 KB), dQ staging (32 KB), the statistics tiles that
// travel with Q (x3) and dO (x2), and a 128 x 16 tile of ones.
constexpr int kOffK = 0;
constexpr int kOffV = kOffK + kKStages * kTileBytes;
constexpr int kOffQ = kOffV + kTileBytes;
constexpr int kOffDO = kOffQ + kQStages * kTileBytes;
constexpr int kOffDS = kOffDO + kDoStages * kTileBytes;
constexpr int kOffStage = kOffDS + 2 * kTileBytes;
constexpr int kOffLseExt = kOffStage + 2 * kTileBytes;
constexpr int kOffDExt = kOffLseExt + kQStages * kExtBytes;
constexpr int kOffOnes = kOffDExt + kDoStages * kExtBytes;
constexpr int kSmemBytes = kOffOnes + kExtBytes;
static_assert(kSmemBytes <= 227 * 1024 - 1024, "dynamic shared memory plus the static barriers must fit in 227 KB");

struct Barriers {
    uint64_t item_full[kItemRing];
    uint64_t k_full[kKStages], k_empty[kKStages], v_full, v_empty;
    uint64_t q_full[kQStages], q_empty[kQStages], do_full[kDoStages], do_empty[kDoStages];
    uint64_t s_full, s_free, dp_full, dp_free, p_ready, p_free;
    uint64_t ds_ready, dq_full, dq_empty, acc_free, dv_done;
};

// Position in the CTA's stream of steps. All roles walk the same stream; `n` counts work items and `g`
// steps since the CTA started (they index the rings and give the barrier parities).
struct Cursor {
    int n, g;
    int bh, jt, n_it, it, hh, bb;
    bool valid;
    __device__ __forceinline__ bool first() const { return it == 0; }
    __device__ __forceinline__ bool last() const { return it == n_it - 1; }
    __device__ __forceinline__ int q_tile() const { return jt + it; }
};
// (slab, key tile, head, batch) of work item w: ascending item index = descending length (tile-major) or slab by slab.
// Out of line: the integer divisions are needed once per item and role, and inlined at every use they were a
// fifth of the kernel's code.
static __device__ __noinline__ int4 decode_item(int w, int BH, int H, int n_tiles, int tile_major) {
    const int bh = tile_major ? (w % BH) : (w / n_tiles);
    const int jt = tile_major ? (w / BH) : (w % n_tiles);
    return make_int4(bh, jt, bh % H, bh / H);
}

// Shared-memory descriptor of a K-major operand of exactly 16 BF16 per row (32-byte rows, 32-byte swizzle,
// 8-row groups 256 bytes apart): the statistics tiles and the tile of ones.
__device__ __forceinline__ uint64_t make_smem_desc_sw32(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
    d |= uint64_t(1) << 16;           // leading byte offset: unused for a swizzled K-major operand
    d |= uint64_t(256 >> 4) << 32;    // stride between groups of 8 rows
    d |= uint64_t(1) << 46;           // descriptor version for sm_100
    d |= uint64_t(6) << 61;           // SWIZZLE_32B
    return d;
}

template <bool GRADS_F32>
__global__ void __launch_bounds__(kThreads, 1) attn_bwd_tc64_kernel(const __grid_constant__ TcBwdArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem + kOffK;
    uint8_t* sV = smem + kOffV;
    uint8_t* sQ = smem + kOffQ;
    uint8_t* sDO = smem + kOffDO;
    uint8_t* sDS = smem + kOffDS;
    uint8_t* sStage = smem + kOffStage;
    uint8_t* sLseExt = smem + kOffLseExt;
    uint8_t* sDExt = smem + kOffDExt;
    uint8_t* sOnes = smem + kOffOnes;

    __shared__ Barriers bars;
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t abort_flag;
    __shared__ int s_item[kItemRing];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    pdl_launch_dependents();

    if (tid == 0) {
        for (int i = 0; i < kItemRing; ++i) mbar_init(&bars.item_full[i], 1);
        for (int s = 0; s < kKStages; ++s) {
            mbar_init(&bars.k_full[s], 1);
            mbar_init(&bars.k_empty[s], 1);
        }
        mbar_init(&bars.v_full, 1);
        mbar_init(&bars.v_empty, 1);
        for (int s = 0; s < kQStages; ++s) {
            mbar_init(&bars.q_full[s], 1);
            mbar_init(&bars.q_empty[s], 1);
        }
        for (int s = 0; s < kDoStages; ++s) {
            mbar_init(&bars.do_full[s], 1);
            mbar_init(&bars.do_empty[s], 1);
        }
        mbar_init(&bars.s_full, 1);
        mbar_init(&bars.s_free, kGroupThreads);
        mbar_init(&bars.dp_full, 1);
        mbar_init(&bars.dp_free, kGroupThreads);
        mbar_init(&bars.p_ready, kGroupThreads);
        mbar_init(&bars.p_free, kGroupThreads + 1);  // group B has read P^T and the dV MMAs have retired
        mbar_init(&bars.ds_ready, kGroupThreads);
        mbar_init(&bars.dq_full, 1);
        mbar_init(&bars.dq_empty, kGroupThreads);
        mbar_init(&bars.acc_free, kGroupThreads);
        mbar_init(&bars.dv_done, 1);
        abort_flag = 0;
        if ((smem_u32(smem) & 1023u) != 0 && a.fault_word) atomicCAS(a.fault_word, 0u, kFaultWaitTimeout | 0xA12u);
        mbar_fence_init();
    }
    // the tile of ones (A operand of the statistics K-step): every element 1.0, so its swizzle is immaterial
    if (tid < kExtBytes / 16) {
        *reinterpret_cast<uint4*>(sOnes + tid * 16) = make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
        fence_proxy_async_smem();
    }
    if (warp == kProducerWarp) {
        tmem_alloc(&tmem_base_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_slot;
    // barriers and TMEM are set up: from here on global memory is touched, so wait for the kernel in front of
    // this one in the stream (returns at once for an ordinary launch)
    pdl_wait();

    const int n_tiles = (a.T + kBKV - 1) / kBKV;
    const int total_items = n_tiles * a.BH;
    // Waits: one try, then the shared out-of-line polling loop. The roles that spend most of their time waiting
    // (producer, MMA issuers, group B) sleep between polls; group A, whose waits are short, does not.
    const uint32_t sleep_ns = (warp < 4) ? 0u : 32u;
    auto wait = [&](uint64_t* bar, uint32_t parity, uint32_t id) {
        mbar_wait_compact(bar, parity, &abort_flag, a.fault_word, id, sleep_ns);
    };
    auto fill = [&](Cursor& c, int w) {
        c.valid = w >= 0;
        if (c.valid) {
            const int4 f = decode_item(w, a.BH, a.H, n_tiles, a.tile_major_order);
            c.bh = f.x, c.jt = f.y, c.hh = f.z, c.bb = f.w;
            c.n_it = n_tiles - c.jt;  // query tiles jt .. n_tiles-1; tiles before the diagonal are skipped
        }
        c.it = 0;
    };
    // Moves a consumer role to the next step of the stream (the first call gives step 0). At an item boundary it
    // waits until the producer has published the next item. Whether the stream goes on must be decided
    // identically by all threads that later meet in a named barrier (a compute group) or in a warp-wide
    // instruction (an MMA warp), also when a wait has given up and the abort flag is being set concurrently: the
    // flag is therefore combined over the group (bar.red.or) or the warp (vote) before it is used, and an aborted
    // role leaves its loop at the next item boundary.
    auto next_step = [&](Cursor& c) -> bool {
        ++c.g;
        if (c.n < 0 || ++c.it == c.n_it) {
            ++c.n;
            wait(&bars.item_full[c.n % kItemRing], (c.n / kItemRing) & 1, 0x70);
            const int w = *reinterpret_cast<volatile int*>(&s_item[c.n % kItemRing]);
            const uint32_t mine = *reinterpret_cast<volatile uint32_t*>(&abort_flag);
            bool aborted;
            if (warp < 4) aborted = named_bar_or(4, kGroupThreads, mine != 0);
            else if (warp < 8) aborted = named_bar_or(5, kGroupThreads, mine != 0);
            else aborted = __any_sync(0xffffffffu, mine != 0) != 0;
            fill(c, aborted ? -1 : w);
        }
        return c.valid;
    };
    Cursor cur;
    cur.n = -1, cur.g = -1, cur.it = 0, cur.n_it = 0, cur.valid = false;

    constexpr uint32_t idesc_st = make_idesc_bf16(kBKV, kBQ, 0, 0);  // S^T, dP^T
    constexpr uint32_t idesc_kv = make_idesc_bf16(kBKV, kD, 0, 1);   // dV, dK: B is MN-major
    constexpr uint32_t idesc_dq = make_idesc_bf16(kBQ, kD, 1, 1);    // dQ: A and B MN-major

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ TMA producer (one thread)
        if (lane == 0) {
            tma_prefetch_desc(&a.map_q);
            tma_prefetch_desc(&a.map_k);
            tma_prefetch_desc(&a.map_v);
            tma_prefetch_desc(&a.map_do);
            tma_prefetch_desc(&a.map_lse_ext);
            tma_prefetch_desc(&a.map_d_ext);
            int published = 0;
            auto publish_next = [&]() {
                int w = int(atomicAdd(a.work_counter, 1u));
                if (w >= total_items) w = -1;
                s_item[published % kItemRing] = w;
                mbar_arrive(&bars.item_full[published % kItemRing]);  // release: the slot is written before the arrival
                ++published;
                return w;
            };
            cur.n = 0, cur.g = 0;
            fill(cur, publish_next());
            int w_next = -1;
            while (cur.valid) {
                const int g = cur.g, n = cur.n;
                if (cur.first()) {
                    w_next = publish_next();  // the other roles look one item ahead
                    const int ks = n % kKStages;
                    if (n >= kKStages) wait(&bars.k_empty[ks], (n / kKStages - 1) & 1, 0x42);
                    mbar_expect_tx(&bars.k_full[ks], kTileBytes);
                    tma_load_4d(sK + ks * kTileBytes, &a.map_k, &bars.k_full[ks], 0, cur.jt * kBKV, cur.hh, cur.bb);
                }
                const int qs = g % kQStages;
                if (g >= kQStages) wait(&bars.q_empty[qs], (g / kQStages - 1) & 1, 0x40);
                mbar_expect_tx(&bars.q_full[qs], kTileBytes + kExtBytes);
                tma_load_4d(sQ + qs * kTileBytes, &a.map_q, &bars.q_full[qs], 0, cur.q_tile() * kBQ, cur.hh, cur.bb);
                tma_load_4d(sLseExt + qs * kExtBytes, &a.map_lse_ext, &bars.q_full[qs], 0, cur.q_tile() * kBQ, cur.hh, cur.bb);
                if (cur.first()) {
                    // V has one buffer: it is free once dP^T of the previous item's last step has retired,
                    // about one step before dP^T of this item's first step is issued
                    if (n >= 1) wait(&bars.v_empty, (n - 1) & 1, 0x43);
                    mbar_expect_tx(&bars.v_full, kTileBytes);
                    tma_load_4d(sV, &a.map_v, &bars.v_full, 0, cur.jt * kBKV, cur.hh, cur.bb);
                }
                const int os = g % kDoStages;
                if (g >= kDoStages) wait(&bars.do_empty[os], (g / kDoStages - 1) & 1, 0x41);
                mbar_expect_tx(&bars.do_full[os], kTileBytes + kExtBytes);
                tma_load_4d(sDO + os * kTileBytes, &a.map_do, &bars.do_full[os], 0, cur.q_tile() * kBQ, cur.hh, cur.bb);
                tma_load_4d(sDExt + os * kExtBytes, &a.map_d_ext, &bars.do_full[os], 0, cur.q_tile() * kBQ, cur.hh, cur.bb);
                // next step of the stream (the producer decodes its own published ids, no ring wait)
                ++cur.g;
                if (++cur.it == cur.n_it) {
                    ++cur.n;
                    fill(cur, abort_flag ? -1 : w_next);
                }
            }
        }
        __syncwarp();
    } else if (warp == kMmaWarpS) {
        // ------------------------------------------------------------ MMA issuer 1: S^T = K Q^T - 1 (lse/scale)^T
        const uint64_t ones = make_smem_desc_sw32(smem_u32(sOnes));
        while (next_step(cur)) {
            const int g = cur.g, ks = cur.n % kKStages, qs = g % kQStages;
            // group A holds the previous step's scores in registers
            if (g > 0) wait(&bars.s_free, (g - 1) & 1, 0x59);
            if (cur.first()) wait(&bars.k_full[ks], (cur.n / kKStages) & 1, 0x53);
            wait(&bars.q_full[qs], (g / kQStages) & 1, 0x50);
            tc_fence_after();
            if (lane == 0) T64(2, g, 0);
            if (elect_one()) {
                const uint64_t k_kmaj = make_smem_desc_sw128(smem_u32(sK + ks * kTileBytes), 0, 1024);
                const uint64_t q_kmaj = make_smem_desc_sw128(smem_u32(sQ + qs * kTileBytes), 0, 1024);
#pragma unroll 1
                for (int kk = 0; kk < kD / 16; ++kk)
                    tc_mma_ss(tmem + kColS, desc_advance(k_kmaj, kk * 32), desc_advance(q_kmaj, kk * 32), idesc_st, kk > 0);
                tc_mma_ss(tmem + kColS, ones, make_smem_desc_sw32(smem_u32(sLseExt + qs * kExtBytes)), idesc_st, 1);
                tc_commit(&bars.s_full);
            }
            __syncwarp();
            if (lane == 0) T64(2, g, 1);
        }
    } else if (warp == kMmaWarpV) {
        // ------------------------------------------------------------ MMA issuer 2: dP^T = V dO^T - 1 D^T ; dV += P^T dO
        const uint64_t ones = make_smem_desc_sw32(smem_u32(sOnes));
        const uint64_t v_kmaj = make_smem_desc_sw128(smem_u32(sV), 0, 1024);
        while (next_step(cur)) {
            const int g = cur.g, n = cur.n, os = g % kDoStages;
            // group B holds the previous step's dP^T in registers
            if (g > 0) wait(&bars.dp_free, (g - 1) & 1, 0x5A);
            if (cur.first()) wait(&bars.v_full, n & 1, 0x54);
            wait(&bars.do_full[os], (g / kDoStages) & 1, 0x51);
            tc_fence_after();
            if (lane == 0) T64(3, g, 0);
            if (elect_one()) {
                const uint64_t do_kmaj = make_smem_desc_sw128(smem_u32(sDO + os * kTileBytes), 0, 1024);
#pragma unroll 1
                for (int kk = 0; kk < kD / 16; ++kk)
                    tc_mma_ss(tmem + kColDP, desc_advance(v_kmaj, kk * 32), desc_advance(do_kmaj, kk * 32), idesc_st, kk > 0);
                tc_mma_ss(tmem + kColDP, ones, make_smem_desc_sw32(smem_u32(sDExt + os * kExtBytes)), idesc_st, 1);
                tc_commit(&bars.dp_full);
                if (cur.last()) tc_commit(&bars.v_empty);  // the last reader of this item's V
            }
            __syncwarp();
            if (lane == 0) T64(3, g, 1);
            wait(&bars.p_ready, g & 1, 0x55);
            if (cur.first() && n > 0) wait(&bars.acc_free, (n - 1) & 1, 0x58);  // the previous item's dV has been read out of TMEM
            tc_fence_after();
            if (lane == 0) T64(3, g, 2);
            if (elect_one()) {
                const uint64_t do_mnmaj = make_smem_desc_sw128(smem_u32(sDO + os * kTileBytes), kTileBytes, 1024);
                const uint32_t acc0 = cur.first() ? 0u : 1u;
#pragma unroll 1
                for (int kk = 0; kk < kBQ / 16; ++kk)
                    tc_mma_ts(tmem + kColDV, tmem + kColP + kk * 8, desc_advance(do_mnmaj, kk * 2048), idesc_kv, acc0 | uint32_t(kk > 0));
                tc_commit(&bars.do_empty[os]);  // dP^T and dV of this step were the readers of this dO tile
                tc_commit(&bars.p_free);        // P^T has been consumed by the tensor pipe
                if (cur.last()) tc_commit(&bars.dv_done);
            }
            __syncwarp();
            if (lane == 0) T64(3, g, 3);
        }
    } else if (warp == kMmaWarpK) {
        // ------------------------------------------------------------ MMA issuer 3: dK += dS^T Q ; dQ = dS K
        const uint64_t ds_kmaj = make_smem_desc_sw128(smem_u32(sDS), 0, 1024);
        const uint64_t ds_mnmaj = make_smem_desc_sw128(smem_u32(sDS), kTileBytes, 1024);
        while (next_step(cur)) {
            const int g = cur.g, n = cur.n, ks = n % kKStages, qs = g % kQStages;
            wait(&bars.ds_ready, g & 1, 0x56);
            if (cur.first() && n > 0) wait(&bars.acc_free, (n - 1) & 1, 0x5B);  // the previous item's dK has been read out of TMEM
            tc_fence_after();
            if (lane == 0) T64(4, g, 0);
            if (elect_one()) {
                const uint64_t q_mnmaj = make_smem_desc_sw128(smem_u32(sQ + qs * kTileBytes), kTileBytes, 1024);
                const uint32_t acc0 = cur.first() ? 0u : 1u;
#pragma unroll 1
                for (int kk = 0; kk < kBQ / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kTileBytes + (kk & 3) * 32;
                    tc_mma_ss(tmem + kColDK, desc_advance(ds_kmaj, off), desc_advance(q_mnmaj, kk * 2048), idesc_kv, acc0 | uint32_t(kk > 0));
                }
                tc_commit(&bars.q_empty[qs]);  // S^T (retired long ago) and dK of this step were the readers of this Q tile
            }
            __syncwarp();
            if (lane == 0) T64(4, g, 1);
            if (g > 0) {  // the previous dQ partial must have been read out of its columns
                wait(&bars.dq_empty, (g - 1) & 1, 0x57);
                tc_fence_after();
            }
            if (lane == 0) T64(4, g, 2);
            if (elect_one()) {
                const uint64_t k_mnmaj = make_smem_desc_sw128(smem_u32(sK + ks * kTileBytes), kTileBytes, 1024);
#pragma unroll 1
                for (int kk = 0; kk < kBKV / 16; ++kk)
                    tc_mma_ss(tmem + kColDQ, desc_advance(ds_mnmaj, kk * 2048), desc_advance(k_mnmaj, kk * 2048), idesc_dq, kk > 0);
                tc_commit(&bars.dq_full);
                if (cur.last()) tc_commit(&bars.k_empty[ks]);  // the item's last reader of K (its S^T MMAs retired before)
            }
            __syncwarp();
            if (lane == 0) T64(4, g, 3);
        }
    } else if (warp < 4) {
        // ------------------------------------------------------------ group A: P^T = exp2((S^T - lse/scale) * scale*log2e)
        const int r = tid;  // key row of the tile = TMEM lane
        const uint32_t lane_base = uint32_t(warp) * 32u;
        const float scale_log2 = a.scale * kLog2e;
        while (next_step(cur)) {
            const int g = cur.g;
            const bool diag = cur.first();  // the diagonal tile of this item: query column c is masked for key row r when c < r
            if (r == 0) T64(0, g, 0);
            wait(&bars.s_full, g & 1, 0x61);
            tc_fence_after();
            if (r == 0) T64(0, g, 1);
            // The row is handled in four chunks of 32 queries inside ROLLED loops (the TMEM load of the next chunk in
            // flight under the exponentials of this one): unrolled over the whole row the pass is some 7 KB of
            // straight-line code that every step fetches once per warp, and with one warp of each role per scheduler
            // that fetch, not the arithmetic, set the pace.
            uint32_t buf0[32], buf1[32];
            tmem_ld32(tmem_addr(tmem, lane_base, kColS), buf0);
            tmem_wait_ld();
            if (r == 0) T64(0, g, 2);
            if (!diag) {
                // chunk of the row: 32 scores -> 16 packed BF16 pairs of P^T
                auto exp_chunk = [&](const uint32_t* sv, uint32_t* pk) {
#pragma unroll
                    for (int x = 0; x < 32; x += 2) {
                        const float2 t = mul2(__uint_as_float(sv[x]), __uint_as_float(sv[x + 1]), scale_log2, scale_log2);
                        pk[x >> 1] = pack_bf16x2(fast_exp2(t.x), fast_exp2(t.y));
                    }
                };
#pragma unroll 1
                for (int c = 0; c < 4; c += 2) {
                    uint32_t pk0[16], pk1[16];
                    tmem_ld32(tmem_addr(tmem, lane_base, kColS + (c + 1) * 32), buf1);
                    exp_chunk(buf0, pk0);
                    tmem_wait_ld();
                    if (c == 0) {
                        tmem_ld32(tmem_addr(tmem, lane_base, kColS + 64), buf0);
                    } else {
                        // the whole score row has left TMEM: S^T of the next step may be produced
                        tc_fence_before();
                        mbar_arrive(&bars.s_free);
                    }
                    exp_chunk(buf1, pk1);
                    if (c == 0 && g > 0) {
                        // half of the exponentials are done before P^T of the previous step has to be gone from TMEM
                        // (its dV MMAs retired, group B has read it)
                        wait(&bars.p_free, (g - 1) & 1, 0x63);
                        tc_fence_after();
                    }
                    tmem_st16(tmem_addr(tmem, lane_base, kColP + c * 16), pk0);
                    tmem_st16(tmem_addr(tmem, lane_base, kColP + (c + 1) * 16), pk1);
                    if (c == 0) tmem_wait_ld();
                }
            } else {
                // diagonal tile (the first step of every item): warp w (key rows 32w .. 32w+31) sees chunk c < w fully
                // masked, chunk c > w unmasked, and masks query x of chunk w when x < lane
                if (g > 0) {
                    wait(&bars.p_free, (g - 1) & 1, 0x67);
                    tc_fence_after();
                }
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    if (c > 0) {
                        tmem_ld32(tmem_addr(tmem, lane_base, kColS + c * 32), buf0);
                        tmem_wait_ld();
                    }
                    if (c == 3) {
                        tc_fence_before();
                        mbar_arrive(&bars.s_free);
                    }
                    uint32_t pk[16];
                    const int visible_from = (c < warp) ? 32 : ((c == warp) ? lane : 0);  // first unmasked query of the chunk
#pragma unroll
                    for (int x = 0; x < 32; x += 2) {
                        float e0 = fast_exp2(__uint_as_float(buf0[x]) * scale_log2);
                        float e1 = fast_exp2(__uint_as_float(buf0[x + 1]) * scale_log2);
                        if (x < visible_from) e0 = 0.f;
                        if (x + 1 < visible_from) e1 = 0.f;
                        pk[x >> 1] = pack_bf16x2(e0, e1);
                    }
                    tmem_st16(tmem_addr(tmem, lane_base, kColP + c * 16), pk);
                }
            }
            if (r == 0) T64(0, g, 3);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars.p_ready);
            if (r == 0) T64(0, g, 5);
        }
    } else {
        // ------------------------------------------------------------ group B: dS^T, dQ partials, dK / dV of finished items
        const int r = tid - kGroupThreads;  // key row (dS^T, dK, dV) or query row (dQ partial) = TMEM lane
        const uint32_t lane_base = uint32_t(warp & 3) * 32u;
        const bool leader = (r == 0);
        Cursor prev;
        prev.valid = false;
        // One pass of the loop = dS^T of step `cur` (if the stream goes on), then the dQ partial of step `prev` and, when
        // that step closed an item, its dK / dV. The pass after the last step only does the second half.
        for (;;) {
            const bool more = next_step(cur);
            const int g = cur.g;
            if (more) {
                if (leader) T64(1, g, 0);
                wait(&bars.p_ready, g & 1, 0x64);
                if (leader) T64(1, g, 1);
                wait(&bars.dp_full, g & 1, 0x62);
                tc_fence_after();
                if (leader) T64(1, g, 2);
            }
            // dS^T of the whole row goes to registers first (64 packed words): the single shared-memory tile is still
            // being read by dK / dQ of the previous step
            uint32_t dsw[kBQ / 2];
            if (more) {
#pragma unroll
                for (int h = 0; h < 4; ++h) {  // 32 queries at a time
                    uint32_t pp[16], dv[32];
                    tmem_ld16(tmem_addr(tmem, lane_base, kColP + h * 16), pp);
                    tmem_ld32(tmem_addr(tmem, lane_base, kColDP + h * 32), dv);
                    tmem_wait_ld();
                    if (h == 3) {  // the whole row is in registers: dP^T and P^T columns may be overwritten
                        tc_fence_before();
                        mbar_arrive(&bars.dp_free);
                        mbar_arrive(&bars.p_free);
                    }
                    // dS^T = P^T * (dP^T - D), FP32 product of the BF16 P^T and the FP32 dP^T - D (the softmax scale is
                    // applied to dK when it is stored and to dQ when it is converted)
#pragma unroll
                    for (int x = 0; x < 16; ++x) {
                        const uint32_t w = pp[x];  // P^T of queries 2x (low half) and 2x+1 (high half)
                        const float2 t = mul2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u), __uint_as_float(dv[2 * x]),
                                              __uint_as_float(dv[2 * x + 1]));
                        dsw[h * 16 + x] = pack_bf16x2(t.x, t.y);
                    }
                }
                if (leader) T64(1, g, 3);
            }
            if (prev.valid) {  // dK / dQ of the previous step have retired: the dS^T tile may be rewritten
                wait(&bars.dq_full, prev.g & 1, 0x60);
                tc_fence_after();
            }
            if (more) {
                if (leader) T64(1, g, 4);
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int x = 0; x < 32; x += 4)
                        *reinterpret_cast<uint4*>(sDS + h * kTileBytes + swz128(r, x >> 2)) =
                            make_uint4(dsw[h * 32 + x], dsw[h * 32 + x + 1], dsw[h * 32 + x + 2], dsw[h * 32 + x + 3]);
                fence_proxy_async_smem();
                tc_fence_before();
                mbar_arrive(&bars.ds_ready);
                if (leader) T64(1, g, 8);
            }
            if (prev.valid) {
                // dQ partial of step prev: TMEM -> registers (frees the columns) -> swizzled FP32 staging tile -> TMA
                // reduce-add of whole 128-byte lines into the accumulator. The reduce runs behind the next step's work;
                // its read of the staging tile is waited for only when the tile is needed again.
                uint32_t dq[kD];
                tmem_ld32(tmem_addr(tmem, lane_base, kColDQ), &dq[0]);
                tmem_ld32(tmem_addr(tmem, lane_base, kColDQ + 32), &dq[32]);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(&bars.dq_empty);
                if (leader) T64(1, prev.g + 1, 5);
                if (leader) tma_store_wait_read();  // earlier reductions have finished reading the staging tile
                named_bar_sync(2, kGroupThreads);
                if (leader) T64(1, prev.g + 1, 6);
                if constexpr (GRADS_F32) {  // the accumulator is the caller's dq: no conversion pass will apply the scale
#pragma unroll
                    for (int x = 0; x < kD; ++x) dq[x] = __float_as_uint(__uint_as_float(dq[x]) * a.scale);
                }
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int x = 0; x < 32; x += 4)
                        *reinterpret_cast<uint4*>(sStage + h * kTileBytes + swz128(r, x >> 2)) =
                            make_uint4(dq[h * 32 + x], dq[h * 32 + x + 1], dq[h * 32 + x + 2], dq[h * 32 + x + 3]);
                fence_proxy_async_smem();
                named_bar_sync(2, kGroupThreads);
                if (leader) T64(1, prev.g + 1, 7);
                if (leader) {
                    tma_reduce_add_4d(&a.map_dq_acc, sStage, 0, prev.q_tile() * kBQ, prev.hh, prev.bb);
                    tma_reduce_add_4d(&a.map_dq_acc, sStage + kTileBytes, 32, prev.q_tile() * kBQ, prev.hh, prev.bb);
                    tma_store_commit();
                }
                if (prev.last()) {
                    // dV and dK of the finished item: TMEM -> registers (the columns go back to the MMA warps at once) ->
                    // global. A thread owns one key row: 128 bytes of BF16 (256 of FP32) per tensor, 16-byte stores.
                    wait(&bars.dv_done, prev.n & 1, 0x65);  // the dV MMAs come from another thread than the dQ ones
                    tc_fence_after();
                    const int kv_g = prev.jt * kBKV + r;
#pragma unroll 1
                    for (int which = 0; which < 2; ++which) {
                        uint32_t acc[kD];
                        tmem_ld32(tmem_addr(tmem, lane_base, (which == 0 ? kColDV : kColDK)), &acc[0]);
                        tmem_ld32(tmem_addr(tmem, lane_base, (which == 0 ? kColDV : kColDK) + 32), &acc[32]);
                        tmem_wait_ld();
                        if (which == 1) {
                            tc_fence_before();
                            mbar_arrive(&bars.acc_free);
                        }
                        const float mul = (which == 1) ? a.scale : 1.0f;  // dK: dS was left unscaled
                        if (kv_g < a.T) {
                            if constexpr (GRADS_F32) {
                                float* dst = reinterpret_cast<float*>(which == 0 ? a.dv : a.dk) + ((long long)prev.bh * a.T + kv_g) * kD;
#pragma unroll
                                for (int x = 0; x < kD; x += 4)
                                    *reinterpret_cast<float4*>(dst + x) =
                                        make_float4(__uint_as_float(acc[x]) * mul, __uint_as_float(acc[x + 1]) * mul,
                                                    __uint_as_float(acc[x + 2]) * mul, __uint_as_float(acc[x + 3]) * mul);
                            } else {
                                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(which == 0 ? a.dv : a.dk) + (long long)prev.bb * a.grad_lb +
                                                     (long long)prev.hh * a.grad_lh + (long long)kv_g * a.grad_lt;
#pragma unroll
                                for (int x = 0; x < kD; x += 8) {
                                    uint4 w;
                                    w.x = pack_bf16x2(__uint_as_float(acc[x]) * mul, __uint_as_float(acc[x + 1]) * mul);
                                    w.y = pack_bf16x2(__uint_as_float(acc[x + 2]) * mul, __uint_as_float(acc[x + 3]) * mul);
                                    w.z = pack_bf16x2(__uint_as_float(acc[x + 4]) * mul, __uint_as_float(acc[x + 5]) * mul);
                                    w.w = pack_bf16x2(__uint_as_float(acc[x + 6]) * mul, __uint_as_float(acc[x + 7]) * mul);
                                    *reinterpret_cast<uint4*>(dst + x) = w;
                                }
                            }
                        }
                    }
                }
            }
            if (leader) T64(1, g, 9);
            if (!more) break;
            prev = cur;
        }
        // shared memory must outlive the bulk reads of every reduce issued by this thread; their global writes
        // complete before the grid does
        if (leader) tma_store_wait_read();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kProducerWarp) tmem_dealloc(tmem, kTmemCols);
}

template <bool GRADS_F32>
cudaError_t launch_bwd64(const TcBwdArgs& a, cudaStream_t stream) {
    auto kern = attn_bwd_tc64_kernel<GRADS_F32>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    int dev = 0, sms = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    const long long items = (long long)((a.T + kBKV - 1) / kBKV) * a.BH;
    const long long blocks = items < sms ? items : sms;  // one persistent CTA per SM
    return launch_pdl(kern, dim3((unsigned int)blocks), dim3(kThreads), kSmemBytes, stream, a);
}

}  // namespace

cudaError_t launch_attn_bwd_tc64(const TcBwdArgs& a, cudaStream_t stream) {
    if (a.BH == 0 || a.T == 0) return cudaSuccess;
    if (a.d != 64 || a.work_counter == nullptr) return cudaErrorInvalidValue;
    return a.grads_are_f32 ? launch_bwd64<true>(a, stream) : launch_bwd64<false>(a, stream);
}

}  // namespace b200attn
