// Device-side building blocks for the sm_100a tensor-core attention kernels:
// mbarrier waits with an iteration limit, TMA (cp.async.bulk.tensor) loads and
// stores without multicast, tcgen05 TMEM allocation / MMA / load / store, and the
// 64-bit shared-memory and 32-bit instruction descriptors the MMA consumes.
//
// Everything here is inline PTX for sm_100a; nothing falls back to another path.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>

namespace b200attn {

// ----------------------------------------------------------------------------
// Error word written by kernels whose bounded waits ran out. Host code reads it
// after synchronisation; 0 means every wait completed.
// ----------------------------------------------------------------------------
enum DeviceFault : unsigned int {
    kFaultNone = 0u,
    kFaultWaitTimeout = 0x57410000u  // low 16 bits: identifier of the wait that gave up
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Programmatic dependent launch. launch_dependents: the next kernel in the stream may start being scheduled once
// every CTA of this grid has passed this point (or exited). wait: blocks until the grids this one depends on have
// completed and their memory is visible; returns at once when the kernel was launched the ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// One lane of a converged warp. The MMA warps branch on this, not on `lane == 0`: measured on a B200,
// the same tcgen05.mma sequence (the backward's 32 MMAs per step at d = 64) issues in 1557 cycles
// behind elect.sync and in 2169 cycles behind a lane-id compare, i.e. the latter is issue-bound at
// about 62 cycles per MMA while M=128, N=64 MMAs execute in 32-48.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------- mbarrier -----------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}

// Limit on polls of one wait. try_wait itself suspends for a hardware-chosen
// interval, so this is of the order of a second before the wait gives up.
#ifndef B200ATTN_WAIT_LIMIT
#define B200ATTN_WAIT_LIMIT (1u << 22)
#endif

// Bounded wait. `abort_flag` lives in shared memory and is set by the first wait
// that gives up; once it is set every later wait returns at once, so a kernel
// that lost a signal still runs to its end (with wrong data) instead of hanging.
// The identifier of the wait is recorded in `fault_word` (global memory).
// The polling loop lives OUT OF LINE (one copy per kernel instead of one per wait): a kernel with dozens of waits
// and several warp roles otherwise carries some 20 KB of polling code, and instruction-cache misses - not arithmetic -
// then pace its single-warp roles (measured on the head-dim-64 backward: instruction-cache hit rate 67 % -> 86 %,
// "no instruction" stalls 5.1 -> 0.8 per issue, 76 -> 62 us). `sleep_ns` > 0 makes the warp sleep between polls.
static __device__ __noinline__ void mbar_wait_poll(uint32_t bar_addr, uint32_t parity, volatile uint32_t* abort_flag,
                                                   unsigned int* fault_word, uint32_t wait_id, uint32_t limit,
                                                   uint32_t sleep_ns) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (sleep_ns) __nanosleep(sleep_ns);
        uint32_t ok;
        asm volatile(
            "{\n\t"
            ".reg .pred P;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, P;\n\t"
            "}\n"
            : "=r"(ok)
            : "r"(bar_addr), "r"(parity)
            : "memory");
        if (ok) return;
        if ((it & 1023u) == 1023u && *abort_flag) return;
    }
    *abort_flag = 1u;
    if (fault_word) atomicCAS(fault_word, 0u, kFaultWaitTimeout | (wait_id & 0xffffu));
}
// Inline form (polling loop at every call site): kept for the kernels with few roles and waits, where the call into
// the shared loop measured slightly slower (head dim 128: 2.24 vs 2.16 ms per step at T = 8192).
__device__ __forceinline__ void mbar_wait_limited(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  unsigned int* fault_word, uint32_t wait_id, uint32_t limit) {
    if (mbar_try_wait(bar, parity)) return;
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return;
        if ((it & 1023u) == 1023u && *abort_flag) return;
    }
    *abort_flag = 1u;
    if (fault_word) atomicCAS(fault_word, 0u, kFaultWaitTimeout | (wait_id & 0xffffu));
}
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          unsigned int* fault_word, uint32_t wait_id) {
    mbar_wait_limited(bar, parity, abort_flag, fault_word, wait_id, B200ATTN_WAIT_LIMIT);
}
__device__ __forceinline__ void mbar_wait_compact(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  unsigned int* fault_word, uint32_t wait_id, uint32_t sleep_ns) {
    if (mbar_try_wait(bar, parity)) return;
    mbar_wait_poll(smem_u32(bar), parity, abort_flag, fault_word, wait_id, B200ATTN_WAIT_LIMIT, sleep_ns);
}

// --------------------------------- TMA --------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tiled load: coordinates (x = element in row, y = row, z = slab).
// x * sizeof(element) must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
        "[%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
// 4-D tiled load: coordinates (x = element in row, y = row, h = head, b = batch). Every operand of
// the attention kernels is described as (d, T, H, B) with arbitrary T/H/B strides, so the same
// kernels read (B, H, T, d) slabs and the interleaved (B, T, 3*H*d) projection buffer.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int h,
                                            int b) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
        "[%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(h), "r"(b)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// 3-D tiled store shared -> global (rows outside the tensor are clipped by the unit).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
// 3-D tiled reduction shared -> global: global += shared, element type taken from the tensor map
// (FP32 here). Rows outside the tensor are clipped. Never start it at a negative coordinate.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* smem_src, int x, int y, int z) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int x, int y, int h, int b) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(h), "r"(b)
                 : "memory");
}
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* smem_src, int x, int y, int h, int b) {
    asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(h), "r"(b)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// ------------------------------- tcgen05 ------------------------------------
// TMEM allocation: executed by one whole warp; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// All MMAs issued so far by this thread arrive (once) on `bar` when they retire.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; accumulate = 0 overwrites D.
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A is M lanes x K/2 32-bit columns of packed bf16 pairs.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Instruction descriptor for kind::f16 with BF16 operands and FP32 accumulation.
// a_mn / b_mn = 1 when that operand is stored MN-major (its M or N index contiguous).
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn, int b_mn) {
    return (1u << 4)                      // D format: F32
           | (1u << 7)                    // A format: BF16
           | (1u << 10)                   // B format: BF16
           | (uint32_t(a_mn & 1) << 15)   // A major
           | (uint32_t(b_mn & 1) << 16)   // B major
           | (uint32_t(N >> 3) << 17)     // N / 8
           | (uint32_t(M >> 4) << 24);    // M / 16
}

// Shared-memory operand descriptor, 128-byte swizzle. The operand tile is a stack of
// 128-byte rows (64 bf16), 1024-byte aligned, written by TMA with SWIZZLE_128B or by
// threads through swz128(). `sbo` is the byte distance between groups of 8 rows;
// `lbo` is the byte distance between 64-element atoms along the contiguous (MN)
// direction of an MN-major operand (unused for K-major).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
    d |= uint64_t((lbo >> 4) & 0x3FFFu) << 16;
    d |= uint64_t((sbo >> 4) & 0x3FFFu) << 32;
    d |= uint64_t(1) << 46;  // descriptor version for sm_100
    d |= uint64_t(2) << 61;  // SWIZZLE_128B
    return d;
}
// Advance the start-address field of a descriptor by `bytes` (multiple of 16).
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) {
    return desc + uint64_t(bytes >> 4);
}

// Byte offset of 16-byte chunk `chunk` (0..7) of 128-byte row `row` inside a
// SWIZZLE_128B tile whose base is 1024-byte aligned.
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) {
    return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

// TMEM address = (lane << 16) | column.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
    return base + (lane << 16) + col;
}

// tcgen05.ld / st, shape 32x32b: thread t of the warp touches TMEM lane
// (32 * (warp_id % 4) + t), N consecutive 32-bit columns starting at the address.
#define B200ATTN_R8(v, o) "=r"(v[o + 0]), "=r"(v[o + 1]), "=r"(v[o + 2]), "=r"(v[o + 3]), "=r"(v[o + 4]), "=r"(v[o + 5]), "=r"(v[o + 6]), "=r"(v[o + 7])
#define B200ATTN_W8(v, o) "r"(v[o + 0]), "r"(v[o + 1]), "r"(v[o + 2]), "r"(v[o + 3]), "r"(v[o + 4]), "r"(v[o + 5]), "r"(v[o + 6]), "r"(v[o + 7])

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : B200ATTN_R8(v, 0)
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : B200ATTN_R8(v, 0), B200ATTN_R8(v, 8)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : B200ATTN_R8(v, 0), B200ATTN_R8(v, 8), B200ATTN_R8(v, 16), B200ATTN_R8(v, 24)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};"
                 :
                 : B200ATTN_W8(v, 0), "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
        :
        : B200ATTN_W8(v, 0), B200ATTN_W8(v, 8), "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
        :
        : B200ATTN_W8(v, 0), B200ATTN_W8(v, 8), B200ATTN_W8(v, 16), B200ATTN_W8(v, 24), "r"(taddr)
        : "memory");
}

// Pack two floats into one bf16x2 word: `lo` in bits [0,16), `hi` in bits [16,32).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Elementwise product of two packed bf16x2 words.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Packed FP32 pairs (sm_100: one instruction for two FMAs / adds). The softmax loops are paced by instruction issue as much
// as by the 16-per-clock exponential unit; pairing the scale-and-shift and the row-sum additions takes two of the
// seven instructions per pair of scores away.
__device__ __forceinline__ float2 fma2(float ax, float ay, float b, float c) {
    uint64_t ra, rb, rc, rd;
    float2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(ax), "f"(ay));
    asm("mov.b64 %0, {%1, %1};" : "=l"(rb) : "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(rc) : "f"(c));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 mul2(float ax, float ay, float bx, float by) {
    uint64_t ra, rb, rd;
    float2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(ax), "f"(ay));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(bx), "f"(by));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float bx, float by) {
    uint64_t ra, rb, rd;
    float2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(bx), "f"(by));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x on the FMA / integer pipes, for x <= ~100 (larger arguments do not occur: scores are taken
// relative to a running maximum): round-to-nearest split x = i + f with the 1.5*2^23 trick, a
// degree-3 minimax polynomial for 2^f on [-0.5, 0.5] (relative error 2.1e-4, far below BF16
// resolution), and i added into the exponent field. Arguments below -126 (masked scores) give 2^-126.
// Used for a fraction of the exponentials so that the 16-per-clock MUFU unit is not the only path.
__device__ __forceinline__ float poly_exp2(float x) {
    x = fmaxf(x, -126.0f);
    const float xf = __fadd_rn(x, 12582912.0f);
    const float f = __fsub_rn(x, __fsub_rn(xf, 12582912.0f));
    float p = fmaf(f, 0.05484806f, 0.24180646f);
    p = fmaf(f, p, 0.69324815f);
    p = fmaf(f, p, 0.99998868f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(xf) << 23));
}
// Fraction of exponentials sent to poly_exp2: element index e uses it when (e & 3) == 3.
// OFF by default: measured on B200 with 25 % of the exponentials on the polynomial, both kernels got
// 4-7 % SLOWER (forward T=8192 d=128 0.583 -> 0.626 ms, backward 1.474 -> 1.584 ms): the softmax /
// compute warps are bound by instruction issue, not by the MUFU unit, and the polynomial costs nine
// issue slots against two.
#ifndef B200ATTN_POLY_EXP2
#define B200ATTN_POLY_EXP2 0
#endif
__device__ __forceinline__ float mixed_exp2(float x, int e) {
#if B200ATTN_POLY_EXP2
    return ((e & 3) == 3) ? poly_exp2(x) : fast_exp2(x);
#else
    return fast_exp2(x);
#endif
}

// Named barrier over a subset of the CTA's warps (id 1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// The same barrier returning the OR of `pred` over all participating threads (identical in every one of them).
__device__ __forceinline__ bool named_bar_or(uint32_t id, uint32_t nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"(uint32_t(pred))
        : "memory");
    return r != 0;
}

// Vector reduction into global FP32 memory (16-byte aligned address).
__device__ __forceinline__ void red_add_v4(float* gaddr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(gaddr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

}  // namespace b200attn
