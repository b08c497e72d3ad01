// Fused softmax cross-entropy, loss and d_logits in one launch, for sm_100a. Replaces
// cross_entropy_forward_backward of sarimahsan/transformer-cuda (src/kernels/loss.cu:24-125): same arithmetic
// (row maximum, sum of exponentials, (p - onehot) / rows, row loss = log(sum) - (logit[target] - max)), different
// data movement. The operation is a pure HBM stream - 4 bytes in and 4 bytes out per logit, one exponential - and
// at the model sizes it matters for (50257 logits per row, 16384 rows: 3.3 GB each way) a row is 201 KB, which fits
// the 227 KB of shared memory of one SM. So:
//
//   * One persistent CTA per SM walks rows blockIdx.x, blockIdx.x + gridDim.x, ... A row is brought into shared
//     memory ONCE by bulk asynchronous copies (cp.async.bulk, 16 KB chunks, one mbarrier per chunk), the maximum
//     is taken as the chunks land, the exponentials replace the logits in place, and the finished d_logits leave
//     by bulk copies from the same buffer. The reference's kernel reads every row three times from global memory.
//   * The copies of consecutive rows overlap: as soon as the bulk store of chunk c has read its 16 KB, the load of
//     chunk c of the CTA's next row is issued into the same place, so loads of row r+1 and stores of row r are in
//     flight while the exponentials of row r run. No thread touches data it does not own between the passes
//     (thread t owns floats [4t, 4t+4) of every chunk), so the only CTA-wide barriers are the two reductions and
//     one per chunk in front of its bulk store.
//   * Rows start at multiples of V floats, i.e. at any 4-byte phase, while bulk copies need 16-byte aligned
//     addresses and sizes: a row is split into a head of 0-3 floats, a 16-byte aligned interior that travels by
//     bulk copy, and a tail of 0-3 floats; head and tail live in registers of the threads that load and store them.
//   * The row losses go to a scratch array and the LAST CTA to finish (atomic ticket) adds them in a fixed order,
//     in double precision, and writes the mean: the result does not depend on the order CTAs ran in, and the host
//     reads 4 bytes instead of B * T floats (src/kernels/loss.cu:116-124 copies them all and sums on the host).
//
// Rows that do not fit shared memory (V > 57344), V < 8 or buffers that are not 16-byte aligned take a streaming
// kernel: one CTA per row, an online (max, sum) pass and a second pass that writes d_logits - two reads instead of
// the reference's three. Every mbarrier wait is bounded (tc_common.cuh); no cluster-wide copy is used.
#include "kernels/loss.cuh"

#include <cfloat>
#include <cstdio>
#include <mutex>
#include <string>

#include "b200loss.h"
#include "tc_common.cuh"

// Defined by the GEMM drop-in (libb200gemm.a) when it is linked into the same program and B200GEMM_TWINS=1, else NULL: a
// BF16 twin of d_logits (rows of round_up(V, 8) elements), written here beside the FP32 values so that the two head
// GEMMs of the backward pass, which read d_logits next, convert nothing.
extern "C" void* b200gemm_bf16_twin(const void* fp32, int rows, int cols) __attribute__((weak));

namespace {

using namespace b200attn;

constexpr int kThreads = 1024;
constexpr int kChunk = 4 * kThreads;  // floats per bulk copy: one float4 per thread
constexpr int kMaxChunks = 14;
constexpr int kLag = 2;               // bulk stores allowed to be still reading when the next load is issued
constexpr int kMaxResidentV = kMaxChunks * kChunk;
constexpr float kLog2e = 1.4426950408889634f;
constexpr unsigned kWaitIdLoad = 0x4c00u;

// Split of row `row` into head (registers), 16-byte aligned interior (shared memory) and tail (registers).
struct RowGeom {
    long long start;  // index of the row's first float
    int head, inter, tail, chunks;
};
__device__ __forceinline__ RowGeom row_geom(int row, int V) {
    RowGeom g;
    g.start = (long long)row * V;
    g.head = (4 - (int)(g.start & 3)) & 3;
    g.inter = (V - g.head) & ~3;
    g.tail = V - g.head - g.inter;
    g.chunks = (g.inter + kChunk - 1) / kChunk;
    return g;
}
__device__ __forceinline__ int chunk_floats(const RowGeom& g, int c) { return min(kChunk, g.inter - c * kChunk); }

__device__ __forceinline__ void bulk_load(float* smem_dst, const float* gsrc, uint32_t bytes, uint64_t* bar) {
    mbar_expect_tx(bar, bytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_store(float* gdst, const float* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Adds the row losses in a fixed order (thread t takes rows t, t + blockDim, ...; then a shuffle tree and a serial sum
// over warps) and writes their mean. Called by every thread of the last CTA to finish.
__device__ void finish_mean_loss(const float* row_loss, int rows, float* loss_out, double* red) {
    double acc = 0.0;
    for (int i = threadIdx.x; i < rows; i += blockDim.x) acc += (double)__ldcg(row_loss + i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double total = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += red[w];
        *loss_out = (float)(total / (double)rows);
    }
}

// words[0] = ticket of finished CTAs, words[1] = record of a wait that ran out
__global__ void __launch_bounds__(kThreads, 1)
    cross_entropy_resident_kernel(const float* __restrict__ logits, const int* __restrict__ targets, float* dlogits,
                                  float* row_loss, float* loss_out, unsigned int* words, int rows, int V, float scale,
                                  __nv_bfloat16* __restrict__ twin, int twin_ld) {
    extern __shared__ __align__(128) float buf[];  // the interior of the current row
    __shared__ uint64_t load_bar[kMaxChunks];
    __shared__ float red_max[32], red_sum[32];
    __shared__ double red_loss[32];
    __shared__ float target_logit;
    __shared__ uint32_t abort_flag, is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int c = 0; c < kMaxChunks; ++c) mbar_init(&load_bar[c], 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    int row = blockIdx.x;
    if (tid == 0 && row < rows) {
        const RowGeom g = row_geom(row, V);
        for (int c = 0; c < g.chunks; ++c)
            bulk_load(buf + c * kChunk, logits + g.start + g.head + (long long)c * kChunk, chunk_floats(g, c) * 4, &load_bar[c]);
    }
    uint32_t phases = 0;  // bit c: parity the next wait on load_bar[c] uses

    for (; row < rows; row += gridDim.x) {
        const RowGeom g = row_geom(row, V);
        const float* src = logits + g.start;
        float* dst = dlogits + g.start;
        const int target = targets[row];
        // the head / tail element this thread carries in a register (threads 0-2: head, 32-34: tail), else none
        const int edge = tid < g.head ? tid : (tid >= 32 && tid < 32 + g.tail) ? g.head + g.inter + (tid - 32) : -1;
        float edge_x = edge >= 0 ? src[edge] : -FLT_MAX;
        if (tid == 0) target_logit = 0.f;

        // pass 1: maximum, chunk by chunk as the copies land
        float m = edge_x;
        for (int c = 0; c < g.chunks; ++c) {
            mbar_wait_compact(&load_bar[c], (phases >> c) & 1u, &abort_flag, words + 1, kWaitIdLoad + c, 0);
            phases ^= 1u << c;
            if (tid * 4 < chunk_floats(g, c)) {
                const float4 x = *reinterpret_cast<const float4*>(buf + c * kChunk + tid * 4);
                m = fmaxf(m, fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w)));
            }
        }
        m = warp_max(m);
        if (lane == 0) red_max[warp] = m;
        __syncthreads();
        m = warp_max(red_max[lane]);
        const float m2 = m * kLog2e;

        // pass 2: exponentials in place, their sum, and the target's logit
        float sum = 0.f;
        if (edge >= 0) {
            if (edge == target) target_logit = edge_x - m;
            edge_x = fast_exp2(fmaf(edge_x, kLog2e, -m2));
            sum = edge_x;
        }
        for (int c = 0; c < g.chunks; ++c) {
            if (tid * 4 < chunk_floats(g, c)) {
                float4* p = reinterpret_cast<float4*>(buf + c * kChunk + tid * 4);
                float4 x = *p;
                const int v0 = g.head + c * kChunk + tid * 4;
                const int at = target - v0;
                if ((unsigned)at < 4u) target_logit = (at == 0 ? x.x : at == 1 ? x.y : at == 2 ? x.z : x.w) - m;
                x.x = fast_exp2(fmaf(x.x, kLog2e, -m2));
                x.y = fast_exp2(fmaf(x.y, kLog2e, -m2));
                x.z = fast_exp2(fmaf(x.z, kLog2e, -m2));
                x.w = fast_exp2(fmaf(x.w, kLog2e, -m2));
                sum += (x.x + x.y) + (x.z + x.w);
                *p = x;
            }
        }
        sum = warp_sum(sum);
        if (lane == 0) red_sum[warp] = sum;
        __syncthreads();
        sum = warp_sum(red_sum[lane]);
        if (tid == 0 && row_loss != nullptr) row_loss[row] = logf(sum) - target_logit;

        // pass 3: d_logits, chunk by chunk into the bulk stores; the next row's loads follow kLag chunks behind
        const float k = scale / (sum + 1e-12f);
        __nv_bfloat16* trow = twin ? twin + (long long)row * twin_ld : nullptr;
        if (edge >= 0) {
            const float d = fmaf(edge_x, k, edge == target ? -scale : 0.f);
            dst[edge] = d;
            if (trow) trow[edge] = __float2bfloat16_rn(d);
        }
        const int next = row + gridDim.x;
        const bool has_next = next < rows;
        const RowGeom gn = row_geom(has_next ? next : row, V);
        const float* next_src = logits + gn.start + gn.head;
        for (int c = 0; c < g.chunks; ++c) {
            if (tid * 4 < chunk_floats(g, c)) {
                float4* p = reinterpret_cast<float4*>(buf + c * kChunk + tid * 4);
                float4 x = *p;
                x.x *= k, x.y *= k, x.z *= k, x.w *= k;
                const int v0 = g.head + c * kChunk + tid * 4;
                const int at = target - v0;
                x.x -= at == 0 ? scale : 0.f, x.y -= at == 1 ? scale : 0.f;
                x.z -= at == 2 ? scale : 0.f, x.w -= at == 3 ? scale : 0.f;
                *p = x;
                if (trow) {  // v0 = head (mod 4): 4-byte aligned pairs when the head is even, else one element on each side
                    if ((v0 & 1) == 0) {
                        *reinterpret_cast<__nv_bfloat162*>(trow + v0) = __floats2bfloat162_rn(x.x, x.y);
                        *reinterpret_cast<__nv_bfloat162*>(trow + v0 + 2) = __floats2bfloat162_rn(x.z, x.w);
                    } else {
                        trow[v0] = __float2bfloat16_rn(x.x);
                        *reinterpret_cast<__nv_bfloat162*>(trow + v0 + 1) = __floats2bfloat162_rn(x.y, x.z);
                        trow[v0 + 3] = __float2bfloat16_rn(x.w);
                    }
                }
            }
            fence_proxy_async_smem();
            __syncthreads();
            if (tid == 0) {
                bulk_store(dst + g.head + (long long)c * kChunk, buf + c * kChunk, chunk_floats(g, c) * 4);
                bulk_commit();
                if (c >= kLag) {
                    bulk_wait_read<kLag>();
                    const int cn = c - kLag;
                    if (has_next && cn < gn.chunks)
                        bulk_load(buf + cn * kChunk, next_src + (long long)cn * kChunk, chunk_floats(gn, cn) * 4, &load_bar[cn]);
                }
            }
        }
        if (tid == 0) {
            bulk_wait_read<0>();
            if (has_next)
                for (int cn = max(g.chunks - kLag, 0); cn < gn.chunks; ++cn)
                    bulk_load(buf + cn * kChunk, next_src + (long long)cn * kChunk, chunk_floats(gn, cn) * 4, &load_bar[cn]);
        }
    }
    if (tid == 0) bulk_wait_all();

    if (row_loss != nullptr) {
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            is_last = atomicAdd(words, 1u) == gridDim.x - 1 ? 1u : 0u;
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            finish_mean_loss(row_loss, rows, loss_out, red_loss);
            if (tid == 0) words[0] = 0u;
        }
    }
}

// Any V, any alignment: one CTA per row, online (max, sum), then the write pass.
constexpr int kStreamThreads = 512;
__global__ void __launch_bounds__(kStreamThreads)
    cross_entropy_stream_kernel(const float* __restrict__ logits, const int* __restrict__ targets, float* dlogits,
                                float* row_loss, float* loss_out, unsigned int* words, int rows, int V, float scale,
                                __nv_bfloat16* __restrict__ twin, int twin_ld) {
    __shared__ float red_max[32], red_sum[32];
    __shared__ double red_loss[32];
    __shared__ uint32_t is_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = kStreamThreads / 32;
    const int row = blockIdx.x;
    const float* src = logits + (long long)row * V;
    float* dst = dlogits + (long long)row * V;
    const int target = targets[row];

    float m = -FLT_MAX, s = 0.f;
    for (int v = tid; v < V; v += kStreamThreads) {
        const float x = src[v];
        if (x > m) {
            s = s * fast_exp2((m - x) * kLog2e) + 1.f;
            m = x;
        } else {
            s += fast_exp2((x - m) * kLog2e);
        }
    }
    const float row_max = warp_max(m);
    if (lane == 0) red_max[warp] = row_max;
    __syncthreads();
    const float gmax = warp_max(lane < n_warps ? red_max[lane] : -FLT_MAX);
    s *= fast_exp2((m - gmax) * kLog2e);  // s = 0 where the thread saw no element
    s = warp_sum(s);
    if (lane == 0) red_sum[warp] = s;
    __syncthreads();
    const float sum = warp_sum(lane < n_warps ? red_sum[lane] : 0.f);
    if (tid == 0 && row_loss != nullptr) {
        const float t = (target >= 0 && target < V) ? src[target] - gmax : 0.f;
        row_loss[row] = logf(sum) - t;
    }
    const float k = scale / (sum + 1e-12f), m2 = gmax * kLog2e;
    __syncthreads();  // the row's logits are read for the last time above when d_logits aliases logits
    for (int v = tid; v < V; v += kStreamThreads) {
        const float d = fmaf(fast_exp2(fmaf(src[v], kLog2e, -m2)), k, v == target ? -scale : 0.f);
        dst[v] = d;
        if (twin) twin[(long long)row * twin_ld + v] = __float2bfloat16_rn(d);
    }

    if (row_loss != nullptr) {
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            is_last = atomicAdd(words, 1u) == gridDim.x - 1 ? 1u : 0u;
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            finish_mean_loss(row_loss, rows, loss_out, red_loss);
            if (tid == 0) words[0] = 0u;
        }
    }
}

// ---------------------------------------------------------------- host side
thread_local std::string g_last_error;

struct DeviceScratch {
    float* row_loss = nullptr;
    size_t rows_cap = 0;
    unsigned int* words = nullptr;  // ticket, fault record, [2] = loss when the caller keeps none
    int sm_count = 0;
    bool attr_set = false;
};
constexpr int kMaxDevices = 64;
DeviceScratch g_scratch[kMaxDevices];
std::mutex g_mutex;

int fail(int code, const std::string& what) {
    g_last_error = what;
    return code;
}
int cuda_fail(const char* what, cudaError_t e) {
    return fail(B200LOSS_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

bool resident_path(const float* logits, const float* dlogits, int V) {
    return V >= 8 && V <= kMaxResidentV && ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15u) == 0;
}

int launch(const float* logits, const int* targets, float* dlogits, float* device_loss, bool want_loss, int B, int T,
           int V, cudaStream_t stream, float** loss_location) {
    if (!logits || !targets || !dlogits) return fail(B200LOSS_ERR_ARG, "b200loss_cross_entropy: NULL logits, targets or d_logits");
    if (B <= 0 || T <= 0 || V <= 0 || (long long)B * T > 0x7fffffffLL)
        return fail(B200LOSS_ERR_ARG, "b200loss_cross_entropy: B, T and V must be positive and B * T below 2^31");
    const int rows = B * T;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail("cudaGetDevice", e);
    if (dev >= kMaxDevices) return fail(B200LOSS_ERR_ARG, "b200loss_cross_entropy: device index above 63");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceScratch& s = g_scratch[dev];
    if (!s.words) {
        if ((e = cudaMalloc(&s.words, 64)) != cudaSuccess) return cuda_fail("cudaMalloc(words)", e);
        if ((e = cudaMemset(s.words, 0, 64)) != cudaSuccess) return cuda_fail("cudaMemset(words)", e);
        if ((e = cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
            return cuda_fail("cudaDeviceGetAttribute", e);
    }
    if (want_loss && s.rows_cap < (size_t)rows) {
        if (s.row_loss) {
            if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("cudaDeviceSynchronize", e);
            cudaFree(s.row_loss);
            s.row_loss = nullptr, s.rows_cap = 0;
        }
        if ((e = cudaMalloc(&s.row_loss, (size_t)rows * sizeof(float))) != cudaSuccess) return cuda_fail("cudaMalloc(row losses)", e);
        s.rows_cap = rows;
    }
    float* loss_out = device_loss ? device_loss : reinterpret_cast<float*>(s.words + 2);
    if (loss_location) *loss_location = loss_out;
    float* row_loss = want_loss ? s.row_loss : nullptr;
    const float scale = 1.0f / (float)rows;
    __nv_bfloat16* twin = b200gemm_bf16_twin ? static_cast<__nv_bfloat16*>(b200gemm_bf16_twin(dlogits, rows, V)) : nullptr;
    const int twin_ld = (V + 7) / 8 * 8;
    if (resident_path(logits, dlogits, V)) {
        if (!s.attr_set) {
            e = cudaFuncSetAttribute(cross_entropy_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxResidentV * 4);
            if (e != cudaSuccess) return cuda_fail("cudaFuncSetAttribute", e);
            s.attr_set = true;
        }
        const int smem = ((V + 3) & ~3) * 4;
        const int grid = rows < s.sm_count ? rows : s.sm_count;
        cross_entropy_resident_kernel<<<grid, kThreads, smem, stream>>>(logits, targets, dlogits, row_loss, loss_out, s.words,
                                                                        rows, V, scale, twin, twin_ld);
    } else {
        cross_entropy_stream_kernel<<<rows, kStreamThreads, 0, stream>>>(logits, targets, dlogits, row_loss, loss_out, s.words,
                                                                         rows, V, scale, twin, twin_ld);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail("kernel launch", e);
    return B200LOSS_OK;
}

}  // namespace

extern "C" {

int b200loss_cross_entropy(const float* logits, const int* targets, float* d_logits, float* device_loss, int B, int T,
                           int V, void* stream) {
    return launch(logits, targets, d_logits, device_loss, device_loss != nullptr, B, T, V, (cudaStream_t)stream, nullptr);
}

int b200loss_kernel_path(const float* logits, const float* d_logits, int V) { return resident_path(logits, d_logits, V) ? 0 : 1; }
int b200loss_max_resident_vocab(void) { return kMaxResidentV; }

int b200loss_check_device_fault(void) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail("cudaGetDevice", e);
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return cuda_fail("cudaDeviceSynchronize", e);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (dev >= kMaxDevices || !g_scratch[dev].words) return B200LOSS_OK;
    unsigned int word = 0;
    if ((e = cudaMemcpy(&word, g_scratch[dev].words + 1, 4, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail("cudaMemcpy", e);
    if (word == 0) return B200LOSS_OK;
    cudaMemset(g_scratch[dev].words, 0, 8);
    char msg[96];
    snprintf(msg, sizeof msg, "a bounded wait ran out inside the cross-entropy kernel (record 0x%08x)", word);
    return fail(B200LOSS_ERR_WAIT, msg);
}

void b200loss_release(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev >= kMaxDevices) return;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceScratch& s = g_scratch[dev];
    cudaDeviceSynchronize();
    if (s.row_loss) cudaFree(s.row_loss);
    if (s.words) cudaFree(s.words);
    s = DeviceScratch{};
}

const char* b200loss_last_error(void) { return g_last_error.c_str(); }

}  // extern "C"

void cross_entropy_forward_backward_device(const float* logits, const int* targets, float* dlogits, float* device_loss, int B,
                                           int T, int V, cudaStream_t stream) {
    if (launch(logits, targets, dlogits, device_loss, device_loss != nullptr, B, T, V, stream, nullptr) != B200LOSS_OK)
        fprintf(stderr, "[b200loss] %s\n", g_last_error.c_str());
}

void cross_entropy_forward_backward(const float* logits, const int* targets, float* dlogits, float* host_loss, int B, int T,
                                    int V, cudaStream_t stream) {
    float* where = nullptr;
    if (launch(logits, targets, dlogits, nullptr, host_loss != nullptr, B, T, V, stream, &where) != B200LOSS_OK) {
        fprintf(stderr, "[b200loss] %s\n", g_last_error.c_str());
        return;
    }
    if (host_loss != nullptr) {
        cudaError_t e = cudaMemcpyAsync(host_loss, where, sizeof(float), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) fprintf(stderr, "[b200loss] reading the loss back: %s\n", cudaGetErrorString(e));
    }
}
