// GEMM wrappers of the reference model (include/kernels/matmul.cuh of sarimahsan/transformer-cuda) with a
// selectable arithmetic: FP32 SIMT as in the reference (src/kernels/matmul.cu:30,96,196) or BF16 tensor
// cores with FP32 accumulation on the same FP32 buffers. These are plain library GEMMs (cuBLAS /
// cuBLASLt); the point of this file is that the data-parallel training step around the attention engine
// is no longer dominated by FP32 SGEMMs on the CUDA cores. Row-major matrices are handed to the
// column-major libraries as their transposes: C^T (N x M) = op(B)^T op(A)^T.
//
// Built into its own static library (libb200gemm.a); libb200attn does not depend on cuBLAS.
#include "kernels/matmul.cuh"

#include <cuda_bf16.h>

#include "gemm_tc.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

enum class Math { kFp32, kBf16 };

Math math_mode() {
    static const Math mode = [] {
        const char* e = getenv("B200GEMM_MATH");
        return (e && (!strcmp(e, "bf16") || !strcmp(e, "BF16"))) ? Math::kBf16 : Math::kFp32;
    }();
    return mode;
}
cublasComputeType_t compute_type() {
    return math_mode() == Math::kBf16 ? CUBLAS_COMPUTE_32F_FAST_16BF : CUBLAS_COMPUTE_32F;
}

void report(const char* what, int status) {
    if (status != 0) fprintf(stderr, "b200gemm: %s failed with status %d\n", what, status);
}

void bind_stream(cublasHandle_t handle, cudaStream_t stream) {
    cudaStream_t cur = nullptr;
    cublasGetStream(handle, &cur);
    if (cur != stream) report("cublasSetStream", (int)cublasSetStream(handle, stream));
}

// ---------------------------------------------------------------- cuBLASLt plans, one per problem shape
struct PlanKey {
    int M, N, K, transA, transB, epilogue;
    bool operator==(const PlanKey& o) const {
        return M == o.M && N == o.N && K == o.K && transA == o.transA && transB == o.transB && epilogue == o.epilogue;
    }
};
struct PlanKeyHash {
    size_t operator()(const PlanKey& k) const {
        size_t h = 1469598103934665603ull;
        for (int v : {k.M, k.N, k.K, k.transA, k.transB, k.epilogue}) h = (h ^ size_t(unsigned(v))) * 1099511628211ull;
        return h;
    }
};
struct Plan {
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;  // of the column-major problem: a <- B, b <- A
    cublasLtMatmulAlgo_t algo;
    bool has_algo = false;
};
std::unordered_map<PlanKey, Plan, PlanKeyHash> g_plans;
std::mutex g_plans_mutex;

bool build_plan(cublasLtHandle_t lt, const PlanKey& key, cublasComputeType_t ctype, size_t workspace_size, Plan* out) {
    Plan p;
    const cublasOperation_t opA = key.transA ? CUBLAS_OP_T : CUBLAS_OP_N;
    const cublasOperation_t opB = key.transB ? CUBLAS_OP_T : CUBLAS_OP_N;
    if (cublasLtMatmulDescCreate(&p.op, ctype, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) return false;
    cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &opB, sizeof(opB));
    cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &opA, sizeof(opA));
    const cublasLtEpilogue_t epi = (cublasLtEpilogue_t)key.epilogue;
    if (epi != CUBLASLT_EPILOGUE_DEFAULT) cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_EPILOGUE, &epi, sizeof(epi));
    // row-major op(B) is K x N with leading dimension ldb; seen column-major it is the matrix below
    const int lda = key.transA ? key.M : key.K, ldb = key.transB ? key.K : key.N, ldc = key.N;
    cublasLtMatrixLayoutCreate(&p.a, CUDA_R_32F, key.transB ? key.K : key.N, key.transB ? key.N : key.K, ldb);
    cublasLtMatrixLayoutCreate(&p.b, CUDA_R_32F, key.transA ? key.M : key.K, key.transA ? key.K : key.M, lda);
    cublasLtMatrixLayoutCreate(&p.c, CUDA_R_32F, key.N, key.M, ldc);
    cublasLtMatmulPreference_t pref = nullptr;
    cublasLtMatmulPreferenceCreate(&pref);
    cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_size, sizeof(workspace_size));
    cublasLtMatmulHeuristicResult_t res = {};
    int found = 0;
    const cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(lt, p.op, p.a, p.b, p.c, p.c, pref, 1, &res, &found);
    cublasLtMatmulPreferenceDestroy(pref);
    p.has_algo = (st == CUBLAS_STATUS_SUCCESS && found > 0);
    if (p.has_algo) p.algo = res.algo;
    *out = p;
    return p.has_algo;
}

void destroy_plan(Plan& p) {
    if (p.a) cublasLtMatrixLayoutDestroy(p.a);
    if (p.b) cublasLtMatrixLayoutDestroy(p.b);
    if (p.c) cublasLtMatrixLayoutDestroy(p.c);
    if (p.op) cublasLtMatmulDescDestroy(p.op);
    p = Plan();
}

// ---------------------------------------------------------------- bias kernels
// Y[r][c] += bias[c], four columns per thread when N allows it.
template <int VEC>
__global__ void __launch_bounds__(256) add_bias_kernel(float* __restrict__ Y, const float* __restrict__ bias, long long groups,
                                                       int n_groups_per_row) {
    const long long g = blockIdx.x * 256ll + threadIdx.x;
    if (g >= groups) return;
    const int col = int(g % n_groups_per_row) * VEC;
    if constexpr (VEC == 4) {
        float4 y = reinterpret_cast<float4*>(Y)[g];
        const float4 b = __ldg(reinterpret_cast<const float4*>(bias + col));
        y.x += b.x, y.y += b.y, y.z += b.z, y.w += b.w;
        reinterpret_cast<float4*>(Y)[g] = y;
    } else {
        Y[g] += __ldg(bias + col);
    }
}

// dbias[c] += sum_r dY[r][c]. A CTA owns 32 columns and a strip of rows; each warp walks its rows with
// coalesced 128-byte reads, the eight warps meet in shared memory, one atomic per column and CTA.
__global__ void __launch_bounds__(256) bias_backward_kernel(const float* __restrict__ dY, float* __restrict__ dbias, int M,
                                                            int N, int rows_per_cta) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane;
    const int r0 = blockIdx.y * rows_per_cta;
    const int r1 = min(M, r0 + rows_per_cta);
    float s0 = 0.f, s1 = 0.f;
    if (col < N) {
        int r = r0 + warp;
        for (; r + 8 < r1; r += 16) {
            s0 += __ldg(dY + (long long)r * N + col);
            s1 += __ldg(dY + (long long)(r + 8) * N + col);
        }
        if (r < r1) s0 += __ldg(dY + (long long)r * N + col);
    }
    part[warp][lane] = s0 + s1;
    __syncthreads();
    if (warp == 0 && col < N) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += part[w][lane];
        atomicAdd(dbias + col, s);
    }
}


// ---------------------------------------------------------------- staged BF16 path for unaligned leading dimensions
// The language-model head works on V = 50257 columns: rows of head_w, logits and d_logits start on 4-byte
// boundaries only, which confines cuBLASLt to slow align-1 kernels (measured: 9.5 ms for each of the three
// 1.26 TFLOP head GEMMs, 43 % of the BF16 step). In BF16 arithmetic such a GEMM is staged instead: operands are
// converted once into BF16 scratch with leading dimensions padded to 16 bytes (padding zeroed), the product
// goes to an FP32 tile with a padded leading dimension when C itself is unaligned, and one pass copies it
// into place. Scratch is owned here, grown on demand and never shrunk.
struct Scratch {
    void* p = nullptr;
    size_t bytes = 0;
    void* get(size_t want) {
        if (want > bytes) {
            if (p) cudaFree(p);
            p = nullptr, bytes = 0;
            if (cudaMalloc(&p, want) != cudaSuccess) {
                cudaGetLastError();
                return nullptr;
            }
            bytes = want;
        }
        return p;
    }
};
Scratch g_scratch;
cublasLtHandle_t g_own_lt = nullptr;
std::unordered_map<PlanKey, Plan, PlanKeyHash> g_staged_plans;
constexpr size_t kStagedWorkspace = size_t(64) << 20;

inline int round_up_int(int x, int m) { return (x + m - 1) / m * m; }
inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// FP32 (rows x cols, leading dimension ld_src) -> BF16 (rows_dst x ld_dst), everything outside rows x cols zeroed.
// blockIdx.y walks rows, a thread converts eight consecutive columns into one 16-byte store (ld_dst is a multiple of 8
// and the destination is 256-byte aligned); the source is read with two 16-byte loads when its row is aligned, else
// with scalar loads (a warp still covers one contiguous 1 KB span, so every sector fetched is used).
__global__ void __launch_bounds__(256) stage_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int rows,
                                                         int cols, long long ld_src, int rows_dst, int ld_dst) {
    const int c0 = (blockIdx.x * 256 + threadIdx.x) * 8;
    if (c0 >= ld_dst) return;
    for (int r = blockIdx.y; r < rows_dst; r += gridDim.y) {
        float v[8];
        const float* s = src + (long long)r * ld_src + c0;
        if (r < rows && c0 + 8 <= cols && (reinterpret_cast<uintptr_t>(s) & 15u) == 0) {
            const float4 lo = __ldcs(reinterpret_cast<const float4*>(s)), hi = __ldcs(reinterpret_cast<const float4*>(s) + 1);
            v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (r < rows && c0 + j < cols) ? __ldcs(s + j) : 0.f;
        }
        uint4 out;
        __nv_bfloat162 t;
        t = __floats2bfloat162_rn(v[0], v[1]), out.x = *reinterpret_cast<unsigned int*>(&t);
        t = __floats2bfloat162_rn(v[2], v[3]), out.y = *reinterpret_cast<unsigned int*>(&t);
        t = __floats2bfloat162_rn(v[4], v[5]), out.z = *reinterpret_cast<unsigned int*>(&t);
        t = __floats2bfloat162_rn(v[6], v[7]), out.w = *reinterpret_cast<unsigned int*>(&t);
        *reinterpret_cast<uint4*>(dst + (long long)r * ld_dst + c0) = out;
    }
}
void launch_stage_bf16(const float* src, __nv_bfloat16* dst, int rows, int cols, long long ld_src, int rows_dst, int ld_dst,
                       cudaStream_t stream) {
    const dim3 grid((ld_dst / 8 + 255) / 256, rows_dst < 32768 ? rows_dst : 32768);
    stage_bf16_kernel<<<grid, 256, 0, stream>>>(src, dst, rows, cols, ld_src, rows_dst, ld_dst);
}

// FP32 (rows x cols, padded leading dimension ld_src, 16-byte aligned rows) -> FP32 (rows x cols, leading dimension
// ld_dst, rows at any 4-byte phase). blockIdx.y walks rows; a thread writes one 16-byte aligned group of the
// DESTINATION row (the up to three elements in front of the first aligned group and behind the last one are written
// singly) and reads its four source elements with scalar loads: neighbouring threads read neighbouring 16 bytes, so
// the loads of a warp cover one contiguous span as well.
__global__ void __launch_bounds__(256) unpad_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int cols,
                                                        int ld_src, long long ld_dst) {
    for (int r = blockIdx.y; r < rows; r += gridDim.y) {
        const float* s = src + (long long)r * ld_src;
        float* d = dst + (long long)r * ld_dst;
        const int head = (int)((4 - ((reinterpret_cast<uintptr_t>(d) >> 2) & 3)) & 3);  // elements before the first aligned group
        const int c = head + (blockIdx.x * 256 + threadIdx.x) * 4;
        if (blockIdx.x == 0 && threadIdx.x < head && (int)threadIdx.x < cols) d[threadIdx.x] = __ldcs(s + threadIdx.x);
        if (c + 4 <= cols) {
            *reinterpret_cast<float4*>(d + c) = make_float4(__ldcs(s + c), __ldcs(s + c + 1), __ldcs(s + c + 2), __ldcs(s + c + 3));
        } else {
            for (int j = c; j < cols; ++j) d[j] = __ldcs(s + j);
        }
    }
}
void launch_unpad_f32(const float* src, float* dst, int rows, int cols, int ld_src, long long ld_dst, cudaStream_t stream) {
    const dim3 grid((cols / 4 + 1 + 255) / 256, rows < 32768 ? rows : 32768);
    unpad_f32_kernel<<<grid, 256, 0, stream>>>(src, dst, rows, cols, ld_src, ld_dst);
}

// In BF16 arithmetic every large product is staged (B200GEMM_STAGE=all, the default): handed FP32 operands, the library
// runs TF32 kernels at half the BF16 rate (measured on the GPT-2-small step: layer GEMMs 12.5 ms as TF32, 6.1 ms as BF16
// + 4.0 ms of conversion passes). B200GEMM_STAGE=unaligned stages only the products whose leading dimensions rule the
// library's fast kernels out.
bool stage_all() {
    static const bool v = [] {
        const char* e = getenv("B200GEMM_STAGE");
        return !(e && !strcmp(e, "unaligned"));
    }();
    return v;
}
// Which staged products go to the hand-written tcgen05 kernel (gemm_tc.cu) instead of the library:
//   B200GEMM_KERNEL=auto (default)  those it wins: results with an unaligned leading dimension, which it writes in place
//                                   where the library path needs a padded tile and a copy back (the language-model head:
//                                   forward 1.79 against 2.20 ms, weight gradient 1.50 against 1.59 ms, staging included)
//   B200GEMM_KERNEL=tcgen05         every staged product with at least 74 output tiles (256 x 256) and no epilogue
//   B200GEMM_KERNEL=library         none
// Elsewhere the library's two-CTA kernels are faster (layer shapes, K = 768 ... 3072: 510-570 TFLOP/s against 750-1100,
// staging included): this kernel's main loop keeps the tensor pipe at 92 % of its rate, but its epilogue - 256 KB of FP32
// per tile - is not overlapped with the next tile's MMAs (both accumulators are in use).
enum class TcPolicy { kAuto, kAlways, kNever };
TcPolicy tc_policy() {
    static const TcPolicy v = [] {
        const char* e = getenv("B200GEMM_KERNEL");
        if (e && !strcmp(e, "tcgen05")) return TcPolicy::kAlways;
        if (e && !strcmp(e, "library")) return TcPolicy::kNever;
        return TcPolicy::kAuto;
    }();
    return v;
}
constexpr int kMinTcTiles = 74;  // half the SMs of a B200: below that the persistent grid leaves most of the GPU idle
bool use_tc_kernel(int M, int N, int K, bool unaligned_result) {
    if (tc_policy() == TcPolicy::kNever || b200gemm::tc_gemm_tiles(M, N) < kMinTcTiles) return false;
    if (tc_policy() == TcPolicy::kAlways) return true;
    (void)K;
    return unaligned_result;
}

// Products below this many multiply-adds are never staged (B200GEMM_STAGE_MIN_MACS overrides the default 2^30, for tests
// that want the staged path on small shapes).
double stage_min_macs() {
    static const double v = [] {
        const char* e = getenv("B200GEMM_STAGE_MIN_MACS");
        return e ? atof(e) : double(1ull << 30);
    }();
    return v;
}
bool wants_staging(int M, int N, int K, bool transA, bool transB, float beta) {
    if (math_mode() != Math::kBf16 || beta != 0.0f) return false;
    const int lda = transA ? M : K, ldb = transB ? K : N, ldc = N;
    const bool aligned = lda % 4 == 0 && ldb % 4 == 0 && ldc % 4 == 0 && M % 8 == 0 && N % 8 == 0 && K % 8 == 0;
    if (aligned && !stage_all()) return false;
    return (double)M * N * K >= stage_min_macs();  // small products are not worth the extra passes
}

// B200GEMM_REUSE_STAGED=1: the BF16 copy of the B operand of a staged product is kept, and when the NEXT staged product
// reads the same matrix (same address, same shape) as its A operand the copy is used instead of converting it again. That
// is the pattern of a backward pass - dW = X^T dY followed by dX = dY W^T (src/model.cu:451-476 and every layer) - where the
// conversion of dY (3.3 GB at the language-model head) is otherwise paid twice. Off by default: the caller has to guarantee
// that a matrix is not rewritten between two consecutive GEMM calls that both read it. Only B -> A of the very next call
// is matched, so weights (always B, rewritten by the optimizer between steps) are never taken from a kept copy.
bool reuse_staged() {
    static const bool v = [] {
        const char* e = getenv("B200GEMM_REUSE_STAGED");
        return e && !strcmp(e, "1");
    }();
    return v;
}
struct KeptOperand {
    Scratch buf;
    const void* src = nullptr;
    int rows = 0, cols = 0;
    long long call = -1;  // index of the staged call that wrote it
};
KeptOperand g_kept[2];
long long g_staged_calls = 0, g_staged_reused = 0;

// BF16 twins. A kernel that is the only writer of an FP32 matrix the GEMMs read (a LayerNorm output, a gradient coming out
// of a LayerNorm or attention backward) can ask for a BF16 twin of it - b200gemm_bf16_twin(), below - and write the BF16
// values beside the FP32 ones; a staged product that reads a matrix with a twin (same address, same shape) uses the twin
// and converts nothing. Twins are allocated here on first request in the staged layout (leading dimension and row count
// rounded up to 8, padding zeroed once) and live until b200gemm_release_twins(). Off unless B200GEMM_TWINS=1: the
// arrangement is only sound while nothing else writes those FP32 matrices.
struct Twin {
    void* bf16 = nullptr;
    int rows = 0, cols = 0;   // rows = -1: a flat twin of `count` elements (its producer knows no row structure)
    long long count = 0;
};
std::unordered_map<const void*, Twin> g_twins;
// Twins of a whole buffer that holds many matrices back to back (the optimizer's flat parameter buffer): a matrix that
// starts inside the buffer at a multiple of 128 elements and has nothing to pad finds its BF16 values at the same offset.
struct RangeTwin {
    const float* base = nullptr;
    long long count = 0;
    __nv_bfloat16* bf16 = nullptr;
};
std::vector<RangeTwin> g_range_twins;
long long g_twin_hits = 0;
bool twins_enabled() {
    static const bool v = [] {
        const char* e = getenv("B200GEMM_TWINS");
        return e && !strcmp(e, "1") && math_mode() == Math::kBf16;
    }();
    return v;
}
// caller holds g_plans_mutex
void* find_twin(const void* fp32, int rows, int cols) {
    if (!twins_enabled()) return nullptr;
    auto it = g_twins.find(fp32);
    if (it == g_twins.end()) {
        if (rows % 8 || cols % 8) return nullptr;
        const float* p = static_cast<const float*>(fp32);
        for (const RangeTwin& r : g_range_twins) {
            if (p < r.base || p >= r.base + r.count) continue;
            const long long off = p - r.base;
            // 256-byte aligned BF16 operands, as the staged copies are: the library's kernels were chosen for that
            if (off % 128 || off + (long long)rows * cols > r.count) return nullptr;
            ++g_twin_hits;
            return r.bf16 + off;
        }
        return nullptr;
    }
    const Twin& t = it->second;
    // a flat twin is the staged layout of any rows x cols view with nothing to pad
    const bool match = t.rows >= 0 ? (t.rows == rows && t.cols == cols)
                                   : (t.count == (long long)rows * cols && rows % 8 == 0 && cols % 8 == 0);
    if (!match) return nullptr;
    ++g_twin_hits;
    return t.bf16;
}

// Returns false when the staged path could not run (the caller then takes the direct path).
bool staged_bf16_gemm(const float* A, const float* B, float* C, int M, int N, int K, bool transA, bool transB, float alpha,
                      cudaStream_t stream, cublasLtEpilogue_t epilogue = CUBLASLT_EPILOGUE_DEFAULT, const float* bias = nullptr) {
    std::lock_guard<std::mutex> lock(g_plans_mutex);
    if (!g_own_lt && cublasLtCreate(&g_own_lt) != CUBLAS_STATUS_SUCCESS) return false;
    // The library only picks its fast kernels when the problem dimensions themselves are multiples of 8, so
    // M, N and K are padded too (zero rows / columns; the extra part of the product is dropped by the copy back).
    const int Mp = round_up_int(M, 8), Np = round_up_int(N, 8), Kp = round_up_int(K, 8);
    // stored shapes (row-major): A is rowsA x colsA, B is rowsB x colsB
    const int rowsA = transA ? K : M, colsA = transA ? M : K;
    const int rowsB = transB ? N : K, colsB = transB ? K : N;
    const int rowsA_p = transA ? Kp : Mp, lda_p = transA ? Mp : Kp;
    const int rowsB_p = transB ? Np : Kp, ldb_p = transB ? Kp : Np;
    const bool pad_c = (Np != N) || (Mp != M);
    const int ldc_p = Np;
    const size_t bytesA = align256(size_t(rowsA_p) * lda_p * 2), bytesB = align256(size_t(rowsB_p) * ldb_p * 2);
    const size_t bytesC = pad_c ? align256(size_t(Mp) * ldc_p * 4) : 0;
    uint8_t* base = static_cast<uint8_t*>(g_scratch.get(kStagedWorkspace + bytesA + bytesB + bytesC));
    if (!base) return false;
    void* workspace = base;
    __nv_bfloat16* Ab = reinterpret_cast<__nv_bfloat16*>(base + kStagedWorkspace);
    __nv_bfloat16* Bb = reinterpret_cast<__nv_bfloat16*>(base + kStagedWorkspace + bytesA);
    float* Cp = pad_c ? reinterpret_cast<float*>(base + kStagedWorkspace + bytesA + bytesB) : C;
    bool a_ready = false, b_ready = false;
    const long long call = g_staged_calls++;
    if (void* t = find_twin(A, rowsA, colsA)) Ab = static_cast<__nv_bfloat16*>(t), a_ready = true;
    if (void* t = find_twin(B, rowsB, colsB)) Bb = static_cast<__nv_bfloat16*>(t), b_ready = true;
    if (reuse_staged()) {
        int a_slot = -1;
        for (int i = 0; i < 2 && !a_ready; ++i)
            if (g_kept[i].src == A && g_kept[i].rows == rowsA && g_kept[i].cols == colsA && g_kept[i].call == call - 1) a_slot = i;
        if (a_slot >= 0) Ab = static_cast<__nv_bfloat16*>(g_kept[a_slot].buf.p), a_ready = true, ++g_staged_reused;
        KeptOperand& keep = g_kept[a_slot >= 0 ? 1 - a_slot : int(call & 1)];
        if (!b_ready) {  // (a B with a twin needs no keeping: the next call finds the same twin for its A)
            keep.src = nullptr;
            if (void* kb = keep.buf.get(bytesB)) Bb = static_cast<__nv_bfloat16*>(kb), keep.src = B, keep.rows = rowsB, keep.cols = colsB, keep.call = call;
        }
    }

    const bool pad_any = pad_c || Kp != K;
    if (epilogue != CUBLASLT_EPILOGUE_DEFAULT && pad_any) return false;  // epilogues only on products that need no padding
    // the hand-written kernel multiplies the staged operands and writes C in place, whatever its leading dimension (no
    // padded result tile, no copy back); products with fewer output tiles than SMs stay with the library, which splits K
    if (epilogue == CUBLASLT_EPILOGUE_DEFAULT && use_tc_kernel(M, N, K, pad_c)) {
        if (!a_ready) launch_stage_bf16(A, Ab, rowsA, colsA, colsA, rowsA_p, lda_p, stream);
        if (!b_ready) launch_stage_bf16(B, Bb, rowsB, colsB, colsB, rowsB_p, ldb_p, stream);
        a_ready = b_ready = true;  // also for the library path below, should the kernel refuse
        if (b200gemm::tc_gemm_bf16(Ab, rowsA_p, lda_p, transA, Bb, rowsB_p, ldb_p, transB, C, N, M, N, Kp, alpha, stream)) return true;
    }
    const PlanKey key{M, N, K, transA ? 1 : 0, transB ? 1 : 0, (int)epilogue};
    auto it = g_staged_plans.find(key);
    if (it == g_staged_plans.end()) {
        Plan p;
        const cublasOperation_t opA = transA ? CUBLAS_OP_T : CUBLAS_OP_N, opB = transB ? CUBLAS_OP_T : CUBLAS_OP_N;
        bool ok = cublasLtMatmulDescCreate(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F) == CUBLAS_STATUS_SUCCESS;
        if (ok) {
            cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &opB, sizeof(opB));
            cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &opA, sizeof(opA));
            if (epilogue != CUBLASLT_EPILOGUE_DEFAULT) {
                cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_EPILOGUE, &epilogue, sizeof(epilogue));
                cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias));
            }
            cublasLtMatrixLayoutCreate(&p.a, CUDA_R_16BF, ldb_p, rowsB_p, ldb_p);  // row-major B seen column-major
            cublasLtMatrixLayoutCreate(&p.b, CUDA_R_16BF, lda_p, rowsA_p, lda_p);
            cublasLtMatrixLayoutCreate(&p.c, CUDA_R_32F, Np, Mp, ldc_p);
            cublasLtMatmulPreference_t pref = nullptr;
            cublasLtMatmulPreferenceCreate(&pref);
            cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &kStagedWorkspace, sizeof(kStagedWorkspace));
            cublasLtMatmulHeuristicResult_t res = {};
            int found = 0;
            ok = cublasLtMatmulAlgoGetHeuristic(g_own_lt, p.op, p.a, p.b, p.c, p.c, pref, 1, &res, &found) == CUBLAS_STATUS_SUCCESS && found > 0;
            cublasLtMatmulPreferenceDestroy(pref);
            if (ok) p.algo = res.algo, p.has_algo = true;
        }
        if (!ok) destroy_plan(p);
        it = g_staged_plans.emplace(key, p).first;
    }
    const Plan& plan = it->second;
    if (!plan.has_algo) return false;
    if (epilogue != CUBLASLT_EPILOGUE_DEFAULT) cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias));

    if (!a_ready) launch_stage_bf16(A, Ab, rowsA, colsA, colsA, rowsA_p, lda_p, stream);
    if (!b_ready) launch_stage_bf16(B, Bb, rowsB, colsB, colsB, rowsB_p, ldb_p, stream);
    const float beta = 0.0f;
    const cublasStatus_t st = cublasLtMatmul(g_own_lt, plan.op, &alpha, Bb, plan.a, Ab, plan.b, &beta, Cp, plan.c, Cp, plan.c,
                                             &plan.algo, workspace, kStagedWorkspace, stream);
    if (st != CUBLAS_STATUS_SUCCESS) {
        report("cublasLtMatmul (staged BF16)", (int)st);
        return false;
    }
    if (pad_c) {
        launch_unpad_f32(Cp, C, M, N, ldc_p, N, stream);
    }
    return true;
}

}  // namespace

extern "C" long long b200gemm_tc_launches(void) { return b200gemm::tc_gemm_launches(); }
extern "C" long long b200gemm_staged_reuses(void) { return g_staged_reused; }
extern "C" void* b200gemm_bf16_twin(const void* fp32, int rows, int cols) {
    if (!fp32 || rows <= 0 || cols <= 0) return nullptr;
    std::lock_guard<std::mutex> lock(g_plans_mutex);
    if (!twins_enabled()) return nullptr;
    Twin& t = g_twins[fp32];
    if (t.bf16 && t.rows == rows && t.cols == cols) return t.bf16;
    if (t.bf16) cudaFree(t.bf16);
    t = Twin{};
    const size_t bytes = size_t(round_up_int(rows, 8)) * round_up_int(cols, 8) * 2;
    if (cudaMalloc(&t.bf16, bytes) != cudaSuccess || cudaMemset(t.bf16, 0, bytes) != cudaSuccess) {
        cudaGetLastError();
        if (t.bf16) cudaFree(t.bf16);
        g_twins.erase(fp32);
        return nullptr;
    }
    t.rows = rows, t.cols = cols;
    return t.bf16;
}
extern "C" void* b200gemm_bf16_twin_flat(const void* fp32, long long count) {
    if (!fp32 || count <= 0) return nullptr;
    std::lock_guard<std::mutex> lock(g_plans_mutex);
    if (!twins_enabled()) return nullptr;
    Twin& t = g_twins[fp32];
    if (t.bf16 && t.rows < 0 && t.count == count) return t.bf16;
    if (t.bf16) cudaFree(t.bf16);
    t = Twin{};
    if (cudaMalloc(&t.bf16, size_t(count) * 2) != cudaSuccess) {
        cudaGetLastError();
        g_twins.erase(fp32);
        return nullptr;
    }
    t.rows = -1, t.count = count;
    return t.bf16;
}
extern "C" void* b200gemm_bf16_twin_range(const void* fp32, long long count) {
    if (!fp32 || count <= 0) return nullptr;
    std::lock_guard<std::mutex> lock(g_plans_mutex);
    if (!twins_enabled()) return nullptr;
    for (const RangeTwin& r : g_range_twins)
        if (r.base == fp32 && r.count == count) return r.bf16;
    RangeTwin r;
    r.base = static_cast<const float*>(fp32), r.count = count;
    if (cudaMalloc(&r.bf16, size_t(count) * 2) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    g_range_twins.push_back(r);
    return r.bf16;
}
extern "C" void b200gemm_drop_twin_range(const void* fp32) {
    std::lock_guard<std::mutex> lock(g_plans_mutex);
    for (size_t i = 0; i < g_range_twins.size(); ++i) {
        if (g_range_twins[i].base != fp32) continue;
        cudaDeviceSynchronize();  // a product that reads the twin may still be running
        cudaFree(g_range_twins[i].bf16);
        g_range_twins.erase(g_range_twins.begin() + i);
        return;
    }
}
extern "C" long long b200gemm_twin_hits(void) { return g_twin_hits; }
extern "C" void b200gemm_release_twins(void) {
    std::lock_guard<std::mutex> lock(g_plans_mutex);
    cudaDeviceSynchronize();
    for (auto& kv : g_twins) cudaFree(kv.second.bf16);
    g_twins.clear();
    for (RangeTwin& r : g_range_twins) cudaFree(r.bf16);
    g_range_twins.clear();
}
extern "C" void b200gemm_forget_staged(void) {
    std::lock_guard<std::mutex> lock(g_plans_mutex);
    for (KeptOperand& k : g_kept) k.src = nullptr;
}

extern "C" int b200gemm_check_device_fault(void) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -2;
    const unsigned int word = b200gemm::tc_gemm_take_fault();
    if (word == 0) return 0;
    fprintf(stderr, "b200gemm: a bounded wait ran out inside the tcgen05 GEMM kernel (record 0x%08x)\n", word);
    return -3;
}

void matmul_forward(cublasHandle_t handle, const float* A, const float* B, float* C, int M, int N, int K, bool transA,
                    bool transB, float alpha, float beta, cudaStream_t stream) {
    if (wants_staging(M, N, K, transA, transB, beta) && staged_bf16_gemm(A, B, C, M, N, K, transA, transB, alpha, stream)) return;
    bind_stream(handle, stream);
    const int lda = transA ? M : K, ldb = transB ? K : N, ldc = N;
    report("cublasGemmEx", (int)cublasGemmEx(handle, transB ? CUBLAS_OP_T : CUBLAS_OP_N, transA ? CUBLAS_OP_T : CUBLAS_OP_N, N, M,
                                             K, &alpha, B, CUDA_R_32F, ldb, A, CUDA_R_32F, lda, &beta, C, CUDA_R_32F, ldc,
                                             compute_type(), CUBLAS_GEMM_DEFAULT));
}

void matmul_batched_strided(cublasHandle_t handle, const float* A, const float* B, float* C, int M, int N, int K,
                            long long int strideA, long long int strideB, long long int strideC, int batch_count, bool transA,
                            bool transB, float alpha, float beta, cudaStream_t stream) {
    bind_stream(handle, stream);
    const int lda = transA ? M : K, ldb = transB ? K : N, ldc = N;
    report("cublasGemmStridedBatchedEx",
           (int)cublasGemmStridedBatchedEx(handle, transB ? CUBLAS_OP_T : CUBLAS_OP_N, transA ? CUBLAS_OP_T : CUBLAS_OP_N, N, M, K,
                                           &alpha, B, CUDA_R_32F, ldb, strideB, A, CUDA_R_32F, lda, strideA, &beta, C, CUDA_R_32F,
                                           ldc, strideC, batch_count, compute_type(), CUBLAS_GEMM_DEFAULT));
}

void matmul_cublaslt(cublasLtHandle_t lt_handle, const float* A, const float* B, float* C, int M, int N, int K,
                     cublasLtEpilogue_t epilogue, const float* bias, void* workspace, size_t workspace_size, bool transA,
                     bool transB, float alpha, float beta, cudaStream_t stream) {
    if (workspace == nullptr) workspace_size = 0;
    if (wants_staging(M, N, K, transA, transB, beta) && staged_bf16_gemm(A, B, C, M, N, K, transA, transB, alpha, stream, epilogue, bias))
        return;
    const PlanKey key{M, N, K, transA ? 1 : 0, transB ? 1 : 0, (int)epilogue};
    Plan plan;
    {
        std::lock_guard<std::mutex> lock(g_plans_mutex);
        auto it = g_plans.find(key);
        if (it == g_plans.end()) {
            Plan p;
            if (!build_plan(lt_handle, key, compute_type(), workspace_size, &p) && math_mode() == Math::kBf16) {
                destroy_plan(p);  // no tensor-core algorithm for this shape / epilogue: FP32 arithmetic for it
                build_plan(lt_handle, key, CUBLAS_COMPUTE_32F, workspace_size, &p);
            }
            it = g_plans.emplace(key, p).first;
        }
        plan = it->second;
        if (bias != nullptr) cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias));
    }
    report("cublasLtMatmul", (int)cublasLtMatmul(lt_handle, plan.op, &alpha, B, plan.a, A, plan.b, &beta, C, plan.c, C, plan.c,
                                                 plan.has_algo ? &plan.algo : nullptr, workspace, workspace_size, stream));
}

void add_bias(float* Y, const float* bias, int M, int N, cudaStream_t stream) {
    const long long total = (long long)M * N;
    if (total == 0) return;
    const bool vec = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(bias)) & 15u) == 0;
    if (vec) {
        const long long groups = total / 4;
        add_bias_kernel<4><<<(unsigned int)((groups + 255) / 256), 256, 0, stream>>>(Y, bias, groups, N / 4);
    } else {
        add_bias_kernel<1><<<(unsigned int)((total + 255) / 256), 256, 0, stream>>>(Y, bias, total, N);
    }
}

void bias_backward(const float* dY, float* dbias, int M, int N, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return;
    // enough row strips to fill the 148 SMs a few times over, at least 64 rows each
    const int col_ctas = (N + 31) / 32;
    int strips = (148 * 4 + col_ctas - 1) / col_ctas;
    if (strips > (M + 63) / 64) strips = (M + 63) / 64;
    if (strips < 1) strips = 1;
    const int rows_per_cta = (M + strips - 1) / strips;
    bias_backward_kernel<<<dim3(col_ctas, (M + rows_per_cta - 1) / rows_per_cta), 256, 0, stream>>>(dY, dbias, M, N, rows_per_cta);
}
