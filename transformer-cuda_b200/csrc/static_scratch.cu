// b200attn_bwd_bf16_noalloc: the BF16 backward for callers that must not allocate device memory.
//
// Who needs this. Some hosts hand the whole GPU to their own memory pool at start-up (inference
// servers, frameworks with a caching allocator set to take everything), so a later cudaMalloc from
// a plugin fails or fragments their pool. Others run inside a latency-critical loop where the
// implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable, or load this
// library into a sandbox whose policy forbids allocation calls altogether. b200attn_bwd_bf16 grows a
// library-owned heap buffer on demand and so does not suit them; this entry point takes the
// backward's scratch (FP32 dQ accumulator, D, log2-domain lse, and the fault word of the bounded
// waits) from a fixed array that is part of the loaded module instead. It calls no cudaMalloc,
// cudaFree, cudaMallocAsync or any other allocating routine.
//
// Costs and rules, all of which follow from the array being one static object per device:
//   * every GPU that loads the library holds B200ATTN_NOALLOC_SCRATCH_BYTES (32 MiB) until exit;
//   * shapes whose scratch does not fit are rejected with B200ATTN_ERR_UNSUPPORTED;
//   * all calls on a device share the array and it keeps the previous call's contents: the parts
//     that must start from zero (the dQ accumulator) are cleared on the stream by every call, and
//     two calls that overlap on the GPU (different streams, no dependency) race on it;
//   * the first call on each device looks up the array's device address and clears the fault word
//     with a synchronous memset, so make that first call before starting any stream capture.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/b200attn.h"
#include "kernels.cuh"

namespace {

using namespace b200attn;

constexpr size_t kScratchBytes = B200ATTN_NOALLOC_SCRATCH_BYTES;
constexpr size_t kFaultRegion = 256;  // first 256 bytes: the fault word of the kernels' bounded waits

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
struct PerDevice {
    unsigned char* base = nullptr;  // device address of g_noalloc_scratch on this device
    bool is_sm100 = false;
};
PerDevice g_per_device[kMaxDevices];
std::mutex g_setup_mutex;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_fn = nullptr;

// Formats the message and hands it to the buffer b200attn_last_error() returns for this thread.
int fail(int code, const char* fmt, ...) {
    char text[480];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(text, sizeof(text), fmt, ap);
    va_end(ap);
    char full[512];
    snprintf(full, sizeof(full), "b200attn_bwd_bf16_noalloc: %s", text);
    set_last_error(full);
    return code;
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Set-up, once per device, with that device current. The first cudaGetSymbolAddress on a device makes the
// driver load this module there, which is when the array's 32 MiB are taken from the device (and the
// driver may synchronise); the memset below is synchronous too. Both are illegal inside a stream capture,
// so a first call that arrives while `stream` is capturing is refused.
int setup_current_device(cudaStream_t stream, PerDevice** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(B200ATTN_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(B200ATTN_ERR_CUDA, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    PerDevice& pd = g_per_device[dev];
    if (pd.base == nullptr) {
        if (stream_is_capturing(stream))
            return fail(B200ATTN_ERR_SCRATCH, "first call on device %d arrives inside a stream capture; make one call before capturing", dev);
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(B200ATTN_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(e));
        e = cudaMemset(ptr, 0, kFaultRegion);
        if (e != cudaSuccess) return fail(B200ATTN_ERR_CUDA, "cudaMemset(fault word): %s", cudaGetErrorString(e));
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return fail(B200ATTN_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        pd.is_sm100 = (major == 10);
        if (!g_encode_fn) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
            if (e != cudaSuccess || !fn) return fail(B200ATTN_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
            g_encode_fn = reinterpret_cast<EncodeTiledFn>(fn);
        }
        pd.base = ptr;
    }
    *out = &pd;
    return B200ATTN_OK;
}

// Dense (BH, T, d) tensors as the 4-D (d, T, H = BH, B = 1) maps the kernels take. BF16: 64 x 128 x 1 x 1 boxes;
// the FP32 dQ accumulator: 32 x 128 x 1 x 1 boxes (both 128 bytes per row).
int encode_map(CUtensorMap* m, const void* base, int BH, int T, int d, bool f32 = false) {
    const cuuint64_t esz = f32 ? 4 : 2;
    cuuint64_t dims[4] = {cuuint64_t(d), cuuint64_t(T), cuuint64_t(BH), 1};
    cuuint64_t strides[3] = {cuuint64_t(d) * esz, cuuint64_t(T) * d * esz, cuuint64_t(BH) * T * d * esz};
    cuuint32_t box[4] = {f32 ? 32u : 64u, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = g_encode_fn(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                             const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200ATTN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", int(r));
    return B200ATTN_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

namespace b200attn {
cudaError_t static_scratch_take_fault(unsigned int* word) {
    *word = 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        base = g_per_device[dev].base;
    }
    if (!base) return cudaSuccess;  // never used on this device: nothing to read, and nothing gets loaded
    e = cudaMemcpy(word, base, sizeof(*word), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    if (*word != 0) e = cudaMemset(base, 0, sizeof(*word));
    return e;
}
}  // namespace b200attn

extern "C" int b200attn_bwd_bf16_noalloc(const void* q, const void* k, const void* v, const void* o, const void* dO,
                                         const float* lse, void* dq, void* dk, void* dv, int BH, int T, int d,
                                         float scale, b200attn_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (BH < 0 || T < 0 || d <= 0) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "negative size or d <= 0 (BH=%d T=%d d=%d)", BH, T, d);
    const size_t rows = size_t(BH) * T;
    if (rows == 0) return B200ATTN_OK;
    if (!q || !k || !v || !o || !dO || !lse || !dq || !dk || !dv) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "a tensor argument is NULL");
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dO) || !aligned16(dq) ||
        !aligned16(dk) || !aligned16(dv))
        return fail(B200ATTN_ERR_INVALID_ARGUMENT, "tensors must be 16-byte aligned");
    if (d != 64 && d != 128) return fail(B200ATTN_ERR_UNSUPPORTED, "d must be 64 or 128, got %d", d);
    // size check in a form that cannot wrap: a row costs 4*d + 8 bytes, so first bound the row count by
    // division, then (the products now being small) compute the exact demand with its 256-byte roundings
    const size_t row_bytes = size_t(d) * sizeof(float) + 2 * sizeof(float);
    const bool rows_fit = rows <= (kScratchBytes - kFaultRegion) / row_bytes;
    const size_t n = rows_fit ? rows * size_t(d) : 0;
    const size_t need = rows_fit ? kFaultRegion + round_up(n * sizeof(float), 256) + 2 * round_up(rows * sizeof(float), 256) : 0;
    if (!rows_fit || need > kScratchBytes)
        return fail(B200ATTN_ERR_UNSUPPORTED,
                    "shape BH=%d T=%d d=%d needs %zu rows of %zu bytes of scratch but the static array holds %zu bytes; use "
                    "b200attn_bwd_bf16 or split the (batch, head) slabs over several calls", BH, T, d, rows, row_bytes, kScratchBytes);
    PerDevice* pd = nullptr;
    int rc = setup_current_device(stream, &pd);
    if (rc) return rc;
    if (!pd->is_sm100) return fail(B200ATTN_ERR_UNSUPPORTED, "needs an sm_100a device (B200)");

    unsigned char* p = pd->base;
    unsigned int* fault_word = reinterpret_cast<unsigned int*>(p);
    p += kFaultRegion;
    float* dq_acc = reinterpret_cast<float*>(p);
    p += round_up(n * sizeof(float), 256);
    float* D = reinterpret_cast<float*>(p);
    p += round_up(rows * sizeof(float), 256);
    float* lse2 = reinterpret_cast<float*>(p);

    TcBwdArgs a;
    memset(&a, 0, sizeof(a));
    if ((rc = encode_map(&a.map_q, q, BH, T, d))) return rc;
    if ((rc = encode_map(&a.map_k, k, BH, T, d))) return rc;
    if ((rc = encode_map(&a.map_v, v, BH, T, d))) return rc;
    if ((rc = encode_map(&a.map_do, dO, BH, T, d))) return rc;
    if ((rc = encode_map(&a.map_dk, dk, BH, T, d))) return rc;
    if ((rc = encode_map(&a.map_dv, dv, BH, T, d))) return rc;
    if ((rc = encode_map(&a.map_dq_acc, dq_acc, BH, T, d, true))) return rc;
    a.lse2 = lse2;
    a.D = D;
    a.dq_acc = dq_acc;
    a.dk = dk;
    a.dv = dv;
    a.grads_are_f32 = 0;
    a.BH = BH, a.T = T, a.d = d, a.H = BH;
    a.tile_major_order = (size_t(BH) * T * d * 2 * 4 <= (size_t(64) << 20)) ? 1 : 0;  // Q,K,V,dO fit in half of L2
    a.scale = scale;
    a.fault_word = fault_word;
    a.work_counter = nullptr;  // one CTA per key tile: the kernel variant whose scratch is what the header documents

    cudaError_t e = launch_bwd_prepass<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dO),
                                                      nullptr, nullptr, lse, D, lse2, nullptr, (long long)rows, d, stream);
    if (e != cudaSuccess) return fail(B200ATTN_ERR_CUDA, "pre-pass launch: %s", cudaGetErrorString(e));
    // the accumulator still holds the previous call's sums: it must start from zero
    e = cudaMemsetAsync(dq_acc, 0, n * sizeof(float), stream);
    if (e != cudaSuccess) return fail(B200ATTN_ERR_CUDA, "cudaMemsetAsync(dq accumulator): %s", cudaGetErrorString(e));
    e = launch_attn_bwd_tc(a, stream);
    if (e != cudaSuccess) return fail(B200ATTN_ERR_CUDA, "backward launch: %s", cudaGetErrorString(e));
    e = launch_dq_convert(dq_acc, static_cast<__nv_bfloat16*>(dq), (long long)n, stream);
    if (e != cudaSuccess) return fail(B200ATTN_ERR_CUDA, "dq convert launch: %s", cudaGetErrorString(e));
    return B200ATTN_OK;
}
