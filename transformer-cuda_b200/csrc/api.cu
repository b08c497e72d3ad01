// Host side of the engine: the extern "C" entry points declared in include/b200attn.h.
// Validates arguments, owns the per-device scratch memory and the device fault word, builds the
// TMA tensor maps, and dispatches to the kernels. No entry point synchronises or allocates on the
// hot path once scratch has been reserved; nothing here has a CPU fallback.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/b200attn.h"
#include "kernels.cuh"

// Defined by the GEMM drop-in (transformer-cuda_b200/gemm/matmul_dropin.cu) when it is linked into the same program;
// NULL otherwise (a weak reference: this library does not depend on it).
extern "C" void* b200gemm_bf16_twin(const void* fp32, int rows, int cols) __attribute__((weak));

namespace {

using namespace b200attn;

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}
int fail_cuda(cudaError_t e, const char* what) {
    return fail(B200ATTN_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define RETURN_IF_CUDA(expr, what)                      \
    do {                                                \
        cudaError_t _e = (expr);                        \
        if (_e != cudaSuccess) return fail_cuda(_e, what); \
    } while (0)

int initial_math_mode() {
    const char* s = getenv("B200ATTN_MATH");
    if (s && (strcmp(s, "bf16") == 0 || strcmp(s, "BF16") == 0 || strcmp(s, "1") == 0)) return B200ATTN_MATH_BF16;
    return B200ATTN_MATH_FP32;
}
std::atomic<int> g_math_mode{initial_math_mode()};
int initial_fused_convert() {
    const char* s = getenv("B200ATTN_FUSED_CONVERT");
    return (s && s[0] != '\0' && s[0] != '0') ? 1 : 0;
}
std::atomic<int> g_fused_convert{initial_fused_convert()};
std::atomic<long long> g_shadow_hits{0};

// ------------------------------------------------------------------ per-device state
constexpr int kMaxDevices = 64;
struct DeviceState {
    bool ready = false;
    bool is_sm100 = false;
    unsigned int* fault_word = nullptr;    // device memory: word 0 of a 64-byte block
    unsigned int* work_counter = nullptr;  // word 4 of the same block: item counter of the persistent backward
    uint8_t* scratch = nullptr;
    size_t scratch_bytes = 0;
    // BF16 copies of FP32 tensors, written by the layout launchers and consumed by the attention launchers of the
    // FP32 API in BF16 math mode (b200attn_set_fused_convert): keyed by the FP32 tensor's address.
    struct Shadow {
        const void* key;
        size_t n;  // elements
        __nv_bfloat16* data;
    };
    std::vector<Shadow> shadows;
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mutex;

// Optional per-launch timing of the two tensor-core kernels (CUDA events on the launching stream).
struct TimedLaunch {
    cudaEvent_t start, stop;
    int kind;  // 0 forward kernel, 1 backward kernel
};
std::atomic<int> g_timing_enabled{0};
std::atomic<int> g_timing_counter[2];
std::vector<TimedLaunch> g_timed;
std::mutex g_timed_mutex;

struct ScopedKernelTimer {
    cudaStream_t stream;
    TimedLaunch t{};
    bool active = false;
    ScopedKernelTimer(int kind, cudaStream_t s) : stream(s) {
        const int stride = g_timing_enabled.load();
        if (stride <= 0) return;
        // every stride-th launch of a kind is bracketed by events; the others keep their back-to-back
        // (programmatically serialised) launch, which an event record in between would undo
        if (g_timing_counter[kind & 1].fetch_add(1) % stride != 0) return;
        if (cudaEventCreate(&t.start) != cudaSuccess || cudaEventCreate(&t.stop) != cudaSuccess) return;
        t.kind = kind;
        active = cudaEventRecord(t.start, stream) == cudaSuccess;
    }
    ~ScopedKernelTimer() {
        if (!active) return;
        cudaEventRecord(t.stop, stream);
        std::lock_guard<std::mutex> lock(g_timed_mutex);
        g_timed.push_back(t);
    }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

using b200attn::stream_is_capturing;

// Looks up (and on first use initialises) the state of the current device.
int device_state(cudaStream_t stream, DeviceState** out) {
    int dev = 0;
    RETURN_IF_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(B200ATTN_ERR_CUDA, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        if (stream_is_capturing(stream))
            return fail(B200ATTN_ERR_SCRATCH, "first use on device %d happens inside a stream capture; call b200attn_reserve before capturing", dev);
        int major = 0, minor = 0;
        RETURN_IF_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "cudaDeviceGetAttribute");
        RETURN_IF_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev), "cudaDeviceGetAttribute");
        st.is_sm100 = (major == 10);
        RETURN_IF_CUDA(cudaMalloc(&st.fault_word, 64), "cudaMalloc(fault word)");
        RETURN_IF_CUDA(cudaMemset(st.fault_word, 0, 64), "cudaMemset(fault word)");
        st.work_counter = st.fault_word + 4;
        if (!g_encode) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            RETURN_IF_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q),
                           "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
            if (!fn) return fail(B200ATTN_ERR_CUDA, "driver does not export cuTensorMapEncodeTiled");
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
        st.ready = true;
    }
    *out = &st;
    return B200ATTN_OK;
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// BF16 twin of an FP32 matrix that a GEMM of the caller reads next (the merged attention output feeds the output
// projection, dqkv the QKV projection's backward): provided by the GEMM drop-in (libb200gemm) when that is linked into
// the same program and B200GEMM_TWINS=1, else there is none and only the FP32 result is written.
__nv_bfloat16* twin_for(const float* fp32, long long rows, long long cols) {
    if (!b200gemm_bf16_twin || rows > 0x7fffffffLL || cols > 0x7fffffffLL) return nullptr;
    return static_cast<__nv_bfloat16*>(b200gemm_bf16_twin(fp32, (int)rows, (int)cols));
}

// The BF16 copy registered for the FP32 tensor at `key` with exactly n elements, or NULL.
__nv_bfloat16* find_shadow(DeviceState* st, const void* key, size_t n) {
    std::lock_guard<std::mutex> lock(g_mutex);
    for (auto& sh : st->shadows)
        if (sh.key == key && sh.n == n) return sh.data;
    return nullptr;
}
// The same, created on first use (never while `stream` is capturing: NULL then, and the caller falls back).
__nv_bfloat16* find_or_make_shadow(DeviceState* st, const void* key, size_t n, cudaStream_t stream) {
    if (__nv_bfloat16* p = find_shadow(st, key, n)) return p;
    if (stream_is_capturing(stream)) return nullptr;
    std::lock_guard<std::mutex> lock(g_mutex);
    for (auto it = st->shadows.begin(); it != st->shadows.end();) {  // a tensor of another size now lives at this address
        if (it->key == key) {
            cudaDeviceSynchronize();
            cudaFree(it->data);
            it = st->shadows.erase(it);
        } else {
            ++it;
        }
    }
    __nv_bfloat16* p = nullptr;
    if (cudaMalloc(&p, round_up(n * sizeof(__nv_bfloat16), 256)) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    st->shadows.push_back(DeviceState::Shadow{key, n, p});
    return p;
}
bool fused_convert_on() { return g_fused_convert.load() != 0 && g_math_mode.load() == B200ATTN_MATH_BF16; }

// Makes the scratch of this device at least `bytes` large. Growing synchronises the device and
// is refused while `stream` is capturing.
int ensure_scratch(DeviceState* st, size_t bytes, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (st->scratch_bytes >= bytes) return B200ATTN_OK;
    if (stream_is_capturing(stream))
        return fail(B200ATTN_ERR_SCRATCH, "scratch of %zu bytes needed but only %zu reserved, and the stream is capturing; call b200attn_reserve first",
                    bytes, st->scratch_bytes);
    RETURN_IF_CUDA(cudaDeviceSynchronize(), "cudaDeviceSynchronize before growing scratch");
    if (st->scratch) RETURN_IF_CUDA(cudaFree(st->scratch), "cudaFree(scratch)");
    st->scratch = nullptr;
    st->scratch_bytes = 0;
    size_t want = round_up(bytes, size_t(1) << 20);
    RETURN_IF_CUDA(cudaMalloc(&st->scratch, want), "cudaMalloc(scratch)");
    st->scratch_bytes = want;
    return B200ATTN_OK;
}

// Scratch demand of the largest consumer (b200attn_bwd_f32 in BF16 mode and b200attn_bwd_bf16).
size_t scratch_for(long long BH, long long T, long long d) {
    const size_t n = size_t(BH) * T * d, rows = size_t(BH) * T;
    const size_t stat_rows = 2 * round_up(rows * 32, 256);                      // lse / D statistics rows (head dim 64)
    size_t f32_api = 4 * round_up(n * 2, 256) + round_up(rows * 4, 256) + stat_rows;   // bf16 q,k,v,dO + lse2
    size_t bf16_api = round_up(n * 4, 256) + 2 * round_up(rows * 4, 256) + stat_rows;  // dq accumulator + D + lse2
    return (f32_api > bf16_api ? f32_api : bf16_api) + 256;
}

struct Bump {
    uint8_t* p;
    template <typename T>
    T* take(size_t count) {
        T* r = reinterpret_cast<T*>(p);
        p += round_up(count * sizeof(T), 256);
        return r;
    }
};

// Element strides of a tensor indexed (b, h, t, e) with e contiguous.
struct Layout {
    long long t, h, b;
};
Layout slab_layout(int H, int T, int d) { return Layout{d, (long long)T * d, (long long)H * T * d}; }                  // (B, H, T, d)
Layout packed_qkv_layout(int H, int T, int d) { return Layout{3LL * H * d, d, 3LL * T * H * d}; }                        // (B, T, 3*H*d), one of Q|K|V
Layout merged_layout(int H, int T, int d) { return Layout{(long long)H * d, d, (long long)T * H * d}; }                // (B, T, H*d)

// (d, T, H, B) view of a BF16 (64 x 128 x 1 x 1 boxes) or FP32 (32 x 128 x 1 x 1 boxes: 128 bytes per row) tensor with
// the 128-byte swizzle. Rows beyond T are zero-filled on load and clipped on store, per (b, h).
int make_map(CUtensorMap* m, const void* base, bool f32, int B, int H, int T, int d, const Layout& L) {
    const cuuint64_t es = f32 ? 4 : 2;
    cuuint64_t dims[4] = {cuuint64_t(d), cuuint64_t(T), cuuint64_t(H), cuuint64_t(B)};
    cuuint64_t strides[3] = {cuuint64_t(L.t) * es, cuuint64_t(L.h) * es, cuuint64_t(L.b) * es};
    cuuint32_t box[4] = {f32 ? 32u : 64u, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = g_encode(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                          const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(B200ATTN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (B=%d H=%d T=%d d=%d, %s)", int(r), B, H, T, d,
                    f32 ? "FP32" : "BF16");
    return B200ATTN_OK;
}

// (16, T, H, B) view of the dense BF16 (B*H*T, 16) statistics rows: 16 x 128 x 1 x 1 boxes, 32-byte swizzle.
int make_stat_map(CUtensorMap* m, const void* base, int B, int H, int T) {
    cuuint64_t dims[4] = {16, cuuint64_t(T), cuuint64_t(H), cuuint64_t(B)};
    cuuint64_t strides[3] = {32, cuuint64_t(T) * 32, cuuint64_t(H) * T * 32};
    cuuint32_t box[4] = {16, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200ATTN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (statistics rows, B=%d H=%d T=%d)", int(r), B, H, T);
    return B200ATTN_OK;
}

// The persistent head-dim-64 backward folds 1/scale into its statistics rows, so it needs a usable scale.
bool use_persistent_bwd(int d, float scale) { return d == 64 && scale > 1e-20f && scale < 1e20f; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_dims4(const char* fn, int B, int H, int T, int d) {
    if (B < 0 || H < 0 || T < 0 || d <= 0) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: negative size or d <= 0 (B=%d H=%d T=%d d=%d)", fn, B, H, T, d);
    if ((long long)B * H > 0x7fffffffLL) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: B*H too large", fn);
    return B200ATTN_OK;
}
#define REQUIRE_PTR(fn, p) \
    if ((p) == nullptr) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: argument '%s' is NULL", fn, #p)

int tc_supported(const char* fn, DeviceState* st, int d) {
    if (!st->is_sm100) return fail(B200ATTN_ERR_UNSUPPORTED, "%s: the tensor-core path needs an sm_100a device (B200)", fn);
    if (d != 64 && d != 128) return fail(B200ATTN_ERR_UNSUPPORTED, "%s: the tensor-core path supports d in {64,128}, got %d", fn, d);
    return B200ATTN_OK;
}

// q, k, v share the layout `in_l`; a BF16 output is written through `out_l`, an FP32 output as dense (B*H, T, d).
int run_fwd_tc(DeviceState* st, const void* q, const void* k, const void* v, void* out, bool out_f32, float* m_out,
               float* l_out, float* lse_out, int B, int H, int T, int d, const Layout& in_l, const Layout& out_l,
               float scale, cudaStream_t stream) {
    TcFwdArgs a;
    memset(&a, 0, sizeof(a));
    const int BH = B * H;
    int rc;
    if ((rc = make_map(&a.map_q, q, false, B, H, T, d, in_l))) return rc;
    if ((rc = make_map(&a.map_k, k, false, B, H, T, d, in_l))) return rc;
    if ((rc = make_map(&a.map_v, v, false, B, H, T, d, in_l))) return rc;
    if (!out_f32) {
        if ((rc = make_map(&a.map_o, out, false, B, H, T, d, out_l))) return rc;
    }
    a.out = out;
    a.out_is_f32 = out_f32 ? 1 : 0;
    a.m_out = m_out;
    a.l_out = l_out;
    a.lse_out = lse_out;
    a.BH = BH, a.T = T, a.d = d, a.H = H;
    a.tile_major_order = (size_t(BH) * T * d * 2 * 4 <= (size_t(64) << 20)) ? 1 : 0;  // Q,K,V,dO fit in half of L2
    a.scale = scale;
    a.fault_word = st->fault_word;
    ScopedKernelTimer timer(0, stream);
    RETURN_IF_CUDA(launch_attn_fwd_tc(a, stream), "tensor-core forward launch");
    return B200ATTN_OK;
}

// q, k, v share `in_l`, dO uses `do_l`; BF16 dK/dV are written through `grad_l`, FP32 ones as dense (B*H, T, d);
// the FP32 dQ accumulator is always dense.
// `ext` holds the statistics rows the pre-pass wrote when use_persistent_bwd(d, scale), null pointers otherwise.
int run_bwd_tc(DeviceState* st, const void* q, const void* k, const void* v, const void* dO, const float* lse2,
               const float* D, float* dq_acc, void* dk, void* dv, bool grads_f32, int B, int H, int T, int d,
               const Layout& in_l, const Layout& do_l, const Layout& grad_l, float scale, cudaStream_t stream,
               const BwdStatRows& ext) {
    TcBwdArgs a;
    memset(&a, 0, sizeof(a));
    const int BH = B * H;
    int rc;
    if ((rc = make_map(&a.map_q, q, false, B, H, T, d, in_l))) return rc;
    if ((rc = make_map(&a.map_k, k, false, B, H, T, d, in_l))) return rc;
    if ((rc = make_map(&a.map_v, v, false, B, H, T, d, in_l))) return rc;
    if ((rc = make_map(&a.map_do, dO, false, B, H, T, d, do_l))) return rc;
    if (!grads_f32) {
        if ((rc = make_map(&a.map_dk, dk, false, B, H, T, d, grad_l))) return rc;
        if ((rc = make_map(&a.map_dv, dv, false, B, H, T, d, grad_l))) return rc;
    }
    if ((rc = make_map(&a.map_dq_acc, dq_acc, true, B, H, T, d, slab_layout(H, T, d)))) return rc;
    a.lse2 = lse2;
    a.D = D;
    a.dq_acc = dq_acc;
    a.dk = dk;
    a.dv = dv;
    a.grads_are_f32 = grads_f32 ? 1 : 0;
    a.BH = BH, a.T = T, a.d = d, a.H = H;
    a.tile_major_order = (size_t(BH) * T * d * 2 * 4 <= (size_t(64) << 20)) ? 1 : 0;  // Q,K,V,dO fit in half of L2
    a.scale = scale;
    a.fault_word = st->fault_word;
    if (ext.lse_ext) {
        if ((rc = make_stat_map(&a.map_lse_ext, ext.lse_ext, B, H, T))) return rc;
        if ((rc = make_stat_map(&a.map_d_ext, ext.d_ext, B, H, T))) return rc;
        a.work_counter = st->work_counter;  // cleared by the pre-pass that precedes this launch in the stream
    }
    a.grad_lt = grad_l.t, a.grad_lh = grad_l.h, a.grad_lb = grad_l.b;
    ScopedKernelTimer timer(1, stream);
    RETURN_IF_CUDA(launch_attn_bwd_tc(a, stream), "tensor-core backward launch");
    return B200ATTN_OK;
}

}  // namespace

namespace b200attn {
void set_last_error(const char* text) { snprintf(g_error, sizeof(g_error), "%s", text ? text : ""); }
bool stream_is_capturing(cudaStream_t s) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return st != cudaStreamCaptureStatusNone;
}
}  // namespace b200attn

// ====================================================================== library state
extern "C" int b200attn_version(void) { return 100; }

extern "C" const char* b200attn_last_error(void) { return g_error; }

extern "C" int b200attn_set_math_mode(int mode) {
    if (mode != B200ATTN_MATH_FP32 && mode != B200ATTN_MATH_BF16)
        return fail(B200ATTN_ERR_INVALID_ARGUMENT, "b200attn_set_math_mode: unknown mode %d", mode);
    g_math_mode.store(mode);
    return B200ATTN_OK;
}
extern "C" int b200attn_get_math_mode(void) { return g_math_mode.load(); }

extern "C" int b200attn_reserve(int BH, int T, int d) {
    if (BH < 0 || T < 0 || d <= 0) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "b200attn_reserve: bad shape (BH=%d T=%d d=%d)", BH, T, d);
    DeviceState* st = nullptr;
    int rc = device_state(nullptr, &st);
    if (rc) return rc;
    return ensure_scratch(st, scratch_for(BH, T, d), nullptr);
}

extern "C" int b200attn_release(void) {
    int dev = 0;
    RETURN_IF_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& st = g_dev[dev];
    if (!st.ready) return B200ATTN_OK;
    RETURN_IF_CUDA(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (st.scratch) cudaFree(st.scratch);
    st.scratch = nullptr;
    st.scratch_bytes = 0;
    for (auto& sh : st.shadows) cudaFree(sh.data);
    st.shadows.clear();
    return B200ATTN_OK;
}

extern "C" int b200attn_set_fused_convert(int on) {
    g_fused_convert.store(on ? 1 : 0);
    return B200ATTN_OK;
}
extern "C" int b200attn_get_fused_convert(void) { return g_fused_convert.load(); }
extern "C" long long b200attn_fused_convert_hits(void) { return g_shadow_hits.load(); }

extern "C" int b200attn_check_device_fault(unsigned int* code) {
    // Two words can hold a fault: the heap word of the allocating entry points (it exists only once one of
    // them has run on this device: this call must not be the one that allocates it, since hosts that use
    // only b200attn_bwd_bf16_noalloc cannot allocate) and the word inside the static scratch array.
    int dev = 0;
    RETURN_IF_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(B200ATTN_ERR_CUDA, "device index %d out of range", dev);
    RETURN_IF_CUDA(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    unsigned int w = 0, w_static = 0;
    unsigned int* heap_word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (g_dev[dev].ready) heap_word = g_dev[dev].fault_word;
    }
    if (heap_word) {
        RETURN_IF_CUDA(cudaMemcpy(&w, heap_word, sizeof(w), cudaMemcpyDeviceToHost), "cudaMemcpy(fault word)");
        if (w != 0) RETURN_IF_CUDA(cudaMemset(heap_word, 0, sizeof(w)), "cudaMemset(fault word)");
    }
    RETURN_IF_CUDA(static_scratch_take_fault(&w_static), "reading the static scratch fault word");
    if (w == 0) w = w_static;
    if (code) *code = w;
    if (w != 0) return fail(B200ATTN_ERR_DEVICE_FAULT, "a bounded wait inside a kernel ran out (fault word 0x%08x)", w);
    return B200ATTN_OK;
}

extern "C" int b200attn_selftest_bounded_wait(unsigned int* report, b200attn_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DeviceState* st = nullptr;
    int rc = device_state(stream, &st);
    if (rc) return rc;
    if (!st->is_sm100) return fail(B200ATTN_ERR_UNSUPPORTED, "b200attn_selftest_bounded_wait: needs an sm_100a device (B200)");
    RETURN_IF_CUDA(launch_wait_selftest(st->fault_word, report, stream), "wait self-test launch");
    return B200ATTN_OK;
}

extern "C" int b200attn_kernel_timing(int enable) {
    std::lock_guard<std::mutex> lock(g_timed_mutex);
    for (auto& t : g_timed) {
        cudaEventDestroy(t.start);
        cudaEventDestroy(t.stop);
    }
    g_timed.clear();
    g_timing_counter[0].store(0);
    g_timing_counter[1].store(0);
    g_timing_enabled.store(enable > 0 ? enable : 0);
    return B200ATTN_OK;
}

extern "C" int b200attn_kernel_times(double* fwd_ms_total, int* fwd_launches, double* bwd_ms_total, int* bwd_launches) {
    std::lock_guard<std::mutex> lock(g_timed_mutex);
    double tot[2] = {0.0, 0.0};
    int cnt[2] = {0, 0};
    for (auto& t : g_timed) {
        RETURN_IF_CUDA(cudaEventSynchronize(t.stop), "cudaEventSynchronize");
        float ms = 0.f;
        RETURN_IF_CUDA(cudaEventElapsedTime(&ms, t.start, t.stop), "cudaEventElapsedTime");
        tot[t.kind] += ms;
        cnt[t.kind] += 1;
    }
    if (fwd_ms_total) *fwd_ms_total = tot[0];
    if (fwd_launches) *fwd_launches = cnt[0];
    if (bwd_ms_total) *bwd_ms_total = tot[1];
    if (bwd_launches) *bwd_launches = cnt[1];
    return B200ATTN_OK;
}

extern "C" int b200attn_kernel_time_samples(int backward, float* ms_out, int capacity, int* count) {
    if (capacity < 0 || (capacity > 0 && !ms_out))
        return fail(B200ATTN_ERR_INVALID_ARGUMENT, "b200attn_kernel_time_samples: capacity %d with %s array", capacity,
                    ms_out ? "an" : "no");
    std::lock_guard<std::mutex> lock(g_timed_mutex);
    const int kind = backward ? 1 : 0;
    int n = 0;
    for (auto& t : g_timed) {
        if (t.kind != kind) continue;
        if (n < capacity) {
            RETURN_IF_CUDA(cudaEventSynchronize(t.stop), "cudaEventSynchronize");
            float ms = 0.f;
            RETURN_IF_CUDA(cudaEventElapsedTime(&ms, t.start, t.stop), "cudaEventElapsedTime");
            ms_out[n] = ms;
        }
        ++n;
    }
    if (count) *count = n;
    return B200ATTN_OK;
}

// ====================================================================== FP32 API
extern "C" int b200attn_qkv_split_f32(const float* qkv, float* q, float* k, float* v, int B, int T, int H, int d,
                                      b200attn_stream_t stream) {
    const char* fn = "b200attn_qkv_split_f32";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * T * H == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, qkv); REQUIRE_PTR(fn, q); REQUIRE_PTR(fn, k); REQUIRE_PTR(fn, v);
    if (fused_convert_on() && dual_layout_supported(d, qkv, q, k, v)) {
        // BF16 copies of q, k, v in the same pass, for the attention launchers that follow (no conversion passes there)
        DeviceState* st = nullptr;
        if ((rc = device_state((cudaStream_t)stream, &st))) return rc;
        const size_t n = size_t(B) * T * H * d;
        __nv_bfloat16* qb = find_or_make_shadow(st, q, n, (cudaStream_t)stream);
        __nv_bfloat16* kb = find_or_make_shadow(st, k, n, (cudaStream_t)stream);
        __nv_bfloat16* vb = find_or_make_shadow(st, v, n, (cudaStream_t)stream);
        if (qb && kb && vb) {
            RETURN_IF_CUDA(launch_qkv_split_dual(qkv, q, k, v, qb, kb, vb, B, T, H, d, (cudaStream_t)stream), fn);
            return B200ATTN_OK;
        }
    }
    RETURN_IF_CUDA(launch_qkv_split<float>(qkv, q, k, v, B, T, H, d, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_qkv_merge_grad_f32(const float* dq, const float* dk, const float* dv, float* dqkv, int B,
                                           int T, int H, int d, b200attn_stream_t stream) {
    const char* fn = "b200attn_qkv_merge_grad_f32";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * T * H == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, dq); REQUIRE_PTR(fn, dk); REQUIRE_PTR(fn, dv); REQUIRE_PTR(fn, dqkv);
    RETURN_IF_CUDA(launch_qkv_merge_grad<float>(dq, dk, dv, dqkv, B, T, H, d, (cudaStream_t)stream, twin_for(dqkv, B * T, 3 * H * d)), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_causal_softmax_fwd_f32(const float* scores, float* probs, int B, int H, int T, float scale,
                                               b200attn_stream_t stream) {
    const char* fn = "b200attn_causal_softmax_fwd_f32";
    int rc = check_dims4(fn, B, H, T, 1);
    if (rc) return rc;
    long long rows = (long long)B * H * T;
    if (rows == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, scores); REQUIRE_PTR(fn, probs);
    RETURN_IF_CUDA(launch_causal_softmax_fwd(scores, probs, rows, T, scale, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_causal_softmax_bwd_f32(const float* dprobs, const float* probs, float* dscores, int B, int H,
                                               int T, float scale, b200attn_stream_t stream) {
    const char* fn = "b200attn_causal_softmax_bwd_f32";
    int rc = check_dims4(fn, B, H, T, 1);
    if (rc) return rc;
    long long rows = (long long)B * H * T;
    if (rows == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, dprobs); REQUIRE_PTR(fn, probs); REQUIRE_PTR(fn, dscores);
    RETURN_IF_CUDA(launch_causal_softmax_bwd(dprobs, probs, dscores, rows, T, scale, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_fwd_f32(const float* q, const float* k, const float* v, float* out, int B, int H, int T, int d,
                                float scale, float* m_out, float* l_out, b200attn_stream_t stream_) {
    const char* fn = "b200attn_fwd_f32";
    cudaStream_t stream = (cudaStream_t)stream_;
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    const int BH = B * H;
    if ((long long)BH * T == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, q); REQUIRE_PTR(fn, k); REQUIRE_PTR(fn, v); REQUIRE_PTR(fn, out);
    if (g_math_mode.load() == B200ATTN_MATH_FP32) {
        if (d > 256) return fail(B200ATTN_ERR_UNSUPPORTED, "%s: FP32 mode supports d <= 256, got %d", fn, d);
        RETURN_IF_CUDA(launch_attn_fwd_f32(q, k, v, out, m_out, l_out, BH, T, d, scale, stream), fn);
        return B200ATTN_OK;
    }
    // BF16 mode: round the operands to BF16 in scratch, run the tensor-core kernel, write FP32 results.
    DeviceState* st = nullptr;
    if ((rc = device_state(stream, &st))) return rc;
    if ((rc = tc_supported(fn, st, d))) return rc;
    if (!aligned16(out)) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: out must be 16-byte aligned", fn);
    const size_t n = size_t(BH) * T * d;
    if ((rc = ensure_scratch(st, scratch_for(BH, T, d), stream))) return rc;
    Bump bump{st->scratch};
    const __nv_bfloat16* qb = fused_convert_on() ? find_shadow(st, q, n) : nullptr;
    const __nv_bfloat16* kb = fused_convert_on() ? find_shadow(st, k, n) : nullptr;
    const __nv_bfloat16* vb = fused_convert_on() ? find_shadow(st, v, n) : nullptr;
    if (qb && kb && vb) {
        g_shadow_hits.fetch_add(3);  // the split launcher left BF16 copies of these very tensors
    } else {
        __nv_bfloat16 *q2 = bump.take<__nv_bfloat16>(n), *k2 = bump.take<__nv_bfloat16>(n), *v2 = bump.take<__nv_bfloat16>(n);
        RETURN_IF_CUDA(launch_f32_to_bf16(q, q2, (long long)n, stream), "convert q");
        RETURN_IF_CUDA(launch_f32_to_bf16(k, k2, (long long)n, stream), "convert k");
        RETURN_IF_CUDA(launch_f32_to_bf16(v, v2, (long long)n, stream), "convert v");
        qb = q2, kb = k2, vb = v2;
    }
    const Layout sl = slab_layout(BH, T, d);
    return run_fwd_tc(st, qb, kb, vb, out, true, m_out, l_out, nullptr, 1, BH, T, d, sl, sl, scale, stream);
}

extern "C" int b200attn_dot_do_o_f32(const float* dO, const float* O, float* D, int B, int H, int T, int d,
                                     b200attn_stream_t stream) {
    const char* fn = "b200attn_dot_do_o_f32";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    long long rows = (long long)B * H * T;
    if (rows == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, dO); REQUIRE_PTR(fn, O); REQUIRE_PTR(fn, D);
    // 16-byte loads with d/4 threads per row when the shape allows it, else one warp per row
    const int tpr = d / 4;
    const bool wide = (d % 4 == 0) && tpr <= 32 && (tpr & (tpr - 1)) == 0 && aligned16(dO) && aligned16(O);
    if (wide)
        RETURN_IF_CUDA(launch_bwd_prepass<float>(O, dO, nullptr, nullptr, nullptr, D, nullptr, nullptr, rows, d, (cudaStream_t)stream), fn);
    else
        RETURN_IF_CUDA(launch_dot_do_o_f32(dO, O, D, rows, d, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_bwd_f32(const float* q, const float* k, const float* v, const float* o, const float* dO,
                                const float* m, const float* l, float* dq, float* dk, float* dv, float* workspace,
                                int B, int H, int T, int d, float scale, b200attn_stream_t stream_) {
    const char* fn = "b200attn_bwd_f32";
    cudaStream_t stream = (cudaStream_t)stream_;
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    const int BH = B * H;
    const long long rows = (long long)BH * T;
    if (rows == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, q); REQUIRE_PTR(fn, k); REQUIRE_PTR(fn, v); REQUIRE_PTR(fn, o); REQUIRE_PTR(fn, dO);
    REQUIRE_PTR(fn, m); REQUIRE_PTR(fn, l); REQUIRE_PTR(fn, dq); REQUIRE_PTR(fn, dk); REQUIRE_PTR(fn, dv);
    REQUIRE_PTR(fn, workspace);
    if (g_math_mode.load() == B200ATTN_MATH_FP32) {
        if (d > 256) return fail(B200ATTN_ERR_UNSUPPORTED, "%s: FP32 mode supports d <= 256, got %d", fn, d);
        {
            const int tpr = d / 4;
            const bool wide = (d % 4 == 0) && tpr <= 32 && (tpr & (tpr - 1)) == 0 && aligned16(dO) && aligned16(o);
            if (wide)
                RETURN_IF_CUDA(launch_bwd_prepass<float>(o, dO, nullptr, nullptr, nullptr, workspace, nullptr, nullptr, rows, d, stream), "D pre-pass");
            else
                RETURN_IF_CUDA(launch_dot_do_o_f32(dO, o, workspace, rows, d, stream), "D pre-pass");
        }
        RETURN_IF_CUDA(launch_attn_bwd_f32(q, k, v, dO, m, l, workspace, dq, dk, dv, BH, T, d, scale, stream), fn);
        return B200ATTN_OK;
    }
    DeviceState* st = nullptr;
    if ((rc = device_state(stream, &st))) return rc;
    if ((rc = tc_supported(fn, st, d))) return rc;
    if (!aligned16(dq) || !aligned16(dk) || !aligned16(dv) || !aligned16(o) || !aligned16(dO))
        return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: tensors must be 16-byte aligned", fn);
    const size_t n = size_t(BH) * T * d;
    if ((rc = ensure_scratch(st, scratch_for(BH, T, d), stream))) return rc;
    Bump bump{st->scratch};
    __nv_bfloat16* q2 = bump.take<__nv_bfloat16>(n);
    __nv_bfloat16* k2 = bump.take<__nv_bfloat16>(n);
    __nv_bfloat16* v2 = bump.take<__nv_bfloat16>(n);
    __nv_bfloat16* do2 = bump.take<__nv_bfloat16>(n);
    float* lse2 = bump.take<float>(size_t(rows));
    const bool fused = fused_convert_on();
    const __nv_bfloat16* qb = fused ? find_shadow(st, q, n) : nullptr;
    const __nv_bfloat16* kb = fused ? find_shadow(st, k, n) : nullptr;
    const __nv_bfloat16* vb = fused ? find_shadow(st, v, n) : nullptr;
    const __nv_bfloat16* dob = fused ? find_shadow(st, dO, n) : nullptr;
    BwdStatRows ext{nullptr, nullptr, 0.f};
    if (use_persistent_bwd(d, scale)) ext = BwdStatRows{bump.take<__nv_bfloat16>(size_t(rows) * 16), bump.take<__nv_bfloat16>(size_t(rows) * 16), 1.0f / scale};
    if (qb && kb && vb) {
        g_shadow_hits.fetch_add(3);
    } else {
        RETURN_IF_CUDA(launch_f32_to_bf16(q, q2, (long long)n, stream), "convert q");
        RETURN_IF_CUDA(launch_f32_to_bf16(k, k2, (long long)n, stream), "convert k");
        RETURN_IF_CUDA(launch_f32_to_bf16(v, v2, (long long)n, stream), "convert v");
        qb = q2, kb = k2, vb = v2;
    }
    if (dob) {
        g_shadow_hits.fetch_add(1);
    } else {
        RETURN_IF_CUDA(launch_f32_to_bf16(dO, do2, (long long)n, stream), "convert dO");
        dob = do2;
    }
    // dq is the FP32 accumulator itself: partial sums are reduced straight into the caller's buffer,
    // which the pre-pass clears
    RETURN_IF_CUDA(launch_bwd_prepass<float>(o, dO, m, l, nullptr, workspace, lse2, dq, rows, d, stream, st->work_counter, ext), "pre-pass");
    const Layout sl = slab_layout(BH, T, d);
    return run_bwd_tc(st, qb, kb, vb, dob, lse2, workspace, dq, dk, dv, true, 1, BH, T, d, sl, sl, sl, scale, stream, ext);
}

extern "C" int b200attn_merge_heads_f32(const float* in, float* out, int B, int H, int T, int d,
                                        b200attn_stream_t stream) {
    const char* fn = "b200attn_merge_heads_f32";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * T * H == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, in); REQUIRE_PTR(fn, out);
    RETURN_IF_CUDA(launch_merge_heads<float>(in, out, B, H, T, d, (cudaStream_t)stream, twin_for(out, B * T, H * d)), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_split_heads_f32(const float* dout, float* din, int B, int H, int T, int d,
                                        b200attn_stream_t stream) {
    const char* fn = "b200attn_split_heads_f32";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * T * H == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, dout); REQUIRE_PTR(fn, din);
    if (fused_convert_on() && dual_layout_supported(d, dout, din, din, din)) {
        DeviceState* st = nullptr;
        if ((rc = device_state((cudaStream_t)stream, &st))) return rc;
        if (__nv_bfloat16* db = find_or_make_shadow(st, din, size_t(B) * H * T * d, (cudaStream_t)stream)) {
            RETURN_IF_CUDA(launch_split_heads_dual(dout, din, db, B, H, T, d, (cudaStream_t)stream), fn);
            return B200ATTN_OK;
        }
    }
    RETURN_IF_CUDA(launch_split_heads<float>(dout, din, B, H, T, d, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

// ====================================================================== BF16 API
extern "C" int b200attn_fwd_bf16(const void* q, const void* k, const void* v, void* out, float* lse, int BH, int T,
                                 int d, float scale, b200attn_stream_t stream_) {
    const char* fn = "b200attn_fwd_bf16";
    cudaStream_t stream = (cudaStream_t)stream_;
    int rc = check_dims4(fn, BH, 1, T, d);
    if (rc) return rc;
    if ((long long)BH * T == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, q); REQUIRE_PTR(fn, k); REQUIRE_PTR(fn, v); REQUIRE_PTR(fn, out); REQUIRE_PTR(fn, lse);
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
        return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: tensors must be 16-byte aligned", fn);
    DeviceState* st = nullptr;
    if ((rc = device_state(stream, &st))) return rc;
    if ((rc = tc_supported(fn, st, d))) return rc;
    const Layout sl = slab_layout(BH, T, d);
    return run_fwd_tc(st, q, k, v, out, false, nullptr, nullptr, lse, 1, BH, T, d, sl, sl, scale, stream);
}

extern "C" int b200attn_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const void* dO,
                                 const float* lse, void* dq, void* dk, void* dv, int BH, int T, int d, float scale,
                                 b200attn_stream_t stream_) {
    const char* fn = "b200attn_bwd_bf16";
    cudaStream_t stream = (cudaStream_t)stream_;
    int rc = check_dims4(fn, BH, 1, T, d);
    if (rc) return rc;
    const long long rows = (long long)BH * T;
    if (rows == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, q); REQUIRE_PTR(fn, k); REQUIRE_PTR(fn, v); REQUIRE_PTR(fn, o); REQUIRE_PTR(fn, dO);
    REQUIRE_PTR(fn, lse); REQUIRE_PTR(fn, dq); REQUIRE_PTR(fn, dk); REQUIRE_PTR(fn, dv);
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dO) || !aligned16(dq) ||
        !aligned16(dk) || !aligned16(dv))
        return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: tensors must be 16-byte aligned", fn);
    DeviceState* st = nullptr;
    if ((rc = device_state(stream, &st))) return rc;
    if ((rc = tc_supported(fn, st, d))) return rc;
    const size_t n = size_t(BH) * T * d;
    if ((rc = ensure_scratch(st, scratch_for(BH, T, d), stream))) return rc;
    Bump bump{st->scratch};
    float* dq_acc = bump.take<float>(n);
    float* D = bump.take<float>(size_t(rows));
    float* lse2 = bump.take<float>(size_t(rows));
    BwdStatRows ext{nullptr, nullptr, 0.f};
    if (use_persistent_bwd(d, scale)) ext = BwdStatRows{bump.take<__nv_bfloat16>(size_t(rows) * 16), bump.take<__nv_bfloat16>(size_t(rows) * 16), 1.0f / scale};
    const __nv_bfloat16* ob = static_cast<const __nv_bfloat16*>(o);
    const __nv_bfloat16* dob = static_cast<const __nv_bfloat16*>(dO);
    RETURN_IF_CUDA(launch_bwd_prepass<__nv_bfloat16>(ob, dob, nullptr, nullptr, lse, D, lse2, dq_acc, rows, d, stream, st->work_counter, ext), "pre-pass");
    const Layout sl = slab_layout(BH, T, d);
    if ((rc = run_bwd_tc(st, q, k, v, dO, lse2, D, dq_acc, dk, dv, false, 1, BH, T, d, sl, sl, sl, scale, stream, ext))) return rc;
    // the persistent kernel leaves the softmax scale out of dS: dK is scaled where it is stored, dQ here
    RETURN_IF_CUDA(launch_dq_convert(dq_acc, static_cast<__nv_bfloat16*>(dq), (long long)n, stream, ext.lse_ext ? scale : 1.0f), "dq convert");
    return B200ATTN_OK;
}

// ---------------------------------------------------------------------- interleaved layouts
// The same kernels on the model's own buffers: Q, K, V tiles are fetched straight from the (B, T, 3*H*d)
// projection output and O is stored merged as (B, T, H*d), through strided tensor maps; no split / merge pass.
extern "C" int b200attn_fwd_bf16_packed(const void* qkv, void* out, float* lse, int B, int T, int H, int d, float scale,
                                        b200attn_stream_t stream_) {
    const char* fn = "b200attn_fwd_bf16_packed";
    cudaStream_t stream = (cudaStream_t)stream_;
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * H * T == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, qkv); REQUIRE_PTR(fn, out); REQUIRE_PTR(fn, lse);
    if (!aligned16(qkv) || !aligned16(out)) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: tensors must be 16-byte aligned", fn);
    DeviceState* st = nullptr;
    if ((rc = device_state(stream, &st))) return rc;
    if ((rc = tc_supported(fn, st, d))) return rc;
    const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(qkv);
    const size_t C = size_t(H) * d;
    return run_fwd_tc(st, base, base + C, base + 2 * C, out, false, nullptr, nullptr, lse, B, H, T, d,
                      packed_qkv_layout(H, T, d), merged_layout(H, T, d), scale, stream);
}

extern "C" int b200attn_bwd_bf16_packed(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                                        int B, int T, int H, int d, float scale, b200attn_stream_t stream_) {
    const char* fn = "b200attn_bwd_bf16_packed";
    cudaStream_t stream = (cudaStream_t)stream_;
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    const long long rows = (long long)B * H * T;
    if (rows == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, qkv); REQUIRE_PTR(fn, out); REQUIRE_PTR(fn, dout); REQUIRE_PTR(fn, lse); REQUIRE_PTR(fn, dqkv);
    if (!aligned16(qkv) || !aligned16(out) || !aligned16(dout) || !aligned16(dqkv))
        return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: tensors must be 16-byte aligned", fn);
    DeviceState* st = nullptr;
    if ((rc = device_state(stream, &st))) return rc;
    if ((rc = tc_supported(fn, st, d))) return rc;
    const int BH = B * H;
    const size_t n = size_t(rows) * d;
    if ((rc = ensure_scratch(st, scratch_for(BH, T, d), stream))) return rc;
    Bump bump{st->scratch};
    float* dq_acc = bump.take<float>(n);
    float* D = bump.take<float>(size_t(rows));
    float* lse2 = bump.take<float>(size_t(rows));
    BwdStatRows ext{nullptr, nullptr, 0.f};
    if (use_persistent_bwd(d, scale)) ext = BwdStatRows{bump.take<__nv_bfloat16>(size_t(rows) * 16), bump.take<__nv_bfloat16>(size_t(rows) * 16), 1.0f / scale};
    const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(qkv);
    __nv_bfloat16* gb = static_cast<__nv_bfloat16*>(dqkv);
    const size_t C = size_t(H) * d;
    const Layout pl = packed_qkv_layout(H, T, d), ml = merged_layout(H, T, d);
    RETURN_IF_CUDA(launch_bwd_prepass_strided(static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout),
                                              lse, D, lse2, dq_acc, rows, d, T, H, ml.t, ml.h, ml.b, stream, st->work_counter, ext), "pre-pass");
    if ((rc = run_bwd_tc(st, qb, qb + C, qb + 2 * C, dout, lse2, D, dq_acc, gb + C, gb + 2 * C, false, B, H, T, d, pl, ml, pl,
                         scale, stream, ext)))
        return rc;
    RETURN_IF_CUDA(launch_dq_convert_strided(dq_acc, gb, rows, d, T, H, pl.t, pl.h, pl.b, stream, ext.lse_ext ? scale : 1.0f), "dq convert");
    return B200ATTN_OK;
}

extern "C" int b200attn_qkv_split_bf16(const float* qkv, void* q, void* k, void* v, int B, int T, int H, int d,
                                       b200attn_stream_t stream) {
    const char* fn = "b200attn_qkv_split_bf16";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * T * H == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, qkv); REQUIRE_PTR(fn, q); REQUIRE_PTR(fn, k); REQUIRE_PTR(fn, v);
    RETURN_IF_CUDA(launch_qkv_split<__nv_bfloat16>(qkv, static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k),
                                                   static_cast<__nv_bfloat16*>(v), B, T, H, d, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_qkv_merge_grad_bf16(const void* dq, const void* dk, const void* dv, float* dqkv, int B, int T,
                                            int H, int d, b200attn_stream_t stream) {
    const char* fn = "b200attn_qkv_merge_grad_bf16";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * T * H == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, dq); REQUIRE_PTR(fn, dk); REQUIRE_PTR(fn, dv); REQUIRE_PTR(fn, dqkv);
    RETURN_IF_CUDA(launch_qkv_merge_grad<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(dq),
                                                        static_cast<const __nv_bfloat16*>(dk),
                                                        static_cast<const __nv_bfloat16*>(dv), dqkv, B, T, H, d,
                                                        (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_merge_heads_bf16(const void* in, float* out, int B, int H, int T, int d,
                                         b200attn_stream_t stream) {
    const char* fn = "b200attn_merge_heads_bf16";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * T * H == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, in); REQUIRE_PTR(fn, out);
    RETURN_IF_CUDA(launch_merge_heads<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(in), out, B, H, T, d, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_split_heads_bf16(const float* dout, void* din, int B, int H, int T, int d,
                                         b200attn_stream_t stream) {
    const char* fn = "b200attn_split_heads_bf16";
    int rc = check_dims4(fn, B, H, T, d);
    if (rc) return rc;
    if ((long long)B * T * H == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, dout); REQUIRE_PTR(fn, din);
    RETURN_IF_CUDA(launch_split_heads<__nv_bfloat16>(dout, static_cast<__nv_bfloat16*>(din), B, H, T, d, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

// ====================================================================== synthetic inputs
extern "C" int b200attn_fill_normal_f32(float* dst, long long n, unsigned long long seed, long long offset,
                                        b200attn_stream_t stream) {
    const char* fn = "b200attn_fill_normal_f32";
    if (n < 0 || offset < 0) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: negative count or offset", fn);
    if (n == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, dst);
    RETURN_IF_CUDA(launch_fill_normal_f32(dst, n, seed, offset, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}

extern "C" int b200attn_fill_normal_bf16(void* dst, long long n, unsigned long long seed, long long offset,
                                         b200attn_stream_t stream) {
    const char* fn = "b200attn_fill_normal_bf16";
    if (n < 0 || offset < 0) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "%s: negative count or offset", fn);
    if (n == 0) return B200ATTN_OK;
    REQUIRE_PTR(fn, dst);
    RETURN_IF_CUDA(launch_fill_normal_bf16(static_cast<__nv_bfloat16*>(dst), n, seed, offset, (cudaStream_t)stream), fn);
    return B200ATTN_OK;
}
