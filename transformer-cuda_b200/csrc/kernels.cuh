// Internal launch interface between the C ABI (api.cu) and the kernel translation units.
// Every launcher enqueues on `stream` and returns the launch status; none allocates.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200attn {

// Launch with programmatic stream serialisation: the kernel may be scheduled while its predecessor in the stream is
// still draining (its prologue then overlaps the predecessor's tail). Kernels launched this way execute
// griddepcontrol.wait (pdl_wait() in tc_common.cuh) before their first global-memory access, so the data
// dependency through the stream is unchanged. Used for the kernels of the BF16 forward/backward chain, where the
// gaps between five short launches are a measurable share of a step.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------ layout_kernels.cu
// TOut is float or __nv_bfloat16 for the split, TIn likewise for the merges.
template <typename TOut>
cudaError_t launch_qkv_split(const float* qkv, TOut* q, TOut* k, TOut* v, int B, int T, int H, int d,
                             cudaStream_t stream);
template <typename TIn>
cudaError_t launch_qkv_merge_grad(const TIn* dq, const TIn* dk, const TIn* dv, float* dqkv, int B, int T, int H, int d,
                                  cudaStream_t stream, __nv_bfloat16* twin = nullptr);
// `twin` (both launchers): optional BF16 copy of the FP32 result written beside it, rows of round_up(row length, 8)
// elements - the layout in which the GEMM drop-in keeps BF16 operands (see twin_for in api.cu).
template <typename TIn>
cudaError_t launch_merge_heads(const TIn* in, float* out, int B, int H, int T, int d, cudaStream_t stream,
                               __nv_bfloat16* twin = nullptr);
template <typename TOut>
cudaError_t launch_split_heads(const float* dout, TOut* din, int B, int H, int T, int d, cudaStream_t stream);
// FP32 outputs plus BF16 copies in the same pass (d % 8 == 0, 16-byte aligned tensors: dual_layout_supported).
bool dual_layout_supported(int d, const void* a, const void* b, const void* c, const void* e);
cudaError_t launch_qkv_split_dual(const float* qkv, float* q, float* k, float* v, __nv_bfloat16* qb, __nv_bfloat16* kb,
                                  __nv_bfloat16* vb, int B, int T, int H, int d, cudaStream_t stream);
cudaError_t launch_split_heads_dual(const float* dout, float* din, __nv_bfloat16* din_bf16, int B, int H, int T, int d,
                                    cudaStream_t stream);
// dst = bf16(src * scale), elementwise
cudaError_t launch_f32_to_bf16(const float* src, __nv_bfloat16* dst, long long n, cudaStream_t stream, float scale = 1.0f);
cudaError_t launch_fill_normal_f32(float* dst, long long n, unsigned long long seed, long long offset,
                                   cudaStream_t stream);
cudaError_t launch_fill_normal_bf16(__nv_bfloat16* dst, long long n, unsigned long long seed, long long offset,
                                    cudaStream_t stream);

// ------------------------------------------------------------------ softmax_kernels.cu
cudaError_t launch_causal_softmax_fwd(const float* scores, float* probs, long long rows, int T, float scale,
                                      cudaStream_t stream);
cudaError_t launch_causal_softmax_bwd(const float* dprobs, const float* probs, float* dscores, long long rows, int T,
                                      float scale, cudaStream_t stream);

// ------------------------------------------------------------------ attn_f32.cu (SIMT FP32, parity mode)
cudaError_t launch_attn_fwd_f32(const float* q, const float* k, const float* v, float* out, float* m_out, float* l_out,
                                int BH, int T, int d, float scale, cudaStream_t stream);
cudaError_t launch_dot_do_o_f32(const float* dO, const float* O, float* D, long long rows, int d, cudaStream_t stream);
cudaError_t launch_attn_bwd_f32(const float* q, const float* k, const float* v, const float* dO, const float* m,
                                const float* l, const float* D, float* dq, float* dk, float* dv, int BH, int T, int d,
                                float scale, cudaStream_t stream);

// attn_f32_tiled.cu: shared-memory tiled variants for d in {32, 64, 128} with 16-byte aligned inputs;
// launch_attn_fwd_f32 / launch_attn_bwd_f32 pick them when attn_f32_tiled_supported() says so.
bool attn_f32_tiled_supported(int d, const void* a, const void* b, const void* c, const void* e);
cudaError_t launch_attn_fwd_f32_tiled(const float* q, const float* k, const float* v, float* out, float* m_out,
                                      float* l_out, int BH, int T, int d, float scale, cudaStream_t stream);
cudaError_t launch_attn_bwd_f32_tiled(const float* q, const float* k, const float* v, const float* dO, const float* m,
                                      const float* l, const float* D, float* dq, float* dk, float* dv, int BH, int T,
                                      int d, float scale, cudaStream_t stream);

// ------------------------------------------------------------------ attn_tc_fwd.cu / attn_tc_bwd.cu (tcgen05)
// Tensor maps are 4-D (d, T, H, B) with free T / H / B strides, box 64 x 128 x 1 x 1 (FP32: 32 x 128 x 1 x 1) and the
// 128-byte swizzle; slab bh = b*H + h. (B, H, T, d) slabs and the interleaved (B, T, 3*H*d) buffer differ only in strides.
struct TcFwdArgs {
    CUtensorMap map_q, map_k, map_v, map_o;  // BF16
    void* out;                               // BF16 or FP32 (BH, T, d), selected by out_is_f32
    int out_is_f32;
    float* m_out;                            // optional (BH, T): row max of scaled scores
    float* l_out;                            // optional (BH, T): sum exp(s - m)
    float* lse_out;                          // optional (BH, T): m + log(l)
    int BH, T, d;
    int H;                 // heads per batch entry of the maps (BH % H == 0); statistics stay (BH, T)
    int tile_major_order;  // 1: CTAs ordered longest tile first across all slabs; 0: slab by slab
    float scale;
    unsigned int* fault_word;
};
cudaError_t launch_attn_fwd_tc(const TcFwdArgs& a, cudaStream_t stream);        // picks the variant by T
cudaError_t launch_attn_fwd_tc_short(const TcFwdArgs& a, cudaStream_t stream);  // two CTAs per SM (d = 64; d = 128 up to T = 4096)

struct TcBwdArgs {
    CUtensorMap map_q, map_k, map_v, map_do;  // BF16
    CUtensorMap map_dk, map_dv;               // BF16 outputs (used when grads_are_f32 == 0)
    CUtensorMap map_dq_acc;                   // FP32 view of dq_acc (always dense (BH, T, d))
    const float* lse2;                        // (BH, T) log-sum-exp in log2 units: lse * log2(e)
    const float* D;                           // (BH, T) rowsum(dO * O)
    float* dq_acc;                            // (BH, T, d) FP32, zeroed before launch, receives sum of partials
    void* dk;                                 // BF16 or FP32 (BH, T, d)
    void* dv;
    int grads_are_f32;
    int BH, T, d;
    int H;                 // heads per batch entry of the maps (BH % H == 0)
    int tile_major_order;  // 1: CTAs ordered longest tile first across all slabs; 0: slab by slab
    float scale;
    unsigned int* fault_word;
    // used by the persistent head-dim-64 kernel only
    unsigned int* work_counter;          // device word, zero at launch: next work item to hand out
    long long grad_lt, grad_lh, grad_lb; // element strides (row, head, batch) of the BF16 dk / dv tensors
    CUtensorMap map_lse_ext, map_d_ext;  // BF16 (BH*T, 16) statistics rows written by the pre-pass (see BwdStatRows)
};
// Statistics rows for the persistent head-dim-64 kernel: per query row 16 BF16 = two identical 16-byte halves
// [hi, mid, lo, 0, 0, 0, 0, 0] with hi + mid + lo = -x/2 to 24 significant bits, x = lse/scale (lse_ext) or D (d_ext).
// One K = 16 MMA step against a tile of ones adds -x to every key row of S^T / dP^T. Both pointers null: not written.
struct BwdStatRows {
    __nv_bfloat16* lse_ext;
    __nv_bfloat16* d_ext;
    float inv_scale;  // 1 / softmax scale
};
// d = 128, and d = 64 when a.work_counter is NULL: one CTA per key tile. d = 64 with a work counter: the persistent
// kernel of attn_tc_bwd64.cu.
cudaError_t launch_attn_bwd_tc(const TcBwdArgs& a, cudaStream_t stream);
cudaError_t launch_attn_bwd_tc64(const TcBwdArgs& a, cudaStream_t stream);

// Backward pre-pass: D = rowsum(dO*O) and lse2 = (m + log l) * log2(e) or lse * log2(e).
// TIn is float or __nv_bfloat16. Exactly one of (m,l) / lse is given. If `zero` is not null the
// pass also clears that (rows, d) FP32 buffer (the dQ accumulator). d/VEC (VEC = 16 bytes of TIn)
// must be a power of two <= 32. If `counter` is not null the pass also clears that word (the work counter of the
// persistent backward kernel that follows it in the stream).
template <typename TIn>
cudaError_t launch_bwd_prepass(const TIn* o, const TIn* dO, const float* m, const float* l, const float* lse,
                               float* D, float* lse2, float* zero, long long rows, int d, cudaStream_t stream,
                               unsigned int* counter = nullptr, BwdStatRows ext = BwdStatRows{nullptr, nullptr, 0.f});
// The same for BF16 O / dO rows addressed as base + b*lb + h*lh + t*lt (+ e), row = (b*H + h)*T + t; lse given.
cudaError_t launch_bwd_prepass_strided(const __nv_bfloat16* o, const __nv_bfloat16* dO, const float* lse, float* D,
                                       float* lse2, float* zero, long long rows, int d, int T, int H, long long lt,
                                       long long lh, long long lb, cudaStream_t stream, unsigned int* counter = nullptr,
                                       BwdStatRows ext = BwdStatRows{nullptr, nullptr, 0.f});
// dq (BF16, rows addressed as above) = dq_acc (FP32, dense rows) * scale. The persistent head-dim-64 kernel leaves the
// softmax scale out of dS, so its dQ sums are scaled here; the other kernels pass 1.
cudaError_t launch_dq_convert_strided(const float* dq_acc, __nv_bfloat16* dq, long long rows, int d, int T, int H,
                                      long long lt, long long lh, long long lb, cudaStream_t stream, float scale = 1.0f);
// dq (BF16) = dq_acc (FP32) * scale, elementwise.
cudaError_t launch_dq_convert(const float* dq_acc, __nv_bfloat16* dq, long long n, cudaStream_t stream, float scale = 1.0f);

// ------------------------------------------------------------------ wait_selftest.cu
// One CTA waits (with a limit of a few thousand polls) on a barrier nothing arrives on, so that the wait gives up and
// records kFaultWaitTimeout | kWaitSelfTestId in *fault_word. report (2 words, device memory, may be NULL): the CTA's
// abort flag and how long a second wait took after the flag was set.
constexpr unsigned int kWaitSelfTestId = 0x7E57u;
cudaError_t launch_wait_selftest(unsigned int* fault_word, unsigned int* report, cudaStream_t stream);

// ------------------------------------------------------------------ host-side hooks between api.cu and static_scratch.cu
// Stores `text` as the calling thread's last error, i.e. what b200attn_last_error() returns (api.cu).
void set_last_error(const char* text);
// True while `stream` is being captured into a graph (api.cu).
bool stream_is_capturing(cudaStream_t stream);
// Fault word of the static-scratch backward on the current device (static_scratch.cu). Copies the word to
// *word and clears it on the device when it was set; *word = 0 when that entry point has not been used on
// this device yet. The caller has synchronised the device. Allocates nothing.
cudaError_t static_scratch_take_fault(unsigned int* word);

}  // namespace b200attn
