/*
 * b200attn - causal multi-head self-attention (forward + backward) for NVIDIA B200 (sm_100a).
 *
 * C ABI of the engine. Plain pointers and sizes only; every pointer is a DEVICE pointer unless
 * stated otherwise, every call is asynchronous on the given stream (pass the cudaStream_t as a
 * void*; NULL is the default stream), and every call returns a status: 0 on success, negative on
 * failure (b200attn_last_error() then describes the failure for the calling thread).
 *
 * Each entry point names the launcher of sarimahsan/transformer-cuda that it stands in for
 * (file:line inside that project). The nine C++ launchers themselves, with their original
 * signatures, are declared in include/kernels/attention.cuh and forward to these functions.
 *
 * There is no CPU fallback: on a machine without a B200-class device every compute call fails.
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#ifdef __cplusplus
extern "C" {
#endif

#define B200ATTN_OK 0
#define B200ATTN_ERR_INVALID_ARGUMENT (-1) /* null pointer, non-positive size, misaligned buffer */
#define B200ATTN_ERR_UNSUPPORTED (-2)      /* shape outside what the selected math mode implements */
#define B200ATTN_ERR_CUDA (-3)             /* a CUDA runtime/driver call failed (message has the text) */
#define B200ATTN_ERR_SCRATCH (-4)          /* scratch memory too small and it cannot grow now
                                              (stream is capturing): call b200attn_reserve first */
#define B200ATTN_ERR_DEVICE_FAULT (-5)     /* a bounded wait inside a kernel ran out */

/* Math mode of the float* entry points b200attn_fwd_f32 / b200attn_bwd_f32. */
#define B200ATTN_MATH_FP32 0 /* SIMT FP32 arithmetic, exact expf: the parity mode (max-abs <= 1e-5) */
#define B200ATTN_MATH_BF16 1 /* inputs rounded to BF16, tcgen05 tensor cores, FP32 accumulation */

typedef void* b200attn_stream_t;

/* ------------------------------------------------------------------ library state ------------- */
int b200attn_version(void);
/* Message of the last failure on the calling thread ("" if none). Host pointer, valid until the
 * next failing call on this thread. */
const char* b200attn_last_error(void);
/* Process-wide math mode of the float* attention entry points. Initial value: the environment
 * variable B200ATTN_MATH ("fp32" or "bf16"), else FP32. */
int b200attn_set_math_mode(int mode);
int b200attn_get_math_mode(void);
/* Fused conversion for the float* API in BF16 math mode (off by default; initial value: the environment variable
 * B200ATTN_FUSED_CONVERT). When on, b200attn_qkv_split_f32 and b200attn_split_heads_f32 also write BF16 copies of
 * their FP32 outputs in the same pass (library-owned, keyed by the output tensor's address), and a later
 * b200attn_fwd_f32 / b200attn_bwd_f32 whose q, k, v (dO) are those very tensors uses the copies instead of running
 * one conversion pass per operand - seven passes per layer of src/model.cu:305-336,602-653. The caller promises not
 * to modify such a tensor between the layout call and the attention calls that consume it (the reference model does
 * not); a tensor that did not come from one of the two launchers is converted as before. The copies (2 bytes per
 * element of every registered tensor) are allocated on first use outside stream capture and freed by
 * b200attn_release. b200attn_fused_convert_hits counts the operand conversions skipped so far. No reference
 * counterpart (the reference is FP32 throughout). */
int b200attn_set_fused_convert(int on);
int b200attn_get_fused_convert(void);
long long b200attn_fused_convert_hits(void);
/* Grow the library-owned scratch of the current device so that later calls with shapes up to
 * (B*H, T, d) allocate nothing - required before such calls are recorded in a CUDA graph. */
int b200attn_reserve(int BH, int T, int d);
/* Free the scratch of the current device (after synchronising it). */
int b200attn_release(void);
/* Synchronise the current device and report the fault word written by kernels whose bounded
 * waits ran out (0 = none); clears the word. `code` is a HOST pointer and may be NULL. Allocates
 * nothing (a device on which no entry point has run yet simply reports 0). */
int b200attn_check_device_fault(unsigned int* code);

/* Self-test of that chain on a healthy GPU: launches one CTA that waits, with a limit of a few
 * thousand polls instead of the production 2^22, on a barrier nothing arrives on. The wait gives up,
 * the kernel ends normally, and the next b200attn_check_device_fault returns
 * B200ATTN_ERR_DEVICE_FAULT with code 0x57417E57 and clears the word; the context stays usable.
 * `report` (DEVICE pointer to 2 words, may be NULL) receives the CTA's abort flag and the duration
 * (in units of 1024 cycles) of a second wait that leaves early because the flag is set.
 * No reference counterpart (the reference has no waits and checks no launch). */
int b200attn_selftest_bounded_wait(unsigned int* report, b200attn_stream_t stream);

/* Per-launch timing of the two tensor-core kernels, for roofline reporting: with enable = N > 0,
 * every N-th launch of the forward / backward tcgen05 kernel is bracketed by CUDA events on its
 * stream (N = 1: every launch; an event record between two kernels undoes their programmatic
 * back-to-back launch, so N > 1 leaves most steps undisturbed; not to be enabled while capturing
 * a graph). Enabling (any N) or disabling (0) clears earlier records.
 * b200attn_kernel_times waits for the recorded launches and returns the summed durations in
 * milliseconds and the launch counts (HOST pointers, any may be NULL). No reference counterpart:
 * the reference times whole phases with its GpuTimer (include/common.h:35-62). */
int b200attn_kernel_timing(int enable);
int b200attn_kernel_times(double* fwd_ms_total, int* fwd_launches, double* bwd_ms_total, int* bwd_launches);
/* The single durations behind those sums, in launch order: up to `capacity` of the recorded launches of the
 * forward (backward = 0) or backward (backward = 1) kernel are written to `ms` (a HOST array, may be NULL
 * with capacity 0) and `count` receives how many were recorded in all. */
int b200attn_kernel_time_samples(int backward, float* ms, int capacity, int* count);

/* ------------------------------------------------------------------ FP32 API (drop-in) -------- */
/* (B,T,3*H*d) -> q,k,v (B,H,T,d).  Replaces qkv_split_transpose_forward,
 * include/kernels/attention.cuh:6, src/kernels/attention.cu:381. */
int b200attn_qkv_split_f32(const float* qkv, float* q, float* k, float* v, int B, int T, int H, int d,
                           b200attn_stream_t stream);
/* dq,dk,dv (B,H,T,d) -> dqkv (B,T,3*H*d), overwritten.  Replaces qkv_split_transpose_backward,
 * include/kernels/attention.cuh:14, src/kernels/attention.cu:408. */
int b200attn_qkv_merge_grad_f32(const float* dq, const float* dk, const float* dv, float* dqkv, int B, int T, int H,
                                int d, b200attn_stream_t stream);
/* probs = causal softmax(scale*scores), rows of length T, zeros above the diagonal.  Replaces
 * causal_softmax_forward, include/kernels/attention.cuh:25, src/kernels/attention.cu:435. */
int b200attn_causal_softmax_fwd_f32(const float* scores, float* probs, int B, int H, int T, float scale,
                                    b200attn_stream_t stream);
/* dscores = scale*p*(dp - sum(dp*p)), zeros above the diagonal.  Replaces causal_softmax_backward,
 * include/kernels/attention.cuh:82, src/kernels/attention.cu:450. */
int b200attn_causal_softmax_bwd_f32(const float* dprobs, const float* probs, float* dscores, int B, int H, int T,
                                    float scale, b200attn_stream_t stream);
/* out = softmax(scale*q k^T + causal) v; optional m_out (row max of scaled scores) and l_out
 * (sum exp(s-m)), each (B,H,T), may be NULL.  Replaces tiled_causal_attention_forward,
 * include/kernels/attention.cuh:39, src/kernels/attention.cu:626.  Unlike the reference, any
 * d in {32,64,128} works in both directions and other shapes fail instead of misbehaving. */
int b200attn_fwd_f32(const float* q, const float* k, const float* v, float* out, int B, int H, int T, int d,
                     float scale, float* m_out, float* l_out, b200attn_stream_t stream);
/* D[row] = sum_e dO*O.  Replaces attention_precompute_dot_do_o,
 * include/kernels/attention.cuh:52, src/kernels/attention.cu:679. */
int b200attn_dot_do_o_f32(const float* dO, const float* O, float* D, int B, int H, int T, int d,
                          b200attn_stream_t stream);
/* dq,dk,dv (overwritten) from q,k,v,o,dO and the saved m,l; `workspace` holds B*H*T floats
 * (caller-owned, receives D).  Replaces tiled_causal_attention_backward,
 * include/kernels/attention.cuh:63, src/kernels/attention.cu:957. */
int b200attn_bwd_f32(const float* q, const float* k, const float* v, const float* o, const float* dO,
                     const float* m, const float* l, float* dq, float* dk, float* dv, float* workspace, int B, int H,
                     int T, int d, float scale, b200attn_stream_t stream);
/* (B,H,T,d) -> (B,T,H*d).  Replaces head_merge_transpose_forward,
 * include/kernels/attention.cuh:92, src/kernels/attention.cu:466. */
int b200attn_merge_heads_f32(const float* in, float* out, int B, int H, int T, int d, b200attn_stream_t stream);
/* (B,T,H*d) -> (B,H,T,d).  Replaces head_merge_transpose_backward,
 * include/kernels/attention.cuh:100, src/kernels/attention.cu:491. */
int b200attn_split_heads_f32(const float* dout, float* din, int B, int H, int T, int d, b200attn_stream_t stream);

/* ------------------------------------------------------------------ BF16 API (tensor cores) --- */
/* BF16 tensors are passed as void* to 2-byte bfloat16 elements, layout (BH, T, d) contiguous with
 * BH = B*H slabs, 16-byte aligned; d in {64, 128}. Statistics are FP32. These are the entry points
 * a (batch, head) shard calls: pass the shard's slab count as BH and its offset pointers.
 * They have no counterpart in the reference, whose API is FP32 only; they compute the same
 * function as b200attn_fwd_f32 / b200attn_bwd_f32 (src/kernels/attention.cu:626, :957). */
/* out (BH,T,d) bf16; lse (BH,T) = m + log(l) in natural-log units (may not be NULL). */
int b200attn_fwd_bf16(const void* q, const void* k, const void* v, void* out, float* lse, int BH, int T, int d,
                      float scale, b200attn_stream_t stream);
/* dq,dk,dv (BH,T,d) bf16, overwritten. Uses library scratch (4*BH*T*d + 8*BH*T bytes). */
int b200attn_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse,
                      void* dq, void* dk, void* dv, int BH, int T, int d, float scale, b200attn_stream_t stream);
/* The same kernels on the model's own buffers, with no layout pass on either side: Q, K, V tiles are
 * fetched straight from the interleaved projection output qkv (B, T, 3*H*d) bf16 (inner order
 * [Q heads | K heads | V heads], the layout qkv_split_transpose_forward reads,
 * src/kernels/attention.cu:24-83) through strided tensor maps, and out is stored merged as
 * (B, T, H*d) bf16 (the layout head_merge_transpose_forward writes, src/kernels/attention.cu:308-345).
 * Replaces the chain split -> attention -> merge of src/model.cu:305-336. lse is (B*H, T). */
int b200attn_fwd_bf16_packed(const void* qkv, void* out, float* lse, int B, int T, int H, int d, float scale,
                             b200attn_stream_t stream);
/* Backward of the above: dout (B, T, H*d) bf16 in; dqkv (B, T, 3*H*d) bf16 out, overwritten (dK and dV
 * tiles are stored, and dQ is converted from its FP32 accumulator, directly into their interleaved
 * places). Replaces head_merge_transpose_backward -> attention backward -> qkv_split_transpose_backward
 * of src/model.cu:602-653. Uses library scratch like b200attn_bwd_bf16. */
int b200attn_bwd_bf16_packed(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv, int B,
                             int T, int H, int d, float scale, b200attn_stream_t stream);
/* The same backward for callers that must not allocate device memory: hosts whose own pool already
 * owns the whole GPU (a cudaMalloc from a plugin would fail or fragment it), latency-critical loops
 * that cannot take the device-wide synchronisation hidden in cudaMalloc/cudaFree, and sandboxes that
 * forbid allocation calls. It has no counterpart in the reference (whose callers allocate every
 * buffer themselves, src/model.cu:35-124). Scratch comes from a static device array of
 * B200ATTN_NOALLOC_SCRATCH_BYTES that every GPU loading the library holds until exit; the call makes
 * no cudaMalloc/cudaFree or other allocating call. Limits: 256 + 4*BH*T*d + 8*BH*T bytes (each part
 * rounded up to 256) must fit in the array, else B200ATTN_ERR_UNSUPPORTED (the benchmark shape
 * BH=96, T=1024, d=64 fits); b200attn_last_error() carries the text like for every other entry
 * point. All calls on a device share the array, which keeps the previous call's contents (each call
 * clears what must start from zero), so calls that overlap on the GPU race. The array also holds the
 * fault word of this entry point's kernels; b200attn_check_device_fault reads and clears it without
 * allocating. The first call on a device looks up the array's address - which makes the driver load
 * the module there: the 32 MiB are taken from the device at that moment and the driver may
 * synchronise - and clears the fault word synchronously. So make that first call at start-up, before
 * the host's own pool claims the rest of the GPU and outside any stream capture (a first call that
 * arrives while its stream is capturing returns B200ATTN_ERR_SCRATCH). */
#define B200ATTN_NOALLOC_SCRATCH_BYTES (32u * 1024u * 1024u)
int b200attn_bwd_bf16_noalloc(const void* q, const void* k, const void* v, const void* o, const void* dO,
                              const float* lse, void* dq, void* dk, void* dv, int BH, int T, int d, float scale,
                              b200attn_stream_t stream);
/* FP32 (B,T,3*H*d) -> BF16 q,k,v (B,H,T,d): the split-transpose fused with the down-conversion
 * (same index map as src/kernels/attention.cu:24-83). */
int b200attn_qkv_split_bf16(const float* qkv, void* q, void* k, void* v, int B, int T, int H, int d,
                            b200attn_stream_t stream);
/* BF16 dq,dk,dv (B,H,T,d) -> FP32 dqkv (B,T,3*H*d) (src/kernels/attention.cu:85-143). */
int b200attn_qkv_merge_grad_bf16(const void* dq, const void* dk, const void* dv, float* dqkv, int B, int T, int H,
                                 int d, b200attn_stream_t stream);
/* BF16 (B,H,T,d) -> FP32 (B,T,H*d) and FP32 (B,T,H*d) -> BF16 (B,H,T,d)
 * (src/kernels/attention.cu:308-379). */
int b200attn_merge_heads_bf16(const void* in, float* out, int B, int H, int T, int d, b200attn_stream_t stream);
int b200attn_split_heads_bf16(const float* dout, void* din, int B, int H, int T, int d, b200attn_stream_t stream);

/* ------------------------------------------------------------------ seeded synthetic inputs --- */
/* dst[i] = N(0,1) sample number (offset + i) of the stream `seed` (counter-based: the value depends
 * only on seed and the global element index, so a shard reproduces its part of the full tensor).
 * No counterpart in the reference (its benchmarks draw from torch.randn). */
int b200attn_fill_normal_f32(float* dst, long long n, unsigned long long seed, long long offset,
                             b200attn_stream_t stream);
int b200attn_fill_normal_bf16(void* dst, long long n, unsigned long long seed, long long offset,
                              b200attn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
