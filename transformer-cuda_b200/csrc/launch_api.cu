// The nine C++ launchers of include/kernels/attention.cuh, each a thin shim over the C ABI.
// The reference's launchers return void and never check launch errors
// (src/kernels/attention.cu:381-514, :626-657, :679-691, :957-1011); here a failure is reported on
// stderr once per call site and kept in b200attn_last_error().
#include <cstdio>

#include "../../include/b200attn.h"
#include "../../include/kernels/attention.cuh"

namespace {
inline void report(int rc, const char* launcher) {
    if (rc != B200ATTN_OK) fprintf(stderr, "[b200attn] %s failed (%d): %s\n", launcher, rc, b200attn_last_error());
}
}  // namespace

void qkv_split_transpose_forward(const float* qkv, float* q, float* k, float* v, int B, int T, int H, int d_head,
                                 cudaStream_t stream) {
    report(b200attn_qkv_split_f32(qkv, q, k, v, B, T, H, d_head, stream), __func__);
}

void qkv_split_transpose_backward(const float* dq, const float* dk, const float* dv, float* dqkv, int B, int T, int H,
                                  int d_head, cudaStream_t stream) {
    report(b200attn_qkv_merge_grad_f32(dq, dk, dv, dqkv, B, T, H, d_head, stream), __func__);
}

void causal_softmax_forward(const float* scores, float* probs, int B, int H, int T, float scale, cudaStream_t stream) {
    report(b200attn_causal_softmax_fwd_f32(scores, probs, B, H, T, scale, stream), __func__);
}

void tiled_causal_attention_forward(const float* q, const float* k, const float* v, float* out, int B, int H, int T,
                                    int d_head, float scale, float* m_out, float* l_out, cudaStream_t stream) {
    report(b200attn_fwd_f32(q, k, v, out, B, H, T, d_head, scale, m_out, l_out, stream), __func__);
}

void attention_precompute_dot_do_o(const float* dO, const float* O, float* D, int B, int H, int T, int d_head,
                                   cudaStream_t stream) {
    report(b200attn_dot_do_o_f32(dO, O, D, B, H, T, d_head, stream), __func__);
}

void tiled_causal_attention_backward(const float* q, const float* k, const float* v, const float* o,
                                     const float* do_ptr, const float* m_ptr, const float* l_ptr, float* dq, float* dk,
                                     float* dv, float* d_workspace, int B, int H, int T, int d_head, float scale,
                                     cudaStream_t stream) {
    report(b200attn_bwd_f32(q, k, v, o, do_ptr, m_ptr, l_ptr, dq, dk, dv, d_workspace, B, H, T, d_head, scale, stream),
           __func__);
}

void causal_softmax_backward(const float* dprobs, const float* probs, float* dscores, int B, int H, int T, float scale,
                             cudaStream_t stream) {
    report(b200attn_causal_softmax_bwd_f32(dprobs, probs, dscores, B, H, T, scale, stream), __func__);
}

void head_merge_transpose_forward(const float* in, float* out, int B, int H, int T, int d_head, cudaStream_t stream) {
    report(b200attn_merge_heads_f32(in, out, B, H, T, d_head, stream), __func__);
}

void head_merge_transpose_backward(const float* dout, float* din, int B, int H, int T, int d_head,
                                   cudaStream_t stream) {
    report(b200attn_split_heads_f32(dout, din, B, H, T, d_head, stream), __func__);
}
