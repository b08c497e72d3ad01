// Times the attention launch API (include/kernels/attention.cuh of sarimahsan/transformer-cuda) on
// one FP32 problem: tiled_causal_attention_forward + tiled_causal_attention_backward, CUDA events,
// best and median of N iterations after warm-up. TEST / BASELINE INFRASTRUCTURE: the same source is
// linked once against the reference's own src/kernels/attention.cu (the "reference kernels on this
// GPU" number) and once against libb200attn (the drop-in), by oracle/Makefile.
//
//   attn_bench B H T d [iters]
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime.h>

#include "kernels/attention.cuh"

#define CK(x)                                                                          \
    do {                                                                               \
        cudaError_t e_ = (x);                                                          \
        if (e_ != cudaSuccess) {                                                       \
            fprintf(stderr, "CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); \
            return 2;                                                                  \
        }                                                                              \
    } while (0)

int main(int argc, char** argv) {
    if (argc < 5) {
        fprintf(stderr, "usage: %s B H T d [iters]\n", argv[0]);
        return 1;
    }
    const int B = atoi(argv[1]), H = atoi(argv[2]), T = atoi(argv[3]), d = atoi(argv[4]);
    const int iters = argc > 5 ? atoi(argv[5]) : 10;
    const size_t n = size_t(B) * H * T * d, rows = size_t(B) * H * T;
    std::vector<float> h(n);
    unsigned long long s = 88172645463325252ull;
    auto rnd = [&]() {  // xorshift, sum of 4 uniforms ~ N(0, 1/3) scaled to unit variance
        float acc = 0.f;
        for (int i = 0; i < 4; ++i) {
            s ^= s << 13; s ^= s >> 7; s ^= s << 17;
            acc += float(s >> 40) * (1.0f / 16777216.0f) - 0.5f;
        }
        return acc * 1.7320508f;
    };
    float *q, *k, *v, *o, *dO, *dq, *dk, *dv, *m, *l, *ws;
    float** bufs[] = {&q, &k, &v, &o, &dO, &dq, &dk, &dv};
    for (auto b : bufs) CK(cudaMalloc(b, n * sizeof(float)));
    CK(cudaMalloc(&m, rows * 4)); CK(cudaMalloc(&l, rows * 4)); CK(cudaMalloc(&ws, rows * 4));
    for (float* dst : {q, k, v, dO}) {
        for (auto& x : h) x = rnd();
        CK(cudaMemcpy(dst, h.data(), n * sizeof(float), cudaMemcpyHostToDevice));
    }
    const float scale = 1.0f / sqrtf(float(d));
    cudaEvent_t e0, e1, e2;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1)); CK(cudaEventCreate(&e2));
    std::vector<float> tf, tb;
    for (int it = 0; it < iters + 3; ++it) {
        CK(cudaEventRecord(e0));
        tiled_causal_attention_forward(q, k, v, o, B, H, T, d, scale, m, l);
        CK(cudaEventRecord(e1));
        tiled_causal_attention_backward(q, k, v, o, dO, m, l, dq, dk, dv, ws, B, H, T, d, scale);
        CK(cudaEventRecord(e2));
        CK(cudaEventSynchronize(e2));
        float a, b;
        CK(cudaEventElapsedTime(&a, e0, e1)); CK(cudaEventElapsedTime(&b, e1, e2));
        if (it >= 3) { tf.push_back(a); tb.push_back(b); }
    }
    CK(cudaMemcpy(h.data(), dq, n * sizeof(float), cudaMemcpyDeviceToHost));
    double chk = 0; for (size_t i = 0; i < n; i += 997) chk += h[i];
    std::sort(tf.begin(), tf.end()); std::sort(tb.begin(), tb.end());
    const double fl = 2.0 * B * H * double(T) * T * d;
    printf("{\"B\":%d,\"H\":%d,\"T\":%d,\"d\":%d,\"fwd_ms_min\":%.4f,\"fwd_ms_med\":%.4f,\"bwd_ms_min\":%.4f,\"bwd_ms_med\":%.4f,"
           "\"fwd_bwd_tflops_med\":%.3f,\"dq_checksum\":%.6e}\n",
           B, H, T, d, tf.front(), tf[tf.size() / 2], tb.front(), tb[tb.size() / 2],
           3.5 * fl / ((tf[tf.size() / 2] + tb[tb.size() / 2]) * 1e-3) / 1e12, chk);
    return 0;
}
