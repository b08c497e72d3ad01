// Checker for the GEMM drop-in (transformer-cuda_b200/gemm/matmul_dropin.cu); test infrastructure, not product.
// Runs every wrapper declared in include/kernels/matmul.cuh on seeded inputs and compares with a plain FP64
// host computation of C = alpha * op(A) op(B) + beta * C on a sample of output elements. Shapes include
// leading dimensions that are not multiples of four floats (the language-model head of the reference model,
// V = 50257), large enough to take the staged BF16 path when B200GEMM_MATH=bf16.
// Prints one JSON line per case: {"case": ..., "max_rel": ..., "ok": ...}; exit code 0 iff all are within tolerance.
// usage: gemm_check [tolerance]   (default 1e-5 relative to the row/column scale; pass 2e-2 for BF16 arithmetic)
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "kernels/matmul.cuh"

#define CK(x)                                                                              \
    do {                                                                                   \
        cudaError_t e_ = (x);                                                              \
        if (e_ != cudaSuccess) {                                                           \
            printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__);        \
            exit(2);                                                                       \
        }                                                                                  \
    } while (0)

static unsigned long long g_state = 88172645463325252ull;
static float next_uniform() {  // xorshift64, values in [-1, 1)
    g_state ^= g_state << 13;
    g_state ^= g_state >> 7;
    g_state ^= g_state << 17;
    return float((g_state >> 11) & 0xFFFFFF) / float(0x800000) - 1.0f;
}

struct Case {
    const char* name;
    int M, N, K;
    bool transA, transB;
    float alpha, beta;
    int api;  // 0 matmul_forward, 1 matmul_cublaslt, 2 matmul_cublaslt + BIAS epilogue
};

int main(int argc, char** argv) {
    const double tol = argc > 1 ? atof(argv[1]) : 1e-5;
    cublasHandle_t handle;
    cublasLtHandle_t lt;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS || cublasLtCreate(&lt) != CUBLAS_STATUS_SUCCESS) return 2;
    void* workspace;
    const size_t ws_bytes = 32u << 20;
    CK(cudaMalloc(&workspace, ws_bytes));
    const Case cases[] = {
        {"aligned_small", 96, 128, 64, false, false, 1.0f, 0.0f, 0},
        {"aligned_lt_bias", 256, 384, 128, false, false, 1.0f, 0.0f, 2},
        {"transA_beta", 64, 96, 200, true, false, 0.5f, 1.0f, 1},
        {"head_forward_unaligned", 2048, 50257, 768, false, false, 1.0f, 0.0f, 1},   // logits = X W
        {"head_dw_unaligned", 768, 50257, 2048, true, false, 1.0f, 0.0f, 1},          // dW = X^T dlogits
        {"head_dx_unaligned", 2048, 768, 50257, false, true, 1.0f, 0.0f, 0},          // dX = dlogits W^T
        {"unaligned_small", 33, 77, 45, false, true, 1.0f, 0.0f, 0},
        // large aligned and ragged products in all four operand layouts: staged in BF16 arithmetic, and with
        // B200GEMM_KERNEL=tcgen05 multiplied by the hand-written kernel (each has at least 120 output tiles of 128 x 256)
        {"layer_nn", 4096, 3072, 768, false, false, 1.0f, 0.0f, 1},
        {"layer_nt", 4096, 3072, 768, false, true, 1.0f, 0.0f, 1},
        {"ragged_tn", 2000, 3000, 1000, true, false, 0.5f, 0.0f, 0},
        {"ragged_tt", 2000, 3000, 1000, true, true, 1.0f, 0.0f, 0},
        {"ragged_unaligned_nn", 1999, 3001, 777, false, false, 1.0f, 0.0f, 1},
    };
    bool all_ok = true;
    for (const Case& c : cases) {
        b200gemm_forget_staged();  // every case fills fresh buffers, possibly at the addresses of the previous case's
        const size_t na = size_t(c.M) * c.K, nb = size_t(c.K) * c.N, nc = size_t(c.M) * c.N;
        std::vector<float> A(na), B(nb), C0(nc), bias(c.N), C(nc);
        for (auto& x : A) x = next_uniform();
        for (auto& x : B) x = next_uniform();
        for (auto& x : C0) x = next_uniform();
        for (auto& x : bias) x = next_uniform();
        float *dA, *dB, *dC, *dbias;
        CK(cudaMalloc(&dA, na * 4)); CK(cudaMalloc(&dB, nb * 4)); CK(cudaMalloc(&dC, nc * 4)); CK(cudaMalloc(&dbias, c.N * 4));
        CK(cudaMemcpy(dA, A.data(), na * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dB, B.data(), nb * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dC, C0.data(), nc * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dbias, bias.data(), c.N * 4, cudaMemcpyHostToDevice));
        if (c.api == 0) matmul_forward(handle, dA, dB, dC, c.M, c.N, c.K, c.transA, c.transB, c.alpha, c.beta, 0);
        else matmul_cublaslt(lt, dA, dB, dC, c.M, c.N, c.K, c.api == 2 ? CUBLASLT_EPILOGUE_BIAS : CUBLASLT_EPILOGUE_DEFAULT,
                             c.api == 2 ? dbias : nullptr, workspace, ws_bytes, c.transA, c.transB, c.alpha, c.beta, 0);
        CK(cudaDeviceSynchronize());
        CK(cudaMemcpy(C.data(), dC, nc * 4, cudaMemcpyDeviceToHost));
        // sample of outputs: corners, last column / row, and a seeded scatter
        double max_rel = 0.0;
        const int samples = 4000;
        for (int s = 0; s < samples; ++s) {
            int i, j;
            if (s == 0) i = 0, j = 0;
            else if (s == 1) i = c.M - 1, j = c.N - 1;
            else if (s == 2) i = 0, j = c.N - 1;
            else if (s == 3) i = c.M - 1, j = 0;
            else i = int((next_uniform() * 0.5f + 0.5f) * c.M) % c.M, j = int((next_uniform() * 0.5f + 0.5f) * c.N) % c.N;
            double acc = 0.0, scale = 0.0;
            for (int k = 0; k < c.K; ++k) {
                const double a = c.transA ? A[size_t(k) * c.M + i] : A[size_t(i) * c.K + k];
                const double b = c.transB ? B[size_t(j) * c.K + k] : B[size_t(k) * c.N + j];
                acc += a * b;
                scale += fabs(a * b);
            }
            double want = c.alpha * acc + c.beta * C0[size_t(i) * c.N + j] + (c.api == 2 ? bias[j] : 0.0);
            const double rel = fabs(double(C[size_t(i) * c.N + j]) - want) / (scale / sqrt(double(c.K)) + 1.0);
            if (!(rel <= max_rel)) max_rel = rel;  // also catches NaN
        }
        const bool ok = max_rel <= tol;
        all_ok = all_ok && ok;
        printf("{\"case\": \"%s\", \"M\": %d, \"N\": %d, \"K\": %d, \"max_rel\": %.3e, \"ok\": %s}\n", c.name, c.M, c.N, c.K, max_rel,
               ok ? "true" : "false");
        cudaFree(dA); cudaFree(dB); cudaFree(dC); cudaFree(dbias);
    }
    // bias helpers
    {
        const int M = 1000, N = 50257;
        std::vector<float> Y(size_t(M) * N), b(N), db(N, 0.25f);
        for (auto& x : Y) x = next_uniform();
        for (auto& x : b) x = next_uniform();
        float *dY, *dbv, *ddb;
        CK(cudaMalloc(&dY, Y.size() * 4)); CK(cudaMalloc(&dbv, N * 4)); CK(cudaMalloc(&ddb, N * 4));
        CK(cudaMemcpy(dY, Y.data(), Y.size() * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dbv, b.data(), N * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(ddb, db.data(), N * 4, cudaMemcpyHostToDevice));
        bias_backward(dY, ddb, M, N, 0);  // accumulates onto 0.25
        add_bias(dY, dbv, M, N, 0);
        std::vector<float> Y2(Y.size()), db2(N);
        CK(cudaDeviceSynchronize());
        CK(cudaMemcpy(Y2.data(), dY, Y.size() * 4, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(db2.data(), ddb, N * 4, cudaMemcpyDeviceToHost));
        double e1 = 0, e2 = 0;
        for (int j = 0; j < N; j += 97) {
            double s = 0.25;
            for (int i = 0; i < M; ++i) s += Y[size_t(i) * N + j];
            e1 = fmax(e1, fabs(s - db2[j]));
        }
        for (size_t idx = 0; idx < Y.size(); idx += 1013) e2 = fmax(e2, fabs(double(Y[idx]) + b[idx % N] - Y2[idx]));
        const bool ok = e1 <= 1e-3 && e2 <= 1e-6;
        all_ok = all_ok && ok;
        printf("{\"case\": \"bias_helpers\", \"bias_backward_max_abs\": %.3e, \"add_bias_max_abs\": %.3e, \"ok\": %s}\n", e1, e2, ok ? "true" : "false");
    }
    // the backward pair dW = X^T dY, dX = dY W^T: with B200GEMM_REUSE_STAGED=1 the second call takes dY's BF16 copy from the first
    {
        const int R = 4096, C1 = 768, C2 = 3072;
        std::vector<float> X(size_t(R) * C1), dY(size_t(R) * C2), W(size_t(C1) * C2), dX(size_t(R) * C1);
        for (auto& x : X) x = next_uniform();
        for (auto& x : dY) x = next_uniform();
        for (auto& x : W) x = next_uniform();
        float *dXa, *ddY, *dW, *ddW, *ddX;
        CK(cudaMalloc(&dXa, X.size() * 4)); CK(cudaMalloc(&ddY, dY.size() * 4)); CK(cudaMalloc(&dW, W.size() * 4));
        CK(cudaMalloc(&ddW, W.size() * 4)); CK(cudaMalloc(&ddX, dX.size() * 4));
        CK(cudaMemcpy(dXa, X.data(), X.size() * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(ddY, dY.data(), dY.size() * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dW, W.data(), W.size() * 4, cudaMemcpyHostToDevice));
        const long long before = b200gemm_staged_reuses();
        matmul_cublaslt(lt, dXa, ddY, ddW, C1, C2, R, CUBLASLT_EPILOGUE_DEFAULT, nullptr, workspace, ws_bytes, true, false, 1.0f, 0.0f, 0);
        matmul_cublaslt(lt, ddY, dW, ddX, R, C1, C2, CUBLASLT_EPILOGUE_DEFAULT, nullptr, workspace, ws_bytes, false, true, 1.0f, 0.0f, 0);
        CK(cudaDeviceSynchronize());
        CK(cudaMemcpy(dX.data(), ddX, dX.size() * 4, cudaMemcpyDeviceToHost));
        double max_rel = 0.0;
        for (int s = 0; s < 2000; ++s) {
            const int i = int((next_uniform() * 0.5f + 0.5f) * R) % R, j = int((next_uniform() * 0.5f + 0.5f) * C1) % C1;
            double acc = 0.0, scale = 0.0;
            for (int k = 0; k < C2; ++k) {
                const double p = double(dY[size_t(i) * C2 + k]) * W[size_t(j) * C2 + k];
                acc += p, scale += fabs(p);
            }
            const double rel = fabs(double(dX[size_t(i) * C1 + j]) - acc) / (scale / sqrt(double(C2)) + 1.0);
            if (!(rel <= max_rel)) max_rel = rel;
        }
        const bool ok = max_rel <= tol;
        all_ok = all_ok && ok;
        printf("{\"case\": \"backward_pair_dx\", \"max_rel\": %.3e, \"staged_reuses\": %lld, \"ok\": %s}\n", max_rel,
               b200gemm_staged_reuses() - before, ok ? "true" : "false");
        cudaFree(dXa); cudaFree(ddY); cudaFree(dW); cudaFree(ddW); cudaFree(ddX);
    }
    // a BF16 twin of a flat buffer that holds matrices back to back (what the AdamW drop-in keeps of the parameters): the
    // twin is filled with TWICE the FP32 values here, so a product that reads it is told apart from one that converts
    {
        const int R = 4096, C1 = 768, C2 = 3072, lead = 128;
        const size_t nw = size_t(C1) * C2, total = lead + nw + 5;
        std::vector<float> P(total), X(size_t(R) * C1), Y(size_t(R) * C2);
        for (auto& x : P) x = next_uniform();
        for (auto& x : X) x = next_uniform();
        float *dP, *dXa, *dYa;
        CK(cudaMalloc(&dP, total * 4)); CK(cudaMalloc(&dXa, X.size() * 4)); CK(cudaMalloc(&dYa, Y.size() * 4));
        CK(cudaMemcpy(dP, P.data(), total * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dXa, X.data(), X.size() * 4, cudaMemcpyHostToDevice));
        void* twin = b200gemm_bf16_twin_range(dP, (long long)total);
        if (!twin) {
            printf("{\"case\": \"range_twin\", \"twins\": \"off\", \"ok\": true}\n");
        } else {
            std::vector<unsigned short> T(total);
            for (size_t i = 0; i < total; ++i) {
                const float f = 2.0f * P[i];
                unsigned int u;
                memcpy(&u, &f, 4);
                T[i] = (unsigned short)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);  // round to nearest even
            }
            CK(cudaMemcpy(twin, T.data(), total * 2, cudaMemcpyHostToDevice));
            double rel_at[2];
            for (int which = 0; which < 2; ++which) {
                // offset 128: read from the twin (factor 2); offset 133: not a multiple of 128, converted as usual (factor 1)
                const size_t off = which == 0 ? lead : lead + 5;
                const double factor = which == 0 ? 2.0 : 1.0;
                b200gemm_forget_staged();
                matmul_cublaslt(lt, dXa, dP + off, dYa, R, C2, C1, CUBLASLT_EPILOGUE_DEFAULT, nullptr, workspace, ws_bytes, false, false,
                                1.0f, 0.0f, 0);
                CK(cudaDeviceSynchronize());
                CK(cudaMemcpy(Y.data(), dYa, Y.size() * 4, cudaMemcpyDeviceToHost));
                double max_rel = 0.0;
                for (int s_ = 0; s_ < 2000; ++s_) {
                    const int i = int((next_uniform() * 0.5f + 0.5f) * R) % R, j = int((next_uniform() * 0.5f + 0.5f) * C2) % C2;
                    double acc = 0.0, scale = 0.0;
                    for (int k = 0; k < C1; ++k) {
                        const double p = double(X[size_t(i) * C1 + k]) * P[off + size_t(k) * C2 + j];
                        acc += p, scale += fabs(p);
                    }
                    const double rel = fabs(double(Y[size_t(i) * C2 + j]) - factor * acc) / (factor * scale / sqrt(double(C1)) + 1.0);
                    if (!(rel <= max_rel)) max_rel = rel;
                }
                rel_at[which] = max_rel;
            }
            const bool ok = rel_at[0] <= tol && rel_at[1] <= tol;
            all_ok = all_ok && ok;
            printf("{\"case\": \"range_twin\", \"twins\": \"on\", \"max_rel_from_twin\": %.3e, \"max_rel_converted\": %.3e, \"ok\": %s}\n",
                   rel_at[0], rel_at[1], ok ? "true" : "false");
            b200gemm_release_twins();
        }
        cudaFree(dP); cudaFree(dXa); cudaFree(dYa);
    }
    const int fault = b200gemm_check_device_fault();
    printf("{\"tcgen05_kernel_launches\": %lld, \"device_fault\": %d}\n", b200gemm_tc_launches(), fault);
    return (all_ok && fault == 0) ? 0 : 1;
}
