// TEST INFRASTRUCTURE. Checks the LayerNorm drop-in (transformer-cuda_b200/norm/layernorm_dropin.cu, linked here as
// libb200norm.a) against a double-precision host restatement of the reference's kernels (src/kernels/layernorm.cu of
// sarimahsan/transformer-cuda):
//   forward  :52-94    mean = sum x / C; rstd = 1 / sqrt(sum (x - mean)^2 / C + eps); out = (x - mean) rstd gamma + beta
//   backward :176-207  s1 = sum dout gamma; s2 = sum dout gamma (x - mean);
//                      dx = rstd (dout gamma - s1 / C - xhat s2 rstd / C) [+ residual] [+ old dx when accumulate]
//            :231-246  dgamma += sum_rows dout xhat; dbeta += sum_rows dout   (added to what the buffers hold)
// over shapes that take the register path (C = 128 k) and the generic path, with and without gamma / beta, residual
// and accumulate. Prints one JSON line per case; exits non-zero if any case exceeds its tolerance.
#include <cmath>
#include <cstdio>
#include <vector>

#include "kernels/layernorm.cuh"

namespace {
unsigned long long g_state = 0x243f6a8885a308d3ull;
float next_uniform() {
    g_state ^= g_state >> 12, g_state ^= g_state << 25, g_state ^= g_state >> 27;
    return (float)((double)((g_state * 2685821657736338717ull) >> 11) / 9007199254740992.0 * 2.0 - 1.0);
}
template <class T>
T* upload(const std::vector<T>& h) {
    T* d = nullptr;
    cudaMalloc(&d, h.size() * sizeof(T));
    cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}
std::vector<float> download(const float* d, size_t n) {
    std::vector<float> h(n);
    cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost);
    return h;
}
double max_err(const std::vector<float>& got, const std::vector<double>& want, double floor_scale) {
    double worst = 0;
    for (size_t i = 0; i < got.size(); ++i)
        worst = std::fmax(worst, std::fabs((double)got[i] - want[i]) / std::fmax(floor_scale, std::fabs(want[i])));
    return worst;
}

bool run_case(int N, int C, bool affine, bool residual, bool accumulate) {
    const float eps = 1e-5f;
    const size_t n = (size_t)N * C;
    std::vector<float> x(n), dy(n), res(n), dx0(n), gamma(C), beta(C), dg0(C), db0(C);
    for (auto& v : x) v = 2.0f * next_uniform() + 0.5f;
    for (auto& v : dy) v = next_uniform();
    for (auto& v : res) v = next_uniform();
    for (auto& v : dx0) v = next_uniform();
    for (int c = 0; c < C; ++c) gamma[c] = 1.0f + 0.5f * next_uniform(), beta[c] = 0.2f * next_uniform(), dg0[c] = next_uniform(), db0[c] = next_uniform();
    float *d_x = upload(x), *d_dy = upload(dy), *d_res = upload(res), *d_dx = upload(dx0), *d_g = upload(gamma), *d_b = upload(beta);
    float *d_dg = upload(dg0), *d_db = upload(db0), *d_out, *d_mean, *d_rstd;
    cudaMalloc(&d_out, n * sizeof(float));
    cudaMalloc(&d_mean, N * sizeof(float));
    cudaMalloc(&d_rstd, N * sizeof(float));
    layernorm_forward(d_x, affine ? d_g : nullptr, affine ? d_b : nullptr, d_out, d_mean, d_rstd, N, C, eps);
    layernorm_backward(d_dy, d_x, affine ? d_g : nullptr, d_mean, d_rstd, d_dx, d_dg, d_db, N, C, residual ? d_res : nullptr, accumulate);
    const bool launched = cudaDeviceSynchronize() == cudaSuccess;

    std::vector<double> out(n), dx(n), mean(N), rstd(N), dg(dg0.begin(), dg0.end()), db(db0.begin(), db0.end());
    for (int r = 0; r < N; ++r) {
        const float* xr = &x[(size_t)r * C];
        double s = 0, q = 0, s1 = 0, s2 = 0;
        for (int c = 0; c < C; ++c) s += xr[c];
        const double m = s / C;
        for (int c = 0; c < C; ++c) q += (xr[c] - m) * (xr[c] - m);
        const double rs = 1.0 / std::sqrt(q / C + eps);
        mean[r] = m, rstd[r] = rs;
        for (int c = 0; c < C; ++c) {
            const double g = affine ? gamma[c] : 1.0, b = affine ? beta[c] : 0.0, d = dy[(size_t)r * C + c];
            out[(size_t)r * C + c] = (xr[c] - m) * rs * g + b;
            s1 += d * g, s2 += d * g * (xr[c] - m);
            dg[c] += d * (xr[c] - m) * rs, db[c] += d;
        }
        for (int c = 0; c < C; ++c) {
            const double g = affine ? gamma[c] : 1.0, d = dy[(size_t)r * C + c], xh = (xr[c] - m) * rs;
            double v = rs * (d * g - s1 / C - xh * s2 * rs / C);
            if (residual) v += res[(size_t)r * C + c];
            if (accumulate) v += dx0[(size_t)r * C + c];
            dx[(size_t)r * C + c] = v;
        }
    }
    const double e_out = max_err(download(d_out, n), out, 1.0), e_dx = max_err(download(d_dx, n), dx, 1.0);
    const double e_mean = max_err(download(d_mean, N), mean, 1.0), e_rstd = max_err(download(d_rstd, N), rstd, 1.0);
    const double col_scale = std::sqrt((double)N);  // column sums of N terms of order one
    const double e_dg = max_err(download(d_dg, C), dg, col_scale), e_db = max_err(download(d_db, C), db, col_scale);
    const bool ok = launched && e_out <= 1e-5 && e_dx <= 2e-5 && e_mean <= 1e-6 && e_rstd <= 1e-5 && e_dg <= 1e-5 && e_db <= 1e-5;
    printf("{\"N\": %d, \"C\": %d, \"affine\": %d, \"residual\": %d, \"accumulate\": %d, \"out\": %.2e, \"dx\": %.2e, \"mean\": %.2e, "
           "\"rstd\": %.2e, \"dgamma\": %.2e, \"dbeta\": %.2e, \"ok\": %s}\n",
           N, C, affine, residual, accumulate, e_out, e_dx, e_mean, e_rstd, e_dg, e_db, ok ? "true" : "false");
    for (float* p : {d_x, d_dy, d_res, d_dx, d_g, d_b, d_dg, d_db, d_out, d_mean, d_rstd}) cudaFree(p);
    return ok;
}
}  // namespace

int main() {
    bool ok = true;
    ok &= run_case(4099, 768, true, true, false);    // the model's shape class: register path, persistent grid, ragged last CTA
    ok &= run_case(1000, 768, true, false, true);
    ok &= run_case(333, 1024, false, true, true);    // widest register path, no gamma / beta
    ok &= run_case(77, 128, true, false, false);     // narrowest register path
    ok &= run_case(64, 64, true, true, false);       // generic path (the parity-audit model has C = 64)
    ok &= run_case(50, 100, false, false, true);
    ok &= run_case(17, 1300, true, true, true);      // generic path beyond the register limit
    return ok ? 0 : 1;
}
