// TEST INFRASTRUCTURE. Checks the AdamW drop-in (transformer-cuda_b200/optim/adamw_dropin.cu, linked here) against a
// CPU restatement in double precision of the reference's optimizer (src/optimizer.cu of sarimahsan/transformer-cuda):
//   fused_step   :225-249  norm = sqrt(sum g^2); g *= max_norm / norm if norm > max_norm and norm > 1e-6;
//                          m = b1 m + (1 - b1) g; v = b2 v + (1 - b2) g^2; p -= lr (m^ / (sqrt(v^) + eps) + wd p); g = 0
//   clip_grad_norm + step + zero_grad  :193-223  the same update as three separate calls
// over a parameter count that is not a multiple of 4, for several steps with fresh gradients, with and without the
// clip taking effect. Prints one JSON line with the largest deviations; exits non-zero above the tolerances.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "optimizer.h"

namespace {
struct HostAdam {
    std::vector<double> p, m, v;
    double b1, b2, eps, wd;
    int t = 0;
    void step(const std::vector<float>& g_in, double lr, double max_norm, bool clip) {
        ++t;
        double ss = 0;
        for (float g : g_in) ss += (double)g * g;
        const double norm = std::sqrt(ss);
        const double scale = (clip && norm > max_norm && norm > 1e-6) ? max_norm / norm : 1.0;
        const double c1 = 1 - std::pow(b1, t), c2 = 1 - std::pow(b2, t);
        for (size_t i = 0; i < p.size(); ++i) {
            const double g = g_in[i] * scale;
            m[i] = b1 * m[i] + (1 - b1) * g;
            v[i] = b2 * v[i] + (1 - b2) * g * g;
            p[i] -= lr * ((m[i] / c1) / (std::sqrt(v[i] / c2) + eps) + wd * p[i]);
        }
    }
};
unsigned long long g_state = 0x9e3779b97f4a7c15ull;
float next_uniform() {  // xorshift64*, in (-1, 1)
    g_state ^= g_state >> 12, g_state ^= g_state << 25, g_state ^= g_state >> 27;
    return (float)((double)((g_state * 2685821657736338717ull) >> 11) / 9007199254740992.0 * 2.0 - 1.0);
}
}  // namespace

int main() {
    const size_t n = 1000003;
    TransformerConfig cfg;
    cfg.beta1 = 0.9f, cfg.beta2 = 0.95f, cfg.weight_decay = 0.1f, cfg.adam_eps = 1e-8f;
    const float lr = 3e-4f, max_norm = 1.0f;
    std::vector<float> p0(n), g(n);
    for (auto& x : p0) x = 0.02f * next_uniform();
    float *d_p, *d_g;
    cudaMalloc(&d_p, n * sizeof(float));
    cudaMalloc(&d_g, n * sizeof(float));
    cudaMemcpy(d_p, p0.data(), n * sizeof(float), cudaMemcpyHostToDevice);
    HostAdam host{std::vector<double>(p0.begin(), p0.end()), std::vector<double>(n, 0.0), std::vector<double>(n, 0.0),
                  (double)cfg.beta1, (double)cfg.beta2, (double)cfg.adam_eps, (double)cfg.weight_decay};
    double worst_p = 0, worst_g = 0;
    {
        AdamW opt(d_p, d_g, n, cfg);
        // gradient amplitudes: norm far above max_norm (clipped), far below (not clipped), then again above
        const float amp[5] = {0.05f, 1e-5f, 0.01f, 2e-4f, 0.03f};
        for (int s = 0; s < 5; ++s) {
            for (auto& x : g) x = amp[s] * next_uniform();
            cudaMemcpy(d_g, g.data(), n * sizeof(float), cudaMemcpyHostToDevice);
            if (s < 3) {
                opt.fused_step(lr, max_norm, 0);
            } else {  // the three-call form used by src/main.cu:75-77
                opt.clip_grad_norm(max_norm, 0);
                opt.step(lr, 0);
                opt.zero_grad(0);
            }
            host.step(g, lr, max_norm, true);
            std::vector<float> p(n), gz(n);
            cudaMemcpy(p.data(), d_p, n * sizeof(float), cudaMemcpyDeviceToHost);
            cudaMemcpy(gz.data(), d_g, n * sizeof(float), cudaMemcpyDeviceToHost);
            for (size_t i = 0; i < n; ++i) {
                worst_p = std::fmax(worst_p, std::fabs((double)p[i] - host.p[i]));
                worst_g = std::fmax(worst_g, std::fabs((double)gz[i]));
            }
        }
        if (opt.get_step_count() != 5) worst_p = 1.0;
    }
    const cudaError_t e = cudaDeviceSynchronize();
    const bool ok = e == cudaSuccess && worst_p <= 2e-6 && worst_g == 0.0;
    printf("{\"params\": %zu, \"steps\": 5, \"max_abs_param_error\": %.3e, \"max_abs_leftover_grad\": %.3e, \"ok\": %s}\n", n,
           worst_p, worst_g, ok ? "true" : "false");
    cudaFree(d_p);
    cudaFree(d_g);
    return ok ? 0 : 1;
}
