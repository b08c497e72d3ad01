// Drop-in declarations of the LayerNorm launchers of the reference model (include/kernels/layernorm.cuh:9-36 of
// sarimahsan/transformer-cuda; called from src/model.cu:279,358,405 and :479,566,687): identical names, parameter order,
// types and default arguments, so src/model.cu and tests/test_kernels.cu compile against this header unchanged. The
// definitions are in transformer-cuda_b200/norm/layernorm_dropin.cu (libb200norm.a).
//
//   forward : out = (x - mean) * rstd * gamma + beta over rows of C; mean and rstd = rsqrt(var + eps) are saved (N each).
//             gamma / beta may be NULL (1 / 0).
//   backward: dx = rstd * (dout*gamma - sum(dout*gamma)/C - xhat * sum(dout*gamma*(x-mean)) * rstd / C) [+ residual_add],
//             stored, or added to dx when `accumulate`; dgamma += sum_rows dout * xhat, dbeta += sum_rows dout (both are
//             ADDED to what the buffers hold, as in the reference; either may be NULL).
// Shapes: x, out, dout, dx, residual_add (N, C); gamma, beta, dgamma, dbeta (C); mean, rstd (N). Asynchronous on `stream`.
#pragma once

#include <cuda_runtime.h>

void layernorm_forward(const float* x, const float* gamma, const float* beta, float* out, float* mean, float* rstd, int N,
                       int C, float eps, cudaStream_t stream = 0);

void layernorm_backward(const float* dout, const float* x, const float* gamma, const float* mean, const float* rstd,
                        float* dx, float* dgamma, float* dbeta, int N, int C, const float* residual_add = nullptr,
                        bool accumulate = false, cudaStream_t stream = 0);

// Extension (not in the reference's header): a host callback run after every layernorm_backward launch, with the number
// of layernorm_backward calls since the last reset (1, 2, ...), the stream and `user`. A data-parallel trainer uses it to
// start the all-reduce of the gradients that are final at that point of the model's backward pass
// (transformer-cuda_b200/harness/gpt_step_dp.cu). NULL removes the hook.
extern "C" void b200norm_set_backward_hook(void (*fn)(int call_index, cudaStream_t stream, void* user), void* user);
extern "C" void b200norm_reset_backward_count(void);
