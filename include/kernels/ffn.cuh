// Drop-in declarations of the GELU launchers of the reference model (include/kernels/ffn.cuh:7-33 of
// sarimahsan/transformer-cuda; called from src/model.cu:379 and :532): identical names, parameter order, types and default
// arguments. The definitions are in transformer-cuda_b200/ffn/gelu_dropin.cu (libb200ffn.a).
//
//   gelu(x) = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))                     (the tanh form, as the reference)
//   gelu_forward:          y = gelu(x)                      N elements
//   add_bias_gelu_forward: y = gelu(x + bias[col])          M x N, bias of length N
//   gelu_backward:         dx = dy * gelu'(x)               N elements
// The arithmetic is the reference's, expression by expression; what the drop-in adds is a BF16 twin of y and of dx,
// written in the same pass for the GEMMs that read them next, when the GEMM drop-in is linked in and B200GEMM_TWINS=1.
#pragma once

#include <cuda_runtime.h>

void gelu_forward(const float* x, float* y, int N, cudaStream_t stream = 0);

void add_bias_gelu_forward(const float* x, const float* bias, float* y, int M, int N, cudaStream_t stream = 0);

void gelu_backward(const float* dy, const float* x, float* dx, int N, cudaStream_t stream = 0);
