// Drop-in declaration of the loss launcher the reference model calls at the top of its backward pass
// (include/kernels/loss.cuh:8-15 of sarimahsan/transformer-cuda, called from src/model.cu:449): identical name,
// parameter order, types and default argument, so src/model.cu and tests/test_kernels.cu compile against this
// header unchanged. The definition is in transformer-cuda_b200/loss/cross_entropy.cu (libb200loss.a / .so).
//
//   dlogits[i, v] = (softmax(logits[i, :])[v] - (v == targets[i])) / (B * T)
//   *host_loss    = mean over the B * T rows of  logsumexp(logits[i, :]) - logits[i, targets[i]]
//
// As in the reference, a non-NULL `host_loss` makes the call wait for the stream (the value is valid on return)
// and a NULL one skips the loss and never waits. What differs is the work behind it: each row is read from HBM once
// (the reference reads it three times), the row losses are summed on the device in a fixed order, and four bytes
// cross to the host instead of B * T floats. Targets must lie in [0, V); a target outside contributes no indicator
// and a row loss of logsumexp alone (the reference reads out of bounds there).
#pragma once

#include <cuda_runtime.h>

void cross_entropy_forward_backward(const float* logits, const int* targets, float* dlogits, float* host_loss, int B,
                                    int T, int V, cudaStream_t stream = 0);

// Extension for callers that keep the loss on the device: same computation, the mean loss is written to
// `device_loss` (one float, may be NULL) by the kernel itself, and the call never waits for the stream.
void cross_entropy_forward_backward_device(const float* logits, const int* targets, float* dlogits,
                                           float* device_loss, int B, int T, int V, cudaStream_t stream = 0);
