/* C ABI of the fused softmax cross-entropy (loss + d_logits) for sm_100a: libb200loss.so / libb200loss.a.
 *
 * Replaces cross_entropy_forward_backward of sarimahsan/transformer-cuda (include/kernels/loss.cuh:8-15,
 * src/kernels/loss.cu:24-125), the first call of the model's backward pass (src/model.cu:449). The C++
 * declaration with the reference's exact signature is include/kernels/loss.cuh; the entry points below are
 * the same launch with plain pointers and sizes, for bindings from other languages and for the parity tests.
 *
 * All pointers are device pointers on the current device unless stated otherwise; `stream` is a cudaStream_t
 * passed as void*. Logits and d_logits are FP32, row-major (rows x V), rows = B * T; targets are int32.
 * Return value: 0 on success, a negative B200LOSS_ERR_* otherwise; b200loss_last_error() describes the failure. */
#ifndef B200LOSS_H
#define B200LOSS_H

#ifdef __cplusplus
extern "C" {
#endif

#define B200LOSS_OK 0
#define B200LOSS_ERR_ARG (-1)   /* NULL pointer, non-positive size */
#define B200LOSS_ERR_CUDA (-2)  /* a CUDA runtime call failed */
#define B200LOSS_ERR_WAIT (-3)  /* a bounded wait inside an earlier launch ran out (see check_device_fault) */

/* d_logits[i, v] = (softmax(logits[i, :])[v] - (v == targets[i])) / rows, and, when `device_loss` is not NULL,
 * *device_loss = mean_i (logsumexp(logits[i, :]) - logits[i, targets[i]]). Asynchronous on `stream`; nothing is
 * copied to the host. d_logits may alias logits (each row is resident on chip before it is written).
 * The first call on a device, and the first call with more rows than any before it, allocates the row-loss scratch
 * (rows * 4 bytes) with cudaMalloc and therefore must not happen inside a stream capture. */
int b200loss_cross_entropy(const float* logits, const int* targets, float* d_logits, float* device_loss, int B, int T,
                           int V, void* stream);

/* Which kernel a call with these arguments takes: 0 = one pass over HBM, the row held in shared memory
 * (16-byte aligned buffers, 8 <= V <= b200loss_max_resident_vocab()), 1 = streaming kernel, two reads of the row. */
int b200loss_kernel_path(const float* logits, const float* d_logits, int V);
int b200loss_max_resident_vocab(void);

/* Waits for the device and returns 0 if no bounded wait has run out since the last call, else B200LOSS_ERR_WAIT
 * (and clears the record). */
int b200loss_check_device_fault(void);

/* Frees the per-device scratch. */
void b200loss_release(void);

/* Text of the last failure on the calling thread ("" if none). */
const char* b200loss_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
