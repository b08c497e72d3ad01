// Interface of the hand-written tcgen05 GEMM (gemm_tc.cu) towards the GEMM drop-in (matmul_dropin.cu).
#pragma once

#include <cuda_runtime.h>

namespace b200gemm {

// C (M x N, FP32, leading dimension ldc in elements, any alignment) = alpha * op(A) * op(B) on `stream`.
// A: BF16, stored (trans_a ? K x M : M x K) with `rows_a` stored rows and leading dimension lda; B: BF16, stored
// (trans_b ? N x K : K x N), `rows_b` rows, leading dimension ldb. Base addresses 16-byte aligned, leading dimensions
// multiples of 8; everything stored beyond the M / N / K extents must be zero. Returns false when the kernel cannot
// run here (not an sm_100 device, tensor-map encoding failed, launch failed): the caller takes the library path.
bool tc_gemm_bf16(const void* A, int rows_a, int lda, bool trans_a, const void* B, int rows_b, int ldb, bool trans_b, float* C,
                  long long ldc, int M, int N, int K, float alpha, cudaStream_t stream);

// Number of 256 x 256 output tiles of an M x N product (the kernel runs one persistent CTA per SM over them).
int tc_gemm_tiles(int M, int N);

// Launches of the kernel by this process so far.
long long tc_gemm_launches();

// Record of a bounded wait that ran out inside the kernel since the last call (0 = none); clears it.
unsigned int tc_gemm_take_fault();

}  // namespace b200gemm
