// Dense products of the training step, row-major FP32 storage:
//   forward   Y[M,N]  = X[M,K] W[K,N]
//   backward  dX[M,K] += dY[M,N] W^T ;  dW[K,N] += X^T dY
// (reference src/ops.c:107-165).  The dispatcher picks the tensor-core kernel
// when the shape qualifies and the FP32 FMA kernel otherwise.
#pragma once

#include <cuda_runtime.h>

namespace vitb200 {

// precision: one of the VITB200_PRECISION_* selectors.  Returns 0, or -1 when
// the requested precision cannot serve the shape.
int gemm_forward(const float *x, const float *w, float *y, int m, int k, int n,
                 int precision, cudaStream_t stream);
// dx_add = false stores dX instead of adding to it (dX known to be zero).
int gemm_backward(const float *x, const float *w, const float *dy, float *dx,
                  float *dw, int m, int k, int n, int precision, bool dx_add,
                  cudaStream_t stream);

// The same policy for other tensor-core capable ops (attention): true when an
// op of `multiply_adds` should use TF32 under `precision`.
bool prefer_tensor_cores(int precision, double multiply_adds);

// Overrides what VITB200_PRECISION_AUTO means (and the VITB200_GEMM
// environment variable); -1 restores the default policy.
void gemm_set_default_precision(int precision);

}  // namespace vitb200
