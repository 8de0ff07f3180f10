// Dense products of the training step, row-major FP32 storage:
//   forward   Y[M,N]  = X[M,K] W[K,N]
//   backward  dX[M,K] += dY[M,N] W^T ;  dW[K,N] += X^T dY
// (reference src/ops.c:107-165).  The dispatcher picks the tensor-core kernel
// when the shape qualifies and the FP32 FMA kernel otherwise.
#pragma once

#include <cuda_runtime.h>

namespace vitb200 {

// What may ride on the forward product's epilogue.  All pointers optional:
//   bias           y += bias[col]                      (reference ops_bias_add)
//   gelu_out       gelu_out = gelu(y)                  (ops_gelu on y)
//   residual(+out) residual_out = residual + y         (ops_residual)
// gelu_out and residual_out exclude each other.
struct GemmEpilogue {
    const float *bias = nullptr;
    float *gelu_out = nullptr;
    const float *residual = nullptr;
    float *residual_out = nullptr;
};

// precision: one of the VITB200_PRECISION_* selectors.  Returns 0, or -1 when
// the requested precision cannot serve the shape.
int gemm_forward(const float *x, const float *w, float *y, int m, int k, int n,
                 int precision, cudaStream_t stream);
// dx_add = false stores dX instead of adding to it (dX known to be zero).
// Forward product with the epilogue above; falls back to separate kernels
// when the tensor-core path does not take the shape.
int gemm_forward_fused(const float *x, const float *w, float *y, int m, int k,
                       int n, const GemmEpilogue &epilogue, int precision,
                       cudaStream_t stream);
int gemm_backward(const float *x, const float *w, const float *dy, float *dx,
                  float *dw, int m, int k, int n, int precision, bool dx_add,
                  cudaStream_t stream);
// Its two halves.
int gemm_backward_input(const float *w, const float *dy, float *dx, int m,
                        int k, int n, int precision, bool dx_add,
                        cudaStream_t stream);
int gemm_backward_weights(const float *x, const float *dy, float *dw, int m,
                          int k, int n, int precision, cudaStream_t stream);
// The input half followed by a GELU's backward pass, in one kernel:
//   d_gelu_input[m,k] = (dY[m,n] W^T) * gelu'(gelu_input[m,k])
// for a layer whose input X = gelu(gelu_input) (reference src/ops.c:107-165
// then 965-1000, with the intermediate dX never stored).  column_partials,
// optional, receives kGemmPartialRows rows of k partial column sums of the
// result.  Tensor-core path only: -1, with nothing done, when the shape or the
// precision policy does not put the product there (`..._supported` tells in
// advance).
bool gemm_backward_input_gelu_supported(const float *w, const float *dy,
                                        const float *gelu_input,
                                        float *d_gelu_input, int m, int k,
                                        int n, int precision);
int gemm_backward_input_gelu(const float *w, const float *dy,
                             const float *gelu_input, float *d_gelu_input,
                             float *column_partials, int m, int k, int n,
                             int precision, cudaStream_t stream);

// The same policy for other tensor-core capable ops (attention): true when an
// op of `multiply_adds` should use TF32 under `precision`.
bool prefer_tensor_cores(int precision, double multiply_adds);

// The precision VITB200_PRECISION_AUTO currently resolves to (AUTO itself
// when no override is active).
int gemm_default_precision();

// Overrides what VITB200_PRECISION_AUTO means (and the VITB200_GEMM
// environment variable); -1 restores the default policy.
void gemm_set_default_precision(int precision);
// Products launched since the library was loaded: on the tensor cores, of
// those with the 128 x 256 tile, and on the FP32 FMA kernel.
void gemm_path_counters(unsigned long long *tensor_core,
                        unsigned long long *wide_tile, unsigned long long *fma);

}  // namespace vitb200
