#include "gemm.h"
#include "kernels.h"
#include "../../include/vitb200.h"

namespace vitb200 {

int gemm_forward(const float *x, const float *w, float *y, int m, int k, int n,
                 int precision, cudaStream_t stream) {
    if (precision == VITB200_PRECISION_TF32) {
        return -1;
    }
    GemmOperands op;
    op.a = x;  op.a_row = k; op.a_col = 1;
    op.b = w;  op.b_row = n; op.b_col = 1;
    op.c = y;  op.c_row = n;
    op.m = m;  op.n = n;     op.k = k;
    op.accumulate = 0;
    launch_gemm_simt(op, stream);
    return 0;
}

int gemm_backward(const float *x, const float *w, const float *dy, float *dx,
                  float *dw, int m, int k, int n, int precision,
                  cudaStream_t stream) {
    if (precision == VITB200_PRECISION_TF32) {
        return -1;
    }
    // dX[M,K] += dY[M,N] * W^T : B(n,k) = w[k*n_cols + n].
    GemmOperands dx_op;
    dx_op.a = dy; dx_op.a_row = n; dx_op.a_col = 1;
    dx_op.b = w;  dx_op.b_row = 1; dx_op.b_col = n;
    dx_op.c = dx; dx_op.c_row = k;
    dx_op.m = m;  dx_op.n = k;     dx_op.k = n;
    dx_op.accumulate = 1;
    launch_gemm_simt(dx_op, stream);
    // dW[K,N] += X^T * dY : A(kk,m) = x[m*k_cols + kk].
    GemmOperands dw_op;
    dw_op.a = x;  dw_op.a_row = 1; dw_op.a_col = k;
    dw_op.b = dy; dw_op.b_row = n; dw_op.b_col = 1;
    dw_op.c = dw; dw_op.c_row = n;
    dw_op.m = k;  dw_op.n = n;     dw_op.k = m;
    dw_op.accumulate = 1;
    launch_gemm_simt(dw_op, stream);
    return 0;
}

}  // namespace vitb200
