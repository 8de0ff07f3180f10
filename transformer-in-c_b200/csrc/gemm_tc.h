// tcgen05 / TMA matrix product (gemm_tc.cu).
#pragma once

#include <cuda_runtime.h>

namespace vitb200 {

// D[m,n] (+)= A * B over a reduction of length k, FP32 row-major storage.
//   a_mn_major = false: A is stored [m rows][k contiguous], pitch lda
//   a_mn_major = true : A is stored [k rows][m contiguous], pitch lda
//   b_mn_major = false: B is stored [n rows][k contiguous], pitch ldb
//   b_mn_major = true : B is stored [k rows][n contiguous], pitch ldb
// accumulate adds into D (atomically, so the reduction may be split).
struct TcGemm {
    const float *a;
    const float *b;
    float *d;
    const float *bias;  // nullable; added per output column (not with accumulate)
    int m, n, k;
    long long lda, ldb, ldd;
    bool a_mn_major, b_mn_major, accumulate;
    // Optional second output of the same shape (not with accumulate):
    //   residual == nullptr:  d2 = gelu(d)          (d = A*B + bias)
    //   residual != nullptr:  d2 = d + residual
    float *d2 = nullptr;
    long long ldd2 = 0;
    const float *residual = nullptr;
    long long ld_residual = 0;
    // Optional (not with accumulate, bias or d2): d = (A*B) * gelu'(gelu_input)
    // element by element, gelu_input of the output's shape.  With
    // column_partials, [kGemmPartialRows][n] floats, the kernel also leaves
    // per-CTA column sums of d there (the launcher clears them first).
    const float *gelu_input = nullptr;
    long long ld_gelu_input = 0;
    float *column_partials = nullptr;
};

// Upper bound of the persistent grid: two CTAs on each of 148 SMs.
constexpr int kGemmPartialRows = 296;

bool gemm_tc_supported(const TcGemm &gemm);
int launch_gemm_tc(const TcGemm &gemm, cudaStream_t stream);
// 0, or the code of the first bounded wait that expired inside the kernel.
int gemm_tc_status();
// Products launched on the tensor cores since the library was loaded, and
// how many of them used the 128 x 256 tile.
extern unsigned long long g_tc_products, g_tc_wide_products;
// Device address of that status word, shared by every kernel of the library
// that waits on an mbarrier (codes 1..15: matrix product, 16..: attention);
// nullptr when it could not be mapped.
int *tc_status_device_pointer();

}  // namespace vitb200
