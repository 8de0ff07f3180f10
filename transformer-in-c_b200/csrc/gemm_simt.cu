// FP32 FMA matrix product for shapes the tensor-core path does not take
// (tiny or oddly sized extents such as K = 4, N = 11) and as the exact-FP32
// path for very small models.  C[M,N] (+)= A[M,K] * B[K,N], where A and B are
// addressed through element strides so that the forward product, the input
// gradient (B read transposed) and the weight gradient (A read transposed)
// all use the same kernel (reference src/ops.c:123-132 and :153-163).
//
// 64x64 output tile per block, 16-deep K steps through shared memory, 4x4
// register micro-tile per thread.  When the reduction is long and the output
// small (weight gradients: K = batch*tokens) the reduction is split across
// blockIdx.z and partial tiles are combined with atomic adds; that is only
// done in accumulate mode, where C already holds the value to add to.
#include "kernels.h"
#include "device_util.cuh"

namespace vitb200 {
namespace {

constexpr int kTileM = 64;
constexpr int kTileN = 64;
constexpr int kTileK = 16;
constexpr int kPitch = kTileM + 4;

__global__ void __launch_bounds__(256)
gemm_simt_kernel(GemmOperands op, int k_per_split) {
    grid_dependency_wait();
    grid_dependency_release();
    __shared__ __align__(16) float a_tile[kTileK][kPitch];
    __shared__ __align__(16) float b_tile[kTileK][kPitch];
    const int tid = threadIdx.x;
    const int tx = tid % 16;
    const int ty = tid / 16;
    const int m0 = blockIdx.x * kTileM;
    const int n0 = blockIdx.y * kTileN;
    const int k_begin = blockIdx.z * k_per_split;
    const int k_end = min(op.k, k_begin + k_per_split);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.0f;
        }
    }
    // Thread-to-element maps chosen so the unit-stride axis of each operand
    // runs along consecutive threads.
    const bool a_k_contiguous = op.a_col == 1;
    const bool b_n_contiguous = op.b_col == 1;
    for (int k0 = k_begin; k0 < k_end; k0 += kTileK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int mm, kk;
            if (a_k_contiguous) {
                kk = tid % kTileK;
                mm = tid / kTileK + 16 * i;
            } else {
                mm = tid % kTileM;
                kk = tid / kTileM + 4 * i;
            }
            const int m = m0 + mm, k = k0 + kk;
            a_tile[kk][mm] = (m < op.m && k < k_end)
                ? op.a[(long long)m * op.a_row + (long long)k * op.a_col]
                : 0.0f;
            int nn, kb;
            if (b_n_contiguous) {
                nn = tid % kTileN;
                kb = tid / kTileN + 4 * i;
            } else {
                kb = tid % kTileK;
                nn = tid / kTileK + 16 * i;
            }
            const int n = n0 + nn, k2 = k0 + kb;
            b_tile[kb][nn] = (n < op.n && k2 < k_end)
                ? op.b[(long long)k2 * op.b_row + (long long)n * op.b_col]
                : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTileK; ++kk) {
            const float4 a = *reinterpret_cast<const float4 *>(&a_tile[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4 *>(&b_tile[kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] += av[i] * bv[j];
                }
            }
        }
        __syncthreads();
    }
    const bool atomic = gridDim.z > 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= op.m) {
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= op.n) {
                continue;
            }
            float *c = op.c + (long long)m * op.c_row + n;
            if (atomic) {
                atomicAdd(c, acc[i][j]);
            } else if (op.accumulate) {
                *c += acc[i][j];
            } else {
                *c = acc[i][j];
            }
        }
    }
}

}  // namespace

unsigned long long g_fma_products = 0;

void launch_gemm_simt(const GemmOperands &operands, cudaStream_t stream) {
    ++g_fma_products;
    const unsigned grid_x = (operands.m + kTileM - 1) / kTileM;
    const unsigned grid_y = (operands.n + kTileN - 1) / kTileN;
    unsigned splits = 1;
    if (operands.accumulate) {
        const unsigned tiles = grid_x * grid_y;
        const unsigned wanted = (2 * kSmCount + tiles - 1) / tiles;
        const unsigned most = (operands.k + 8 * kTileK - 1) / (8 * kTileK);
        splits = wanted < most ? wanted : most;
        if (splits < 1) {
            splits = 1;
        }
    }
    int k_per_split = (operands.k + splits - 1) / splits;
    k_per_split = (k_per_split + kTileK - 1) / kTileK * kTileK;
    splits = (operands.k + k_per_split - 1) / k_per_split;
    launch_chained(gemm_simt_kernel, dim3(grid_x, grid_y, splits), 256, 0,
                   stream, operands, k_per_split);
    ++g_kernel_launches;
}

}  // namespace vitb200
