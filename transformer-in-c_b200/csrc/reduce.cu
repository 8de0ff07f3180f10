// Column sums of a row-major matrix: out[c] += sum_r in[r*ld + c].
// Used for bias gradients and for the positional / CLS gradients.
//
// A block owns a strip of columns (32 threads wide, each thread 1 or 4
// adjacent columns) and a slice of the rows; its 32 row lanes walk the slice
// with fully coalesced 128- or 512-byte row segments, fold through shared
// memory, and one lane per column adds the block's partial with a single
// atomic.  Row slices are sized so the whole grid is about two waves.
#include "kernels.h"
#include "device_util.cuh"

namespace vitb200 {
namespace {

constexpr int kLanesX = 32;
constexpr int kLanesY = 32;

template <int V>
__global__ void __launch_bounds__(kLanesX *kLanesY)
column_sums_kernel(const float *__restrict__ in, float *__restrict__ out,
                   size_t rows, size_t cols, size_t ld, size_t rows_per_block) {
    grid_dependency_wait();
    grid_dependency_release();
    __shared__ float partial[kLanesY][kLanesX * V + 1];
    const size_t col = (size_t(blockIdx.x) * kLanesX + threadIdx.x) * V;
    const size_t row_begin = size_t(blockIdx.y) * rows_per_block;
    const size_t row_end = min(rows, row_begin + rows_per_block);
    float sum[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        sum[j] = 0.0f;
    }
    if (col < cols) {
        for (size_t row = row_begin + threadIdx.y; row < row_end;
             row += kLanesY) {
            const float *p = in + row * ld + col;
            if (V == 4) {
                const float4 v = __ldcs(reinterpret_cast<const float4 *>(p));
                sum[0] += v.x;
                sum[V > 1 ? 1 : 0] += v.y;
                sum[V > 2 ? 2 : 0] += v.z;
                sum[V > 3 ? 3 : 0] += v.w;
            } else {
                sum[0] += __ldcs(p);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
        partial[threadIdx.y][threadIdx.x * V + j] = sum[j];
    }
    __syncthreads();
    // Fold the 32 row lanes: thread (x, y) reduces column slot y*?.. simple
    // tree over y keeps the code independent of V.
    for (int stride = kLanesY / 2; stride > 0; stride >>= 1) {
        if (threadIdx.y < stride) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                partial[threadIdx.y][threadIdx.x * V + j] +=
                    partial[threadIdx.y + stride][threadIdx.x * V + j];
            }
        }
        __syncthreads();
    }
    if (threadIdx.y == 0 && col < cols) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
            atomicAdd(out + col + j, partial[0][threadIdx.x * V + j]);
        }
    }
}

struct ColumnSumBatch {
    ColumnSumJob job[kColumnSumBatch];
};

// Several small column sums in one launch: block (x, j) sums 128 columns of
// job j (a multiple of four columns wide, a few hundred rows at most), 32
// column lanes of four floats by eight row lanes, folded through shared
// memory.  The result replaces or is added to the destination; a one-row
// source that is a running accumulator is cleared for its next user.
__global__ void __launch_bounds__(256)
column_sums_batch_kernel(const ColumnSumBatch batch) {
    grid_dependency_wait();
    grid_dependency_release();
    __shared__ float4 fold[8][32];
    const ColumnSumJob job = batch.job[blockIdx.y];
    const unsigned lane = threadIdx.x & 31, row_lane = threadIdx.x >> 5;
    const unsigned col = (blockIdx.x * 32 + lane) * 4;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < job.cols) {
        for (unsigned row = row_lane; row < job.rows; row += 8) {
            const float4 v = *reinterpret_cast<const float4 *>(
                job.source + size_t(row) * job.cols + col);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
    }
    fold[row_lane][lane] = sum;
    __syncthreads();
    if (row_lane == 0 && col < job.cols) {
#pragma unroll
        for (int other = 1; other < 8; ++other) {
            const float4 v = fold[other][lane];
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        float4 *target = reinterpret_cast<float4 *>(job.destination + col);
        if (job.add) {
            const float4 old = *target;
            sum.x += old.x; sum.y += old.y; sum.z += old.z; sum.w += old.w;
        }
        *target = sum;
        if (job.clear) {
            for (unsigned row = 0; row < job.rows; ++row) {
                *reinterpret_cast<float4 *>(const_cast<float *>(job.source) +
                                            size_t(row) * job.cols + col) =
                    make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
}

}  // namespace

void launch_column_sums_batch(const ColumnSumJob *jobs, int count,
                              cudaStream_t stream) {
    if (count <= 0) {
        return;
    }
    ColumnSumBatch batch = {};
    unsigned widest = 0;
    for (int j = 0; j < count; ++j) {
        batch.job[j] = jobs[j];
        widest = jobs[j].cols > widest ? jobs[j].cols : widest;
    }
    launch_chained(column_sums_batch_kernel, dim3((widest + 127) / 128, count),
                   256, 0, stream, batch);
    ++g_kernel_launches;
}

void launch_column_sums(const float *in, float *out, size_t rows, size_t cols,
                        size_t ld, cudaStream_t stream) {
    if (rows == 0 || cols == 0) {
        return;
    }
    const bool vec = cols % 4 == 0 && ld % 4 == 0;
    const size_t cols_per_block = kLanesX * (vec ? 4 : 1);
    const unsigned grid_x =
        static_cast<unsigned>((cols + cols_per_block - 1) / cols_per_block);
    size_t slices = (2 * kSmCount + grid_x - 1) / grid_x;
    const size_t max_slices = (rows + 4 * kLanesY - 1) / (4 * kLanesY);
    if (slices > max_slices) {
        slices = max_slices;
    }
    if (slices < 1) {
        slices = 1;
    }
    if (slices > 65535) {
        slices = 65535;
    }
    const size_t rows_per_block = (rows + slices - 1) / slices;
    const dim3 grid(grid_x, static_cast<unsigned>(slices));
    const dim3 block(kLanesX, kLanesY);
    if (vec) {
        launch_chained(column_sums_kernel<4>, grid, block, 0, stream, in, out,
                       rows, cols, ld, rows_per_block);
    } else {
        launch_chained(column_sums_kernel<1>, grid, block, 0, stream, in, out,
                       rows, cols, ld, rows_per_block);
    }
    ++g_kernel_launches;
}

}  // namespace vitb200
