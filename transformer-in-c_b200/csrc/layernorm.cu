// LayerNorm forward and backward, one warp per row, the row held in registers
// (128-bit loads, one HBM read of each input), statistics by warp shuffles.
//
// Formulas follow the host implementation (reference src/ops.c:773-815 and
// :845-904): mean, then the biased variance of the centred values in a second
// pass, inverse_std = 1 / sqrtf(variance + epsilon).  The backward pass
// recomputes the statistics from x instead of reading saved ones, and folds
// the gamma / beta gradients (column sums over all rows) into the same pass:
// each lane keeps running sums for the columns it owns, warps of a block
// combine through shared memory, and one atomic per column and block lands
// the result.
#include "kernels.h"
#include "device_util.cuh"

namespace vitb200 {
namespace {

constexpr int kWarpsPerBlock = 8;

// Lane `lane` owns float4 slots j = 0..NV-1 at columns j*128 + lane*4.
template <int NV>
__device__ __forceinline__ void load_row(const float *row, size_t cols,
                                         int lane, float4 (&v)[NV]) {
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const size_t col = size_t(j) * 128 + lane * 4;
        v[j] = col < cols
            ? __ldcs(reinterpret_cast<const float4 *>(row + col))
            : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

template <int NV>
__device__ __forceinline__ void row_statistics(const float4 (&v)[NV],
                                               size_t cols, int lane,
                                               float epsilon, float &mean,
                                               float &inverse_std) {
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    mean = warp_sum(sum) / float(cols);
    float squares = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        if (size_t(j) * 128 + lane * 4 < cols) {
            const float a = v[j].x - mean, b = v[j].y - mean;
            const float c = v[j].z - mean, d = v[j].w - mean;
            squares += (a * a + b * b) + (c * c + d * d);
        }
    }
    const float variance = warp_sum(squares) / float(cols);
    inverse_std = 1.0f / sqrtf(variance + epsilon);
}

// Rows a warp has in flight at a time: with one, a warp's loads (512 B per
// 128 columns) wait behind its own shuffle reductions and the SM cannot keep
// enough bytes outstanding to reach the memory rate.
template <int NV>
struct RowsInFlight {
    static constexpr int value = NV <= 2 ? 2 : 1;
};

template <int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
layer_norm_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                  const float *__restrict__ beta, float epsilon,
                  float *__restrict__ y, size_t rows, size_t cols,
                  const float *__restrict__ addend, float *__restrict__ sum) {
    grid_dependency_wait();
    grid_dependency_release();
    // With `addend`: the input is x + addend (the residual add the host issued
    // just before, reference src/vit.c:520-523), which is also stored to `sum`.
    constexpr int R = RowsInFlight<NV>::value;
    const int lane = threadIdx.x & 31;
    const size_t warp = size_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    const size_t warps = size_t(gridDim.x) * kWarpsPerBlock;
    float4 g[NV], b[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const size_t col = size_t(j) * 128 + lane * 4;
        if (col < cols) {
            g[j] = __ldg(reinterpret_cast<const float4 *>(gamma + col));
            b[j] = __ldg(reinterpret_cast<const float4 *>(beta + col));
        }
    }
    for (size_t first = warp; first < rows; first += warps * R) {
        float4 v[R][NV], w[R][NV];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const size_t row = first + r * warps;
            // cols = 0 makes load_row fill with zeros without touching memory.
            const size_t width = row < rows ? cols : 0;
            const size_t offset = row < rows ? row * cols : 0;
            load_row<NV>(x + offset, width, lane, v[r]);
            if (addend) {
                load_row<NV>(addend + offset, width, lane, w[r]);
            }
        }
        // Rows past the end are computed on zeros and never stored, so that
        // the rows in flight form one straight-line region whose shuffle
        // reductions the scheduler can interleave.
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const size_t row = first + r * warps;
            const bool live = row < rows;
            if (addend) {
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    v[r][j].x += w[r][j].x;
                    v[r][j].y += w[r][j].y;
                    v[r][j].z += w[r][j].z;
                    v[r][j].w += w[r][j].w;
                    const size_t col = size_t(j) * 128 + lane * 4;
                    if (live && col < cols) {
                        *reinterpret_cast<float4 *>(sum + row * cols + col) = v[r][j];
                    }
                }
            }
            float mean, inverse_std;
            row_statistics<NV>(v[r], cols, lane, epsilon, mean, inverse_std);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const size_t col = size_t(j) * 128 + lane * 4;
                if (live && col < cols) {
                    float4 out;
                    out.x = (v[r][j].x - mean) * inverse_std * g[j].x + b[j].x;
                    out.y = (v[r][j].y - mean) * inverse_std * g[j].y + b[j].y;
                    out.z = (v[r][j].z - mean) * inverse_std * g[j].z + b[j].z;
                    out.w = (v[r][j].w - mean) * inverse_std * g[j].w + b[j].w;
                    *reinterpret_cast<float4 *>(y + row * cols + col) = out;
                }
            }
        }
    }
}

// Rows of 257 to 512 columns (NV = 4) would take 150 registers, i.e. one
// block of eight warps per SM; capped at 128 (eight spilled words) two blocks
// fit, which took the kernel from 0.55 to 0.66 of the copy rate at 384
// columns.  The same trade at NV = 2 (three blocks, 29 spilled words) lost.
// The other widths name the block counts they reach anyway (four at 64
// registers, two at 118): with a bound of one the compiler spends more
// registers and a block of the 128-column kernel no longer fits.
template <int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, NV == 1 ? 4 : (NV <= 4 ? 2 : 1))
layer_norm_backward_kernel(const float *__restrict__ x,
                           const float *__restrict__ gamma, float epsilon,
                           const float *__restrict__ dy, float *dx,
                           float *__restrict__ dgamma, float *__restrict__ dbeta,
                           size_t rows, size_t cols, const float *base,
                           float *__restrict__ dx_sums) {
    grid_dependency_wait();
    grid_dependency_release();
    __shared__ float4 fold[kWarpsPerBlock][32];
    const int lane = threadIdx.x & 31;
    const int warp_in_block = threadIdx.x >> 5;
    const size_t warp = size_t(blockIdx.x) * kWarpsPerBlock + warp_in_block;
    const size_t warps = size_t(gridDim.x) * kWarpsPerBlock;
    float4 g[NV], sum_gamma[NV], sum_beta[NV], sum_dx[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const size_t col = size_t(j) * 128 + lane * 4;
        g[j] = col < cols ? __ldg(reinterpret_cast<const float4 *>(gamma + col))
                          : make_float4(0.f, 0.f, 0.f, 0.f);
        sum_gamma[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        sum_beta[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        sum_dx[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float inverse_cols = 1.0f / float(cols);
    constexpr int R = RowsInFlight<NV>::value;
    for (size_t first = warp; first < rows; first += warps * R) {
        float4 vs[R][NV], us[R][NV], bases[R][NV];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const size_t row = first + r * warps;
            // cols = 0 makes load_row fill with zeros without touching memory.
            const size_t width = row < rows ? cols : 0;
            const size_t offset = row < rows ? row * cols : 0;
            load_row<NV>(x + offset, width, lane, vs[r]);
            load_row<NV>(dy + offset, width, lane, us[r]);
            if (base) {
                load_row<NV>(base + offset, width, lane, bases[r]);
            }
        }
        // Rows past the end are computed on zeros (they add nothing to the
        // column sums) and never stored, so that the rows in flight form one
        // straight-line region whose shuffle reductions the scheduler can
        // interleave.
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const size_t row = first + r * warps;
            const bool live = row < rows;
            float4 (&v)[NV] = vs[r];
            float4 (&u)[NV] = us[r];
            float mean, inverse_std;
            row_statistics<NV>(v, cols, lane, epsilon, mean, inverse_std);
            float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                // Out-of-range slots hold x = 0 and dy = 0, so they add nothing.
                v[j].x = (v[j].x - mean) * inverse_std;
                v[j].y = (v[j].y - mean) * inverse_std;
                v[j].z = (v[j].z - mean) * inverse_std;
                v[j].w = (v[j].w - mean) * inverse_std;
                sum_gamma[j].x += u[j].x * v[j].x;
                sum_gamma[j].y += u[j].y * v[j].y;
                sum_gamma[j].z += u[j].z * v[j].z;
                sum_gamma[j].w += u[j].w * v[j].w;
                sum_beta[j].x += u[j].x;
                sum_beta[j].y += u[j].y;
                sum_beta[j].z += u[j].z;
                sum_beta[j].w += u[j].w;
                u[j].x *= g[j].x;
                u[j].y *= g[j].y;
                u[j].z *= g[j].z;
                u[j].w *= g[j].w;
                s1 += (u[j].x + u[j].y) + (u[j].z + u[j].w);
                s2 += (u[j].x * v[j].x + u[j].y * v[j].y) +
                      (u[j].z * v[j].z + u[j].w * v[j].w);
            }
            s1 = warp_sum(s1) * inverse_cols;
            s2 = warp_sum(s2) * inverse_cols;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const size_t col = size_t(j) * 128 + lane * 4;
                if (live && col < cols) {
                    float4 d = base ? bases[r][j]
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                    d.x += inverse_std * (u[j].x - s1 - v[j].x * s2);
                    d.y += inverse_std * (u[j].y - s1 - v[j].y * s2);
                    d.z += inverse_std * (u[j].z - s1 - v[j].z * s2);
                    d.w += inverse_std * (u[j].w - s1 - v[j].w * s2);
                    *reinterpret_cast<float4 *>(dx + row * cols + col) = d;
                    sum_dx[j].x += d.x;
                    sum_dx[j].y += d.y;
                    sum_dx[j].z += d.z;
                    sum_dx[j].w += d.w;
                }
            }
        }
    }
    // Fold the per-lane column sums over the block's warps.
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const size_t col = size_t(j) * 128 + lane * 4;
#pragma unroll
        for (int which = 0; which < (dx_sums ? 3 : 2); ++which) {
            __syncthreads();
            fold[warp_in_block][lane] =
                which == 0 ? sum_gamma[j] : (which == 1 ? sum_beta[j] : sum_dx[j]);
            __syncthreads();
            if (warp_in_block == 0 && col < cols) {
                float4 total = fold[0][lane];
#pragma unroll
                for (int w = 1; w < kWarpsPerBlock; ++w) {
                    const float4 other = fold[w][lane];
                    total.x += other.x;
                    total.y += other.y;
                    total.z += other.z;
                    total.w += other.w;
                }
                float *target =
                    (which == 0 ? dgamma : (which == 1 ? dbeta : dx_sums)) + col;
                atomicAdd(target + 0, total.x);
                atomicAdd(target + 1, total.y);
                atomicAdd(target + 2, total.z);
                atomicAdd(target + 3, total.w);
            }
        }
    }
}

// Any width: three passes over global memory, one warp per row.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
layer_norm_generic_kernel(const float *__restrict__ x,
                          const float *__restrict__ gamma,
                          const float *__restrict__ beta, float epsilon,
                          float *__restrict__ y, size_t rows, size_t cols) {
    const int lane = threadIdx.x & 31;
    const size_t warp = size_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    const size_t warps = size_t(gridDim.x) * kWarpsPerBlock;
    for (size_t row = warp; row < rows; row += warps) {
        const float *values = x + row * cols;
        float sum = 0.0f;
        for (size_t c = lane; c < cols; c += 32) {
            sum += values[c];
        }
        const float mean = warp_sum(sum) / float(cols);
        float squares = 0.0f;
        for (size_t c = lane; c < cols; c += 32) {
            const float centred = values[c] - mean;
            squares += centred * centred;
        }
        const float inverse_std =
            1.0f / sqrtf(warp_sum(squares) / float(cols) + epsilon);
        for (size_t c = lane; c < cols; c += 32) {
            y[row * cols + c] =
                (values[c] - mean) * inverse_std * gamma[c] + beta[c];
        }
    }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
layer_norm_backward_generic_kernel(const float *__restrict__ x,
                                   const float *__restrict__ gamma,
                                   float epsilon, const float *__restrict__ dy,
                                   float *dx,
                                   float *__restrict__ dgamma,
                                   float *__restrict__ dbeta, size_t rows,
                                   size_t cols, const float *base) {
    const int lane = threadIdx.x & 31;
    const size_t warp = size_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    const size_t warps = size_t(gridDim.x) * kWarpsPerBlock;
    for (size_t row = warp; row < rows; row += warps) {
        const float *values = x + row * cols;
        const float *upstream = dy + row * cols;
        float sum = 0.0f;
        for (size_t c = lane; c < cols; c += 32) {
            sum += values[c];
        }
        const float mean = warp_sum(sum) / float(cols);
        float squares = 0.0f;
        for (size_t c = lane; c < cols; c += 32) {
            const float centred = values[c] - mean;
            squares += centred * centred;
        }
        const float inverse_std =
            1.0f / sqrtf(warp_sum(squares) / float(cols) + epsilon);
        float s1 = 0.0f, s2 = 0.0f;
        for (size_t c = lane; c < cols; c += 32) {
            const float normalised = (values[c] - mean) * inverse_std;
            const float dxhat = upstream[c] * gamma[c];
            s1 += dxhat;
            s2 += dxhat * normalised;
            atomicAdd(dgamma + c, upstream[c] * normalised);
            atomicAdd(dbeta + c, upstream[c]);
        }
        s1 = warp_sum(s1) / float(cols);
        s2 = warp_sum(s2) / float(cols);
        for (size_t c = lane; c < cols; c += 32) {
            const float normalised = (values[c] - mean) * inverse_std;
            const float dxhat = upstream[c] * gamma[c];
            dx[row * cols + c] = (base ? base[row * cols + c] : 0.0f) +
                                 inverse_std * (dxhat - s1 - normalised * s2);
        }
    }
}

unsigned row_grid(size_t rows, unsigned blocks_per_sm) {
    const size_t wanted = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const size_t wave = size_t(kSmCount) * blocks_per_sm;
    return static_cast<unsigned>(wanted < wave ? (wanted ? wanted : 1) : wave);
}

}  // namespace

bool layer_norm_takes_addend(size_t cols) {
    return cols % 4 == 0 && (cols + 127) / 128 <= 8;
}

void launch_layer_norm(const float *x, const float *gamma, const float *beta,
                       float epsilon, float *y, size_t rows, size_t cols,
                       cudaStream_t stream, const float *addend, float *sum) {
    const unsigned grid = row_grid(rows, 8);
    const unsigned block = kWarpsPerBlock * 32;
    const size_t slots = (cols + 127) / 128;
    if (cols % 4 != 0 || slots > 8) {
        layer_norm_generic_kernel<<<grid, block, 0, stream>>>(x, gamma, beta,
                                                              epsilon, y, rows,
                                                              cols);
    } else if (slots <= 1) {
        launch_chained(layer_norm_kernel<1>, grid, block, 0, stream, x, gamma,
                       beta, epsilon, y, rows, cols, addend, sum);
    } else if (slots <= 2) {
        launch_chained(layer_norm_kernel<2>, grid, block, 0, stream, x, gamma,
                       beta, epsilon, y, rows, cols, addend, sum);
    } else if (slots <= 4) {
        launch_chained(layer_norm_kernel<4>, grid, block, 0, stream, x, gamma,
                       beta, epsilon, y, rows, cols, addend, sum);
    } else {
        launch_chained(layer_norm_kernel<8>, grid, block, 0, stream, x, gamma,
                       beta, epsilon, y, rows, cols, addend, sum);
    }
    ++g_kernel_launches;
}

void launch_layer_norm_backward(const float *x, const float *gamma,
                                float epsilon, const float *dy, float *dx,
                                float *dgamma, float *dbeta, size_t rows,
                                size_t cols, const float *base, float *dx_sums,
                                cudaStream_t stream) {
    const unsigned grid = row_grid(rows, 4);
    const unsigned block = kWarpsPerBlock * 32;
    const size_t slots = (cols + 127) / 128;
    if (cols % 4 != 0 || slots > 8) {
        layer_norm_backward_generic_kernel<<<grid, block, 0, stream>>>(
            x, gamma, epsilon, dy, dx, dgamma, dbeta, rows, cols, base);
        if (dx_sums) {
            launch_column_sums(dx, dx_sums, rows, cols, cols, stream);
        }
    } else if (slots <= 1) {
        launch_chained(layer_norm_backward_kernel<1>, grid, block, 0, stream, x,
                       gamma, epsilon, dy, dx, dgamma, dbeta, rows, cols, base,
                       dx_sums);
    } else if (slots <= 2) {
        launch_chained(layer_norm_backward_kernel<2>, grid, block, 0, stream, x,
                       gamma, epsilon, dy, dx, dgamma, dbeta, rows, cols, base,
                       dx_sums);
    } else if (slots <= 4) {
        launch_chained(layer_norm_backward_kernel<4>, grid, block, 0, stream, x,
                       gamma, epsilon, dy, dx, dgamma, dbeta, rows, cols, base,
                       dx_sums);
    } else {
        launch_chained(layer_norm_backward_kernel<8>, grid, block, 0, stream, x,
                       gamma, epsilon, dy, dx, dgamma, dbeta, rows, cols, base,
                       dx_sums);
    }
    ++g_kernel_launches;
}

}  // namespace vitb200
