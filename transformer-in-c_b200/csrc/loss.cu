// Softmax cross-entropy with label smoothing and optional class weights
// (reference src/ops.c:1025-1072).  Targets arrive as floats in a [rows, 1]
// tensor (reference src/ops.c:359-368).
//
//   off = smoothing / cols, on = 1 - smoothing + off
//   loss = (1/rows) * sum_r w_r * sum_c t_rc * (lse_r - z_rc)
//   grad_rc = (grad_rc + w_r * (p_rc - t_rc)) / rows
//
// One warp per row (any class count); the per-row losses go to a scratch
// array and a single block adds them in a fixed order, so the reported loss is
// reproducible run to run.
#include "kernels.h"
#include "device_util.cuh"

#include <cfloat>

namespace vitb200 {
namespace {

__global__ void cross_entropy_rows_kernel(
    const float *__restrict__ logits, const float *__restrict__ targets,
    const float *__restrict__ class_weights, float label_smoothing,
    float *__restrict__ logits_grad, float *__restrict__ row_losses,
    size_t rows, size_t cols) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const size_t warps = (size_t(gridDim.x) * blockDim.x) >> 5;
    const float off = label_smoothing / float(cols);
    const float on = 1.0f - label_smoothing + off;
    for (size_t row = warp; row < rows; row += warps) {
        const float *z = logits + row * cols;
        const size_t target = static_cast<size_t>(targets[row]);
        float maximum = -FLT_MAX;
        for (size_t c = lane; c < cols; c += 32) {
            maximum = fmaxf(maximum, z[c]);
        }
        maximum = warp_max(maximum);
        float denominator = 0.0f;
        for (size_t c = lane; c < cols; c += 32) {
            denominator += expf(z[c] - maximum);
        }
        denominator = warp_sum(denominator);
        const float lse = maximum + logf(denominator);
        const float weight =
            class_weights ? class_weights[target < cols ? target : 0] : 1.0f;
        float loss = 0.0f;
        for (size_t c = lane; c < cols; c += 32) {
            const float t = c == target ? on : off;
            const float probability = expf(z[c] - lse);
            loss += weight * t * (lse - z[c]);
            float *g = logits_grad + row * cols + c;
            // Same rounding as "accumulate, then divide by rows" on the host.
            *g = (*g + weight * (probability - t)) / float(rows);
        }
        loss = warp_sum(loss);
        if (lane == 0) {
            row_losses[row] = loss;
        }
    }
}

__global__ void mean_of_rows_kernel(const float *__restrict__ row_losses,
                                    float *__restrict__ loss, size_t rows) {
    __shared__ float partial[32];
    float sum = 0.0f;
    for (size_t i = threadIdx.x; i < rows; i += blockDim.x) {
        sum += row_losses[i];
    }
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) {
        partial[threadIdx.x >> 5] = sum;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        sum = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0f;
        sum = warp_sum(sum);
        if (threadIdx.x == 0) {
            loss[0] = sum / float(rows);
        }
    }
}

}  // namespace

void launch_softmax_cross_entropy(const float *logits, const float *targets,
                                  const float *class_weights,
                                  float label_smoothing, float *loss,
                                  float *logits_grad, float *row_losses,
                                  size_t rows, size_t cols,
                                  cudaStream_t stream) {
    cross_entropy_rows_kernel<<<stream_grid(rows * 32), kStreamThreads, 0,
                                stream>>>(logits, targets, class_weights,
                                          label_smoothing, logits_grad,
                                          row_losses, rows, cols);
    mean_of_rows_kernel<<<1, 1024, 0, stream>>>(row_losses, loss, rows);
    g_kernel_launches += 2;
}

}  // namespace vitb200
