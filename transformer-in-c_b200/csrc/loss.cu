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
#include <cstdio>

namespace vitb200 {
namespace {

__global__ void cross_entropy_rows_kernel(
    const float *__restrict__ logits, const float *__restrict__ targets,
    const float *__restrict__ class_weights, float label_smoothing,
    float *__restrict__ logits_grad, float *__restrict__ row_losses,
    size_t rows, size_t cols) {
    grid_dependency_wait();
    grid_dependency_release();
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
    grid_dependency_wait();
    grid_dependency_release();
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

// Row-loss scratch for launch_softmax_cross_entropy_static.  It lives in the
// library image, so every GPU that loads the library carries these 256 KiB
// until the process exits.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_static_row_losses[kStaticLossMaxRows];

constexpr int kMaxDevices = 64;
float *g_static_row_losses_address[kMaxDevices] = {};

}  // namespace

int launch_softmax_cross_entropy_static(const float *logits,
                                        const float *targets,
                                        const float *class_weights,
                                        float label_smoothing, float *loss,
                                        float *logits_grad, size_t rows,
                                        size_t cols, cudaStream_t stream) {
    if (rows == 0 || cols == 0) {
        return -1;
    }
    if (rows > kStaticLossMaxRows) {
        fprintf(stderr,
                "vitb200: softmax_cross_entropy_static handles at most %zu rows "
                "(got %zu); use the variant that takes a scratch buffer\n",
                size_t(kStaticLossMaxRows), rows);
        return -2;
    }
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 ||
        device >= kMaxDevices) {
        return -1;
    }
    // First call on this device: resolve where the array sits in this
    // device's memory.  The lookup is done once and must not happen while a
    // stream is being captured.
    if (!g_static_row_losses_address[device]) {
        void *address = nullptr;
        const cudaError_t status =
            cudaGetSymbolAddress(&address, g_static_row_losses);
        if (status != cudaSuccess || !address) {
            fprintf(stderr, "vitb200: cudaGetSymbolAddress failed: %s\n",
                    cudaGetErrorString(status));
            return -1;
        }
        g_static_row_losses_address[device] = static_cast<float *>(address);
    }
    // Every row the reduction reads is written by the row kernel first, so
    // nothing left over from the previous call is ever observed and no
    // clearing is needed.
    launch_softmax_cross_entropy(logits, targets, class_weights,
                                 label_smoothing, loss, logits_grad,
                                 g_static_row_losses_address[device], rows, cols,
                                 stream);
    return 0;
}

void launch_softmax_cross_entropy(const float *logits, const float *targets,
                                  const float *class_weights,
                                  float label_smoothing, float *loss,
                                  float *logits_grad, float *row_losses,
                                  size_t rows, size_t cols,
                                  cudaStream_t stream) {
    launch_chained(cross_entropy_rows_kernel, stream_grid(rows * 32),
                   kStreamThreads, 0, stream, logits, targets, class_weights,
                   label_smoothing, logits_grad, row_losses, rows, cols);
    launch_chained(mean_of_rows_kernel, 1, 1024, 0, stream, row_losses, loss,
                   rows);
    g_kernel_launches += 2;
}

}  // namespace vitb200
