// Multi-tensor optimiser kernels: global gradient norm, clip scale, gradient
// scaling and AdamW with decoupled weight decay (reference src/ops.c:588-617
// and :1084-1100).
//
// The parameter set is described by a table of slices resident in device
// memory.  Work is cut into blocks of kSliceBlockElements consecutive
// elements of one slice; `first_block` is the running block count, so a block
// finds its slice with a short binary search and then streams its elements
// with 128-bit accesses.  One launch therefore covers every parameter tensor,
// whatever their sizes.
#include "kernels.h"
#include "device_util.cuh"

namespace vitb200 {
namespace {

constexpr unsigned kThreads = 256;

struct BlockRange {
    const ParameterSlice *slice;
    unsigned long long begin;
    unsigned long long end;
};

__device__ __forceinline__ BlockRange locate(const ParameterSlice *slices,
                                             unsigned slices_n,
                                             unsigned block) {
    unsigned low = 0, high = slices_n - 1;
    while (low < high) {
        const unsigned middle = (low + high + 1) / 2;
        if (slices[middle].first_block <= block) {
            low = middle;
        } else {
            high = middle - 1;
        }
    }
    BlockRange range;
    range.slice = slices + low;
    range.begin = (unsigned long long)(block - slices[low].first_block) *
                  kSliceBlockElements;
    const unsigned long long end = range.begin + kSliceBlockElements;
    range.end = end < slices[low].count ? end : slices[low].count;
    return range;
}

__device__ __forceinline__ float block_sum(float value, float *scratch) {
    value = warp_sum(value);
    if ((threadIdx.x & 31) == 0) {
        scratch[threadIdx.x >> 5] = value;
    }
    __syncthreads();
    float total = 0.0f;
    if (threadIdx.x < 32) {
        total = threadIdx.x < (blockDim.x >> 5) ? scratch[threadIdx.x] : 0.0f;
        total = warp_sum(total);
    }
    return total;  // valid in thread 0
}

__global__ void __launch_bounds__(kThreads)
squared_norm_partials_kernel(const ParameterSlice *__restrict__ slices,
                             unsigned slices_n, float *__restrict__ partials) {
    grid_dependency_wait();
    grid_dependency_release();
    __shared__ float scratch[32];
    const BlockRange range = locate(slices, slices_n, blockIdx.x);
    const float *g = range.slice->grad;
    float sum = 0.0f;
    // Slices start 16-byte aligned and block ranges start on multiples of
    // 4096 elements, so the vector path only needs a scalar tail.
    const unsigned long long vector_end =
        range.begin + (range.end - range.begin) / 4 * 4;
    for (unsigned long long i = range.begin + threadIdx.x * 4ull; i < vector_end;
         i += kThreads * 4ull) {
        const float4 v = *reinterpret_cast<const float4 *>(g + i);
        sum += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    }
    for (unsigned long long i = vector_end + threadIdx.x; i < range.end;
         i += kThreads) {
        sum += g[i] * g[i];
    }
    const float total = block_sum(sum, scratch);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = total;
    }
}

// scale = norm > max_norm ? max_norm / norm : 1, with the norm summed in
// double precision in a fixed order (the host sums in double too).
//
// With data parallelism the gradients hold the sum over `1 / inverse_world`
// ranks; the norm of their mean is the summed norm times inverse_world, and the
// same factor is folded into the scale so the optimiser sees the mean.
__global__ void clip_scale_kernel(const float *__restrict__ partials,
                                  unsigned count, float max_norm,
                                  float inverse_world,
                                  float *__restrict__ scale_out) {
    grid_dependency_wait();
    grid_dependency_release();
    __shared__ double scratch[32];
    double sum = 0.0;
    for (unsigned i = threadIdx.x; i < count; i += blockDim.x) {
        sum += double(partials[i]);
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        sum += __shfl_xor_sync(kFullMask, sum, offset);
    }
    if ((threadIdx.x & 31) == 0) {
        scratch[threadIdx.x >> 5] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double total = 0.0;
        for (unsigned w = 0; w < (blockDim.x >> 5); ++w) {
            total += scratch[w];
        }
        const double norm = sqrt(total) * double(inverse_world);
        const float clip = (norm <= double(max_norm) || norm == 0.0)
            ? 1.0f
            : float(double(max_norm) / norm);
        scale_out[0] = inverse_world == 1.0f ? clip : clip * inverse_world;
    }
}

__global__ void __launch_bounds__(kThreads)
scale_gradients_kernel(const ParameterSlice *__restrict__ slices,
                       unsigned slices_n, const float *__restrict__ scale) {
    grid_dependency_wait();
    grid_dependency_release();
    const float s = scale[0];
    if (s == 1.0f) {
        return;
    }
    const BlockRange range = locate(slices, slices_n, blockIdx.x);
    float *g = range.slice->grad;
    for (unsigned long long i = range.begin + threadIdx.x; i < range.end;
         i += kThreads) {
        g[i] *= s;
    }
}

__device__ __forceinline__ void adamw_element(float &w, float &g, float &m,
                                              float &v, float scale, float lr,
                                              float beta1, float beta2,
                                              float epsilon, float weight_decay,
                                              float correction1,
                                              float correction2) {
    const float gradient = scale == 1.0f ? g : g * scale;
    m = beta1 * m + (1.0f - beta1) * gradient;
    v = beta2 * v + (1.0f - beta2) * gradient * gradient;
    const float estimate =
        (m / correction1) / (sqrtf(v / correction2) + epsilon);
    w -= lr * (estimate + weight_decay * w);
    g = 0.0f;
}

__global__ void __launch_bounds__(kThreads)
adamw_kernel(const ParameterSlice *__restrict__ slices, unsigned slices_n,
             const float *__restrict__ scale_pointer, float lr, float beta1,
             float beta2, float epsilon) {
    grid_dependency_wait();
    grid_dependency_release();
    const float scale = scale_pointer ? scale_pointer[0] : 1.0f;
    const BlockRange range = locate(slices, slices_n, blockIdx.x);
    const ParameterSlice s = *range.slice;
    const unsigned long long vector_end =
        range.begin + (range.end - range.begin) / 4 * 4;
    for (unsigned long long i = range.begin + threadIdx.x * 4ull; i < vector_end;
         i += kThreads * 4ull) {
        float4 w = *reinterpret_cast<float4 *>(s.value + i);
        float4 g = *reinterpret_cast<float4 *>(s.grad + i);
        float4 m = *reinterpret_cast<float4 *>(s.m + i);
        float4 v = *reinterpret_cast<float4 *>(s.v + i);
        adamw_element(w.x, g.x, m.x, v.x, scale, lr, beta1, beta2, epsilon,
                      s.weight_decay, s.correction1, s.correction2);
        adamw_element(w.y, g.y, m.y, v.y, scale, lr, beta1, beta2, epsilon,
                      s.weight_decay, s.correction1, s.correction2);
        adamw_element(w.z, g.z, m.z, v.z, scale, lr, beta1, beta2, epsilon,
                      s.weight_decay, s.correction1, s.correction2);
        adamw_element(w.w, g.w, m.w, v.w, scale, lr, beta1, beta2, epsilon,
                      s.weight_decay, s.correction1, s.correction2);
        *reinterpret_cast<float4 *>(s.value + i) = w;
        *reinterpret_cast<float4 *>(s.grad + i) = g;
        *reinterpret_cast<float4 *>(s.m + i) = m;
        *reinterpret_cast<float4 *>(s.v + i) = v;
    }
    for (unsigned long long i = vector_end + threadIdx.x; i < range.end;
         i += kThreads) {
        adamw_element(s.value[i], s.grad[i], s.m[i], s.v[i], scale, lr, beta1,
                      beta2, epsilon, s.weight_decay, s.correction1,
                      s.correction2);
    }
}

__global__ void adamw_single_kernel(float *__restrict__ value,
                                    float *__restrict__ grad,
                                    float *__restrict__ m, float *__restrict__ v,
                                    size_t n, float lr, float beta1, float beta2,
                                    float epsilon, float weight_decay,
                                    float correction1, float correction2) {
    grid_dependency_wait();
    grid_dependency_release();
    for (size_t i = global_thread(); i < n; i += grid_threads()) {
        adamw_element(value[i], grad[i], m[i], v[i], 1.0f, lr, beta1, beta2,
                      epsilon, weight_decay, correction1, correction2);
    }
}

}  // namespace

void launch_gradient_clip_scale(const ParameterSlice *slices, unsigned slices_n,
                                unsigned total_blocks, float max_norm,
                                float inverse_world, float *partials,
                                float *scale_out, cudaStream_t stream) {
    launch_chained(squared_norm_partials_kernel, total_blocks, kThreads, 0,
                   stream, slices, slices_n, partials);
    launch_chained(clip_scale_kernel, 1, 1024, 0, stream, partials,
                   total_blocks, max_norm, inverse_world, scale_out);
    g_kernel_launches += 2;
}

void launch_scale_gradients(const ParameterSlice *slices, unsigned slices_n,
                            unsigned total_blocks, const float *scale,
                            cudaStream_t stream) {
    launch_chained(scale_gradients_kernel, total_blocks, kThreads, 0, stream,
                   slices, slices_n, scale);
    ++g_kernel_launches;
}

void launch_adamw(const ParameterSlice *slices, unsigned slices_n,
                  unsigned total_blocks, const float *scale, float lr,
                  float beta1, float beta2, float epsilon,
                  cudaStream_t stream) {
    launch_chained(adamw_kernel, total_blocks, kThreads, 0, stream, slices,
                   slices_n, scale, lr, beta1, beta2, epsilon);
    ++g_kernel_launches;
}

void launch_adamw_single(float *value, float *grad, float *m, float *v,
                         size_t n, float lr, float beta1, float beta2,
                         float epsilon, float weight_decay, float correction1,
                         float correction2, cudaStream_t stream) {
    launch_chained(adamw_single_kernel, stream_grid(n), kStreamThreads, 0,
                   stream, value, grad, m, v, n, lr, beta1, beta2, epsilon,
                   weight_decay, correction1, correction2);
    ++g_kernel_launches;
}

}  // namespace vitb200
