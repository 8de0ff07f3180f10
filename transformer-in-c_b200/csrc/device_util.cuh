// Small device helpers shared by the kernel files.
#pragma once

#include <cstddef>
#include <cuda_runtime.h>

namespace vitb200 {

constexpr unsigned kStreamThreads = 256;
constexpr unsigned kSmCount = 148;         // B200: 2 dies x 74 SMs
constexpr unsigned kStreamBlocksPerSm = 8; // 2048 threads / 256
constexpr unsigned kFullMask = 0xffffffffu;

// Multiprocessors of the current device, asked once (148 on a B200, which is
// also the answer when the query fails).  Persistent grids are sized by it.
inline unsigned device_sm_count() {
    static const unsigned count = []() -> unsigned {
        int device = 0, value = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) !=
                cudaSuccess ||
            value <= 0) {
            cudaGetLastError();
            return kSmCount;
        }
        return unsigned(value);
    }();
    return count;
}

// Grid for a streaming kernel over `items` work items: enough blocks to cover
// them once, capped at one full wave of resident blocks.
inline unsigned stream_grid(size_t items) {
    const size_t wanted = (items + kStreamThreads - 1) / kStreamThreads;
    const size_t wave = size_t(device_sm_count()) * kStreamBlocksPerSm;
    return static_cast<unsigned>(wanted < 1 ? 1 : (wanted < wave ? wanted : wave));
}

__device__ __forceinline__ size_t global_thread() {
    return size_t(blockIdx.x) * blockDim.x + threadIdx.x;
}

__device__ __forceinline__ size_t grid_threads() {
    return size_t(gridDim.x) * blockDim.x;
}

// Read-once data: keep it out of L1.
__device__ __forceinline__ float4 ld_stream(const float4 *pointer) {
    return __ldcs(pointer);
}

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        value += __shfl_xor_sync(kFullMask, value, offset);
    }
    return value;
}

__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        value = fmaxf(value, __shfl_xor_sync(kFullMask, value, offset));
    }
    return value;
}

// tanh-approximation GELU (reference src/ops.c:944-963); the scale is
// sqrtf(2/pi) rounded to float.
constexpr float kGeluCubic = 0.044715f;
constexpr float kGeluScale = 0.7978845608028654f;

__device__ __forceinline__ float gelu_value(float x) {
    return 0.5f * x * (1.0f + tanhf(kGeluScale * (x + kGeluCubic * x * x * x)));
}

// The same function with tanh(u) = 1 - 2 / (1 + exp(2u)) on the fast
// exponential and reciprocal units: absolute error about 2e-7, a third of the
// instructions.  Used where the GELU shares a kernel with a matrix product and
// instruction issue, not memory, is the limit.
__device__ __forceinline__ float gelu_value_fast(float x) {
    const float u = kGeluScale * (x + kGeluCubic * x * x * x);
    const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
    return 0.5f * x * (1.0f + t);
}

// d/dx of gelu_value (reference src/ops.c:986-992).
__device__ __forceinline__ float gelu_slope(float x) {
    const float t = tanhf(kGeluScale * (x + kGeluCubic * x * x * x));
    return 0.5f * (1.0f + t) +
           0.5f * x * (1.0f - t * t) * kGeluScale *
               (1.0f + 3.0f * kGeluCubic * x * x);
}


// gelu_slope with the same fast tanh as gelu_value_fast (absolute error about
// 3e-7), for the epilogue of the product that feeds a GELU's backward pass.
__device__ __forceinline__ float gelu_slope_fast(float x) {
    const float x2 = x * x;
    const float u = kGeluScale * (x + kGeluCubic * x * x2);
    const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
    const float half = 0.5f * (1.0f + t);
    // 0.5 x (1 - t^2) = x half (1 - t)
    return half + x * half * (1.0f - t) * kGeluScale *
                      (1.0f + 3.0f * kGeluCubic * x2);
}

}  // namespace vitb200
