// Small device helpers shared by the kernel files.
#pragma once

#include <cstddef>
#include <cstdlib>
#include <utility>
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

// ---------------------------------------------------------------------------
// Chained launches (programmatic dependent launch).  A kernel launched through
// launch_chained may be scheduled while its predecessor in the stream is still
// running: its blocks become resident as the predecessor's leave, run whatever
// does not touch global memory, and park in grid_dependency_wait() until the
// predecessor has completed and its writes are visible.  That takes the launch
// latency and the block set-up out of the gap between two dependent kernels.
//
// Rules for a kernel launched this way: every thread calls
// grid_dependency_wait() before its first access to global memory and before it
// can return (a grid whose blocks left without waiting would count as complete
// while its predecessors still run, and its successor's wait would pass too
// early).  grid_dependency_release() right after it lets the successor's
// blocks become resident from then on; they park in their own wait.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_dependency_release() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// VITB200_CHAINED_LAUNCHES=0 turns the attribute off (plain stream order).
inline bool chained_launches_enabled() {
    static const bool enabled = []() {
        const char *value = getenv("VITB200_CHAINED_LAUNCHES");
        return !(value && value[0] == '0');
    }();
    return enabled;
}

template <typename... Params, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid,
                                  dim3 block, size_t shared_bytes,
                                  cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed =
        chained_launches_enabled() ? 1 : 0;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
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
