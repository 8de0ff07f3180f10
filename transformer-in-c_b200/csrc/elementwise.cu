// Streaming elementwise kernels: 128-bit loads and stores, grid sized to a
// multiple of the SM count, grid-stride loops.  All of them are HBM-bound.
#include "kernels.h"
#include "device_util.cuh"

namespace vitb200 {

unsigned long long g_kernel_launches = 0;

namespace {

// ---- functors: each maps one float4 lane set (and a scalar tail) ----------

__global__ void add_kernel(const float *__restrict__ a,
                           const float *__restrict__ b, float *__restrict__ out,
                           size_t n) {
    grid_dependency_wait();
    grid_dependency_release();
    const size_t vectors = n / 4;
    const float4 *a4 = reinterpret_cast<const float4 *>(a);
    const float4 *b4 = reinterpret_cast<const float4 *>(b);
    float4 *o4 = reinterpret_cast<float4 *>(out);
    for (size_t i = global_thread(); i < vectors; i += grid_threads()) {
        const float4 x = ld_stream(a4 + i);
        const float4 y = ld_stream(b4 + i);
        o4[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
    for (size_t i = vectors * 4 + global_thread(); i < n; i += grid_threads()) {
        out[i] = a[i] + b[i];
    }
}

// add = false turns "+=" into "=" (the destination is known to be zero).
__global__ void accumulate_kernel(float *__restrict__ dst,
                                  const float *__restrict__ src, size_t n,
                                  bool add) {
    grid_dependency_wait();
    grid_dependency_release();
    const size_t vectors = n / 4;
    float4 *d4 = reinterpret_cast<float4 *>(dst);
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    for (size_t i = global_thread(); i < vectors; i += grid_threads()) {
        float4 d = add ? d4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 s = ld_stream(s4 + i);
        d.x += s.x; d.y += s.y; d.z += s.z; d.w += s.w;
        d4[i] = d;
    }
    for (size_t i = vectors * 4 + global_thread(); i < n; i += grid_threads()) {
        dst[i] = (add ? dst[i] : 0.0f) + src[i];
    }
}

__global__ void accumulate2_kernel(float *__restrict__ dst_a,
                                   float *__restrict__ dst_b,
                                   const float *__restrict__ src, size_t n,
                                   bool add_a, bool add_b) {
    grid_dependency_wait();
    grid_dependency_release();
    const size_t vectors = n / 4;
    float4 *a4 = reinterpret_cast<float4 *>(dst_a);
    float4 *b4 = reinterpret_cast<float4 *>(dst_b);
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    for (size_t i = global_thread(); i < vectors; i += grid_threads()) {
        const float4 s = ld_stream(s4 + i);
        float4 a = add_a ? a4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 b = add_b ? b4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        a.x += s.x; a.y += s.y; a.z += s.z; a.w += s.w;
        b.x += s.x; b.y += s.y; b.z += s.z; b.w += s.w;
        a4[i] = a;
        b4[i] = b;
    }
    for (size_t i = vectors * 4 + global_thread(); i < n; i += grid_threads()) {
        dst_a[i] = (add_a ? dst_a[i] : 0.0f) + src[i];
        dst_b[i] = (add_b ? dst_b[i] : 0.0f) + src[i];
    }
}

// in and out may be the same buffer, so neither is __restrict__.
__global__ void bias_add_vec_kernel(const float *in,
                                    const float *__restrict__ bias, float *out,
                                    size_t rows, size_t cols) {
    grid_dependency_wait();
    grid_dependency_release();
    const size_t row_vectors = cols / 4;
    const size_t vectors = rows * row_vectors;
    const float4 *i4 = reinterpret_cast<const float4 *>(in);
    const float4 *b4 = reinterpret_cast<const float4 *>(bias);
    float4 *o4 = reinterpret_cast<float4 *>(out);
    for (size_t i = global_thread(); i < vectors; i += grid_threads()) {
        const float4 x = i4[i];
        const float4 b = __ldg(b4 + i % row_vectors);
        o4[i] = make_float4(x.x + b.x, x.y + b.y, x.z + b.z, x.w + b.w);
    }
}

__global__ void bias_add_scalar_kernel(const float *in,
                                       const float *__restrict__ bias,
                                       float *out, size_t rows, size_t cols) {
    grid_dependency_wait();
    grid_dependency_release();
    const size_t n = rows * cols;
    for (size_t i = global_thread(); i < n; i += grid_threads()) {
        out[i] = in[i] + __ldg(bias + i % cols);
    }
}

__global__ void gelu_kernel(const float *__restrict__ in,
                            float *__restrict__ out, size_t n) {
    grid_dependency_wait();
    grid_dependency_release();
    const size_t vectors = n / 4;
    const float4 *i4 = reinterpret_cast<const float4 *>(in);
    float4 *o4 = reinterpret_cast<float4 *>(out);
    for (size_t i = global_thread(); i < vectors; i += grid_threads()) {
        const float4 x = i4[i];
        o4[i] = make_float4(gelu_value(x.x), gelu_value(x.y), gelu_value(x.z),
                            gelu_value(x.w));
    }
    for (size_t i = vectors * 4 + global_thread(); i < n; i += grid_threads()) {
        out[i] = gelu_value(in[i]);
    }
}

__global__ void gelu_backward_kernel(const float *__restrict__ x,
                                     const float *__restrict__ dy,
                                     float *__restrict__ dx, size_t n,
                                     bool add) {
    grid_dependency_wait();
    grid_dependency_release();
    const size_t vectors = n / 4;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *g4 = reinterpret_cast<const float4 *>(dy);
    float4 *d4 = reinterpret_cast<float4 *>(dx);
    for (size_t i = global_thread(); i < vectors; i += grid_threads()) {
        const float4 v = ld_stream(x4 + i);
        const float4 g = ld_stream(g4 + i);
        float4 d = add ? d4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        d.x += g.x * gelu_slope(v.x);
        d.y += g.y * gelu_slope(v.y);
        d.z += g.z * gelu_slope(v.z);
        d.w += g.w * gelu_slope(v.w);
        d4[i] = d;
    }
    for (size_t i = vectors * 4 + global_thread(); i < n; i += grid_threads()) {
        dx[i] = (add ? dx[i] : 0.0f) + dy[i] * gelu_slope(x[i]);
    }
}

// The same with the column sums of the result accumulated on the way (they
// are the bias gradient the host asks for next, reference src/vit.c:554-555).
// A row is cols / 4 threads wide and that divides the block, so a thread keeps
// its four columns for every row it visits and sums them in registers; the
// block's threads that share columns are folded in shared memory, and the
// block writes its sums as row blockIdx.x of `partials` ([gridDim.x, cols]);
// atomics from a full wave of blocks onto so few addresses cost more than the
// pass they save.
__global__ void __launch_bounds__(kStreamThreads)
gelu_backward_sums_kernel(const float *__restrict__ x,
                          const float *__restrict__ dy, float *__restrict__ dx,
                          float *__restrict__ partials, size_t rows,
                          size_t cols, bool add) {
    grid_dependency_wait();
    grid_dependency_release();
    __shared__ float4 fold[kStreamThreads];
    const unsigned row_threads = unsigned(cols / 4);
    const unsigned rows_per_block = kStreamThreads / row_threads;
    const unsigned column = threadIdx.x % row_threads;
    const unsigned sub_row = threadIdx.x / row_threads;
    float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
    for (size_t row = size_t(blockIdx.x) * rows_per_block + sub_row; row < rows;
         row += size_t(gridDim.x) * rows_per_block) {
        const size_t i = row * row_threads + column;
        const float4 v = ld_stream(reinterpret_cast<const float4 *>(x) + i);
        const float4 g = ld_stream(reinterpret_cast<const float4 *>(dy) + i);
        float4 *target = reinterpret_cast<float4 *>(dx) + i;
        float4 d = add ? *target : make_float4(0.f, 0.f, 0.f, 0.f);
        d.x += g.x * gelu_slope(v.x);
        d.y += g.y * gelu_slope(v.y);
        d.z += g.z * gelu_slope(v.z);
        d.w += g.w * gelu_slope(v.w);
        *target = d;
        total.x += d.x;
        total.y += d.y;
        total.z += d.z;
        total.w += d.w;
    }
    fold[threadIdx.x] = total;
    __syncthreads();
    if (sub_row == 0) {
        for (unsigned r = 1; r < rows_per_block; ++r) {
            const float4 other = fold[r * row_threads + column];
            total.x += other.x;
            total.y += other.y;
            total.z += other.z;
            total.w += other.w;
        }
        reinterpret_cast<float4 *>(partials + size_t(blockIdx.x) * cols)[column] =
            total;
    }
}

// out (+)= sums, and the sums go back to zero for their next user.
__global__ void take_column_sums_kernel(float *__restrict__ out,
                                        float *__restrict__ sums, size_t cols,
                                        bool add) {
    grid_dependency_wait();
    grid_dependency_release();
    for (size_t c = global_thread(); c < cols; c += grid_threads()) {
        out[c] = (add ? out[c] : 0.0f) + sums[c];
        sums[c] = 0.0f;
    }
}

__global__ void scale_by_device_scalar_kernel(float *__restrict__ values,
                                              size_t n,
                                              const float *__restrict__ scale) {
    grid_dependency_wait();
    grid_dependency_release();
    const float s = __ldg(scale);
    if (s == 1.0f) {
        return;
    }
    const size_t vectors = n / 4;
    float4 *v4 = reinterpret_cast<float4 *>(values);
    for (size_t i = global_thread(); i < vectors; i += grid_threads()) {
        float4 v = v4[i];
        v.x *= s; v.y *= s; v.z *= s; v.w *= s;
        v4[i] = v;
    }
    for (size_t i = vectors * 4 + global_thread(); i < n; i += grid_threads()) {
        values[i] *= s;
    }
}

}  // namespace

void launch_add(const float *a, const float *b, float *out, size_t n,
                cudaStream_t stream) {
    launch_chained(add_kernel, stream_grid(n / 4 + 1), kStreamThreads, 0,
                   stream, a, b, out, n);
    ++g_kernel_launches;
}

void launch_accumulate(float *dst, const float *src, size_t n, bool add,
                       cudaStream_t stream) {
    launch_chained(accumulate_kernel, stream_grid(n / 4 + 1), kStreamThreads, 0,
                   stream, dst, src, n, add);
    ++g_kernel_launches;
}

void launch_accumulate2(float *dst_a, float *dst_b, const float *src, size_t n,
                        bool add_a, bool add_b, cudaStream_t stream) {
    launch_chained(accumulate2_kernel, stream_grid(n / 4 + 1), kStreamThreads,
                   0, stream, dst_a, dst_b, src, n, add_a, add_b);
    ++g_kernel_launches;
}

void launch_bias_add(const float *in, const float *bias, float *out,
                     size_t rows, size_t cols, cudaStream_t stream) {
    if (cols % 4 == 0) {
        launch_chained(bias_add_vec_kernel, stream_grid(rows * cols / 4),
                       kStreamThreads, 0, stream, in, bias, out, rows, cols);
    } else {
        launch_chained(bias_add_scalar_kernel, stream_grid(rows * cols),
                       kStreamThreads, 0, stream, in, bias, out, rows, cols);
    }
    ++g_kernel_launches;
}

void launch_gelu(const float *in, float *out, size_t n, cudaStream_t stream) {
    launch_chained(gelu_kernel, stream_grid(n / 4 + 1), kStreamThreads, 0,
                   stream, in, out, n);
    ++g_kernel_launches;
}

void launch_gelu_backward(const float *x, const float *dy, float *dx, size_t n,
                          bool add, cudaStream_t stream) {
    launch_chained(gelu_backward_kernel, stream_grid(n / 4 + 1), kStreamThreads,
                   0, stream, x, dy, dx, n, add);
    ++g_kernel_launches;
}

bool gelu_backward_sums_supported(size_t cols) {
    return cols >= 4 && cols % 4 == 0 && cols / 4 <= kStreamThreads &&
           kStreamThreads % (cols / 4) == 0;
}

size_t gelu_backward_sums_blocks(size_t rows, size_t cols) {
    const size_t rows_per_block = kStreamThreads / (cols / 4);
    const size_t wanted = (rows + rows_per_block - 1) / rows_per_block;
    const size_t limit = size_t(kSmCount) * kStreamBlocksPerSm;   // one wave
    return wanted < limit ? wanted : limit;
}

void launch_gelu_backward_sums(const float *x, const float *dy, float *dx,
                               float *partials, size_t rows, size_t cols,
                               bool add, cudaStream_t stream) {
    launch_chained(gelu_backward_sums_kernel,
                   unsigned(gelu_backward_sums_blocks(rows, cols)),
                   kStreamThreads, 0, stream, x, dy, dx, partials, rows, cols,
                   add);
    ++g_kernel_launches;
}

void launch_take_column_sums(float *out, float *sums, size_t cols, bool add,
                             cudaStream_t stream) {
    launch_chained(take_column_sums_kernel, stream_grid(cols), kStreamThreads,
                   0, stream, out, sums, cols, add);
    ++g_kernel_launches;
}

void launch_scale_by_device_scalar(float *values, size_t n, const float *scale,
                                   cudaStream_t stream) {
    launch_chained(scale_by_device_scalar_kernel, stream_grid(n / 4 + 1),
                   kStreamThreads, 0, stream, values, n, scale);
    ++g_kernel_launches;
}

}  // namespace vitb200
