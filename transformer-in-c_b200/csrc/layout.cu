// Re-layout kernels: head split/merge, patch extraction, token embedding and
// row gathers.  Pure data movement plus at most one add; every kernel walks
// its *destination* contiguously so stores are fully coalesced.
#include "kernels.h"
#include "device_util.cuh"

namespace vitb200 {
namespace {

template <int V> struct Vec;
template <> struct Vec<1> { using type = float; };
template <> struct Vec<4> { using type = float4; };

__device__ __forceinline__ float vadd(float a, float b) { return a + b; }
__device__ __forceinline__ float4 vadd(float4 a, float4 b) {
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

// Head-major row (reference src/ops.c:298-301): (sample*heads + head)*seq + pos.
// `i` indexes vectors of V floats in a [batch*heads*seq, head_dim] tensor; the
// result is the vector index of the same element inside a token-major matrix
// whose rows have `row_floats` floats, at column offset `col0`.
template <int V>
__device__ __forceinline__ size_t token_major_index(size_t i, size_t seq,
                                                    size_t heads,
                                                    size_t head_dim,
                                                    size_t row_floats,
                                                    size_t col0) {
    const size_t vectors_per_head_row = head_dim / V;
    const size_t head_row = i / vectors_per_head_row;
    const size_t dim = (i % vectors_per_head_row) * V;
    const size_t group = head_row / seq;
    const size_t position = head_row % seq;
    const size_t sample = group / heads;
    const size_t head = group % heads;
    return ((sample * seq + position) * row_floats + col0 + head * head_dim +
            dim) / V;
}

template <int V>
__global__ void split_heads_kernel(const float *__restrict__ projected,
                                   float *__restrict__ q, float *__restrict__ k,
                                   float *__restrict__ v, size_t batch,
                                   size_t seq, size_t d_model, size_t heads) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t head_dim = d_model / heads;
    const size_t total = batch * seq * d_model / V;
    const T *source = reinterpret_cast<const T *>(projected);
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t s =
            token_major_index<V>(i, seq, heads, head_dim, 3 * d_model, 0);
        reinterpret_cast<T *>(q)[i] = source[s];
        reinterpret_cast<T *>(k)[i] = source[s + d_model / V];
        reinterpret_cast<T *>(v)[i] = source[s + 2 * d_model / V];
    }
}

// Walks the projected gradient (the destination) contiguously.
template <int V>
__global__ void split_heads_backward_kernel(float *__restrict__ projected_grad,
                                            const float *__restrict__ dq,
                                            const float *__restrict__ dk,
                                            const float *__restrict__ dv,
                                            size_t batch, size_t seq,
                                            size_t d_model, size_t heads,
                                            bool add) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t head_dim = d_model / heads;
    const size_t row_vectors = 3 * d_model / V;
    const size_t total = batch * seq * row_vectors;
    T *destination = reinterpret_cast<T *>(projected_grad);
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t token = i / row_vectors;
        const size_t col = (i % row_vectors) * V;
        const size_t which = col / d_model;
        const size_t inner = col % d_model;
        const size_t head = inner / head_dim;
        const size_t dim = inner % head_dim;
        const size_t sample = token / seq;
        const size_t position = token % seq;
        const size_t source =
            (((sample * heads + head) * seq + position) * head_dim + dim) / V;
        const float *from = which == 0 ? dq : (which == 1 ? dk : dv);
        const T value = reinterpret_cast<const T *>(from)[source];
        destination[i] = add ? vadd(destination[i], value) : value;
    }
}

template <int V>
__global__ void merge_heads_kernel(const float *__restrict__ attended,
                                   float *__restrict__ merged, size_t batch,
                                   size_t seq, size_t d_model, size_t heads) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t head_dim = d_model / heads;
    const size_t row_vectors = d_model / V;
    const size_t total = batch * seq * row_vectors;
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t token = i / row_vectors;
        const size_t col = (i % row_vectors) * V;
        const size_t head = col / head_dim;
        const size_t dim = col % head_dim;
        const size_t sample = token / seq;
        const size_t position = token % seq;
        const size_t source =
            (((sample * heads + head) * seq + position) * head_dim + dim) / V;
        reinterpret_cast<T *>(merged)[i] =
            reinterpret_cast<const T *>(attended)[source];
    }
}

template <int V>
__global__ void merge_heads_backward_kernel(float *__restrict__ attended_grad,
                                            const float *__restrict__ merged_grad,
                                            size_t batch, size_t seq,
                                            size_t d_model, size_t heads,
                                            bool add) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t head_dim = d_model / heads;
    const size_t total = batch * seq * d_model / V;
    T *destination = reinterpret_cast<T *>(attended_grad);
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t s =
            token_major_index<V>(i, seq, heads, head_dim, d_model, 0);
        const T value = reinterpret_cast<const T *>(merged_grad)[s];
        destination[i] = add ? vadd(destination[i], value) : value;
    }
}

// One head-major tensor out of a token-major matrix: columns
// [col0, col0 + d_model) of rows `row_floats` wide, regrouped per head.  This
// is a third of split_heads and all of merge_heads_backward without the add.
template <int V>
__global__ void head_view_kernel(const float *__restrict__ matrix,
                                 float *__restrict__ view, size_t batch,
                                 size_t seq, size_t d_model, size_t heads,
                                 size_t row_floats, size_t col0) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t head_dim = d_model / heads;
    const size_t total = batch * seq * d_model / V;
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        reinterpret_cast<T *>(view)[i] = reinterpret_cast<const T *>(
            matrix)[token_major_index<V>(i, seq, heads, head_dim, row_floats,
                                         col0)];
    }
}

// patches[row, c*P*P + y*P + x] = image pixel (reference src/ops.c:379-392).
template <int V>
__global__ void extract_patches_kernel(const float *__restrict__ images,
                                       float *__restrict__ patches,
                                       size_t batch, size_t channels,
                                       size_t height, size_t width,
                                       size_t patch) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t per_row = width / patch;
    const size_t per_image = (height / patch) * per_row;
    const size_t elements = channels * patch * patch;
    const size_t total = batch * per_image * elements / V;
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t flat = i * V;
        const size_t row = flat / elements;
        const size_t element = flat % elements;
        const size_t sample = row / per_image;
        const size_t index = row % per_image;
        const size_t channel = element / (patch * patch);
        const size_t y = (index / per_row) * patch + (element / patch) % patch;
        const size_t x = (index % per_row) * patch + element % patch;
        const size_t source =
            ((sample * channels + channel) * height + y) * width + x;
        reinterpret_cast<T *>(patches)[i] =
            *reinterpret_cast<const T *>(images + source);
    }
}

template <int V>
__global__ void token_embedding_kernel(const float *__restrict__ patch_tokens,
                                       const float *__restrict__ cls,
                                       const float *__restrict__ positional,
                                       float *__restrict__ tokens, size_t batch,
                                       size_t seq, size_t d_model) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t row_vectors = d_model / V;
    const size_t total = batch * seq * row_vectors;
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t token = i / row_vectors;
        const size_t col = i % row_vectors;
        const size_t sample = token / seq;
        const size_t position = token % seq;
        const T base = position == 0
            ? reinterpret_cast<const T *>(cls)[col]
            : reinterpret_cast<const T *>(patch_tokens)
                  [(sample * (seq - 1) + position - 1) * row_vectors + col];
        reinterpret_cast<T *>(tokens)[i] = vadd(
            base, reinterpret_cast<const T *>(positional)
                      [position * row_vectors + col]);
    }
}

// patch_grad[b, s-1, :] += tokens_grad[b, s, :] for s >= 1.
template <int V>
__global__ void token_patch_grad_kernel(float *__restrict__ patch_grad,
                                        const float *__restrict__ tokens_grad,
                                        size_t batch, size_t seq,
                                        size_t d_model, bool add) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t row_vectors = d_model / V;
    const size_t patches = seq - 1;
    const size_t total = batch * patches * row_vectors;
    T *destination = reinterpret_cast<T *>(patch_grad);
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t row = i / row_vectors;
        const size_t col = i % row_vectors;
        const size_t sample = row / patches;
        const size_t position = row % patches + 1;
        const T value = reinterpret_cast<const T *>(tokens_grad)
            [(sample * seq + position) * row_vectors + col];
        destination[i] = add ? vadd(destination[i], value) : value;
    }
}

template <int V, bool kAccumulate>
__global__ void gather_rows_kernel(const float *__restrict__ strided,
                                   float *__restrict__ compact,
                                   float *__restrict__ strided_out, size_t rows,
                                   size_t cols, size_t row_stride) {
    grid_dependency_wait();
    grid_dependency_release();
    using T = typename Vec<V>::type;
    const size_t row_vectors = cols / V;
    const size_t total = rows * row_vectors;
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t row = i / row_vectors;
        const size_t col = i % row_vectors;
        const size_t far = row * row_stride * row_vectors + col;
        if (kAccumulate) {
            T *destination = reinterpret_cast<T *>(strided_out);
            destination[far] = vadd(destination[far],
                                    reinterpret_cast<const T *>(compact)[i]);
        } else {
            reinterpret_cast<T *>(compact)[i] =
                reinterpret_cast<const T *>(strided)[far];
        }
    }
}

}  // namespace

#define VITB200_LAUNCH_V(vectorisable, kernel, items, ...)                     \
    do {                                                                       \
        if (vectorisable) {                                                    \
            launch_chained(kernel<4>, stream_grid((items) / 4),                \
                           kStreamThreads, 0, stream, __VA_ARGS__);            \
        } else {                                                               \
            launch_chained(kernel<1>, stream_grid(items), kStreamThreads, 0,   \
                           stream, __VA_ARGS__);                               \
        }                                                                      \
        ++g_kernel_launches;                                                   \
    } while (0)

void launch_head_view(const float *matrix, float *view, size_t batch, size_t seq,
                      size_t d_model, size_t heads, size_t row_floats,
                      size_t col0, cudaStream_t stream) {
    const bool vec = (d_model / heads) % 4 == 0 && row_floats % 4 == 0 &&
                     col0 % 4 == 0;
    VITB200_LAUNCH_V(vec, head_view_kernel, batch * seq * d_model, matrix, view,
                     batch, seq, d_model, heads, row_floats, col0);
}

void launch_split_heads(const float *projected, float *q, float *k, float *v,
                        size_t batch, size_t seq, size_t d_model, size_t heads,
                        cudaStream_t stream) {
    const bool vec = (d_model / heads) % 4 == 0;
    VITB200_LAUNCH_V(vec, split_heads_kernel, batch * seq * d_model, projected,
                     q, k, v, batch, seq, d_model, heads);
}

void launch_split_heads_backward(float *projected_grad, const float *dq,
                                 const float *dk, const float *dv, size_t batch,
                                 size_t seq, size_t d_model, size_t heads,
                                 bool add, cudaStream_t stream) {
    const bool vec = (d_model / heads) % 4 == 0;
    VITB200_LAUNCH_V(vec, split_heads_backward_kernel,
                     batch * seq * 3 * d_model, projected_grad, dq, dk, dv,
                     batch, seq, d_model, heads, add);
}

void launch_merge_heads(const float *attended, float *merged, size_t batch,
                        size_t seq, size_t d_model, size_t heads,
                        cudaStream_t stream) {
    const bool vec = (d_model / heads) % 4 == 0;
    VITB200_LAUNCH_V(vec, merge_heads_kernel, batch * seq * d_model, attended,
                     merged, batch, seq, d_model, heads);
}

void launch_merge_heads_backward(float *attended_grad, const float *merged_grad,
                                 size_t batch, size_t seq, size_t d_model,
                                 size_t heads, bool add, cudaStream_t stream) {
    const bool vec = (d_model / heads) % 4 == 0;
    VITB200_LAUNCH_V(vec, merge_heads_backward_kernel, batch * seq * d_model,
                     attended_grad, merged_grad, batch, seq, d_model, heads,
                     add);
}

void launch_extract_patches(const float *images, float *patches, size_t batch,
                            size_t channels, size_t height, size_t width,
                            size_t patch, cudaStream_t stream) {
    // A 4-float vector must stay inside one patch row and start 16-byte
    // aligned in the image.
    const bool vec = patch % 4 == 0 && width % 4 == 0;
    VITB200_LAUNCH_V(vec, extract_patches_kernel,
                     batch * channels * height * width, images, patches, batch,
                     channels, height, width, patch);
}

void launch_token_embedding(const float *patch_tokens, const float *cls,
                            const float *positional, float *tokens,
                            size_t batch, size_t seq, size_t d_model,
                            cudaStream_t stream) {
    VITB200_LAUNCH_V(d_model % 4 == 0, token_embedding_kernel,
                     batch * seq * d_model, patch_tokens, cls, positional,
                     tokens, batch, seq, d_model);
}

void launch_token_embedding_backward(float *patch_grad, float *cls_grad,
                                     float *positional_grad,
                                     const float *tokens_grad, size_t batch,
                                     size_t seq, size_t d_model, bool add_patch,
                                     cudaStream_t stream) {
    VITB200_LAUNCH_V(d_model % 4 == 0, token_patch_grad_kernel,
                     batch * (seq - 1) * d_model, patch_grad, tokens_grad,
                     batch, seq, d_model, add_patch);
    // Seen as a [batch, seq*d_model] matrix, the positional gradient is the
    // column sum over the batch and the CLS gradient the column sum of its
    // first d_model columns (reference src/ops.c:497-511).
    launch_column_sums(tokens_grad, positional_grad, batch, seq * d_model,
                       seq * d_model, stream);
    launch_column_sums(tokens_grad, cls_grad, batch, d_model, seq * d_model,
                       stream);
}

void launch_gather_rows(const float *source, float *destination, size_t rows,
                        size_t cols, size_t row_stride, cudaStream_t stream) {
    if (cols % 4 == 0) {
        launch_chained(gather_rows_kernel<4, false>,
                       stream_grid(rows * cols / 4), kStreamThreads, 0, stream,
                       source, destination, nullptr, rows, cols, row_stride);
    } else {
        launch_chained(gather_rows_kernel<1, false>, stream_grid(rows * cols),
                       kStreamThreads, 0, stream, source, destination, nullptr,
                       rows, cols, row_stride);
    }
    ++g_kernel_launches;
}

void launch_gather_rows_backward(float *source_grad,
                                 const float *destination_grad, size_t rows,
                                 size_t cols, size_t row_stride,
                                 cudaStream_t stream) {
    if (cols % 4 == 0) {
        launch_chained(gather_rows_kernel<4, true>,
                       stream_grid(rows * cols / 4), kStreamThreads, 0, stream,
                       nullptr, const_cast<float *>(destination_grad),
                       source_grad, rows, cols, row_stride);
    } else {
        launch_chained(gather_rows_kernel<1, true>, stream_grid(rows * cols),
                       kStreamThreads, 0, stream, nullptr,
                       const_cast<float *>(destination_grad), source_grad, rows,
                       cols, row_stride);
    }
    ++g_kernel_launches;
}

}  // namespace vitb200
