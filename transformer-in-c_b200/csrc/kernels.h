// Launchers for the device kernels.  Every function takes plain device
// pointers and enqueues on `stream`; none of them allocates or synchronises.
// Each launcher adds the number of kernels it started to g_kernel_launches.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace vitb200 {

extern unsigned long long g_kernel_launches;

// ---- elementwise (elementwise.cu) ----------------------------------------
void launch_add(const float *a, const float *b, float *out, size_t n,
                cudaStream_t stream);                       // out = a + b
// The accumulating launchers take `add` flags: true is the host op's "+=",
// false stores the increment (used when the destination is known to be zero,
// which saves reading it and lets the zero fill be skipped altogether).
void launch_accumulate(float *dst, const float *src, size_t n, bool add,
                       cudaStream_t stream);                // dst (+)= src
void launch_accumulate2(float *dst_a, float *dst_b, const float *src, size_t n,
                        bool add_a, bool add_b,
                        cudaStream_t stream);               // both (+)= src
void launch_bias_add(const float *in, const float *bias, float *out,
                     size_t rows, size_t cols, cudaStream_t stream);
void launch_gelu(const float *in, float *out, size_t n, cudaStream_t stream);
void launch_gelu_backward(const float *x, const float *dy, float *dx, size_t n,
                          bool add, cudaStream_t stream);
// gelu_backward that also leaves partial column sums of dx ([rows, cols]) in
// `partials`, one row of `cols` floats per block
// (gelu_backward_sums_blocks(rows, cols) of them; their column sums are
// dx's); only for widths gelu_backward_sums_supported accepts.
bool gelu_backward_sums_supported(size_t cols);
size_t gelu_backward_sums_blocks(size_t rows, size_t cols);
void launch_gelu_backward_sums(const float *x, const float *dy, float *dx,
                               float *partials, size_t rows, size_t cols,
                               bool add, cudaStream_t stream);
// out (+)= sums; sums = 0.
void launch_take_column_sums(float *out, float *sums, size_t cols, bool add,
                             cudaStream_t stream);   // dx (+)= dy*gelu'(x)
void launch_scale_by_device_scalar(float *values, size_t n, const float *scale,
                                   cudaStream_t stream);

// ---- layout (layout.cu) ---------------------------------------------------
void launch_split_heads(const float *projected, float *q, float *k, float *v,
                        size_t batch, size_t seq, size_t d_model, size_t heads,
                        cudaStream_t stream);
void launch_split_heads_backward(float *projected_grad, const float *dq,
                                 const float *dk, const float *dv, size_t batch,
                                 size_t seq, size_t d_model, size_t heads,
                                 bool add, cudaStream_t stream);
void launch_merge_heads(const float *attended, float *merged, size_t batch,
                        size_t seq, size_t d_model, size_t heads,
                        cudaStream_t stream);
void launch_merge_heads_backward(float *attended_grad, const float *merged_grad,
                                 size_t batch, size_t seq, size_t d_model,
                                 size_t heads, bool add, cudaStream_t stream);
// view = columns [col0, col0 + d_model) of a [batch*seq, row_floats] matrix in
// head-major order ([batch*heads*seq, d_model/heads]).
void launch_head_view(const float *matrix, float *view, size_t batch, size_t seq,
                      size_t d_model, size_t heads, size_t row_floats,
                      size_t col0, cudaStream_t stream);
void launch_extract_patches(const float *images, float *patches, size_t batch,
                            size_t channels, size_t height, size_t width,
                            size_t patch, cudaStream_t stream);
void launch_token_embedding(const float *patch_tokens, const float *cls,
                            const float *positional, float *tokens,
                            size_t batch, size_t seq, size_t d_model,
                            cudaStream_t stream);
void launch_token_embedding_backward(float *patch_grad, float *cls_grad,
                                     float *positional_grad,
                                     const float *tokens_grad, size_t batch,
                                     size_t seq, size_t d_model, bool add_patch,
                                     cudaStream_t stream);
void launch_gather_rows(const float *source, float *destination, size_t rows,
                        size_t cols, size_t row_stride, cudaStream_t stream);
void launch_gather_rows_backward(float *source_grad,
                                 const float *destination_grad, size_t rows,
                                 size_t cols, size_t row_stride,
                                 cudaStream_t stream);

// Up to kColumnSumBatch small column sums in one launch: destination[c] (+)=
// sum over rows of source[r * cols + c].  cols a multiple of 4, both pointers
// 16-byte aligned, rows small (every job is served by cols / 128 blocks).
// clear: the source is zeroed afterwards.
struct ColumnSumJob {
    const float *source;
    float *destination;
    unsigned rows, cols;
    int add, clear;
};
constexpr int kColumnSumBatch = 8;
void launch_column_sums_batch(const ColumnSumJob *jobs, int count,
                              cudaStream_t stream);
// ---- reductions over rows (reduce.cu) ------------------------------------
// out[c] += sum_r in[r * ld + c] for c < cols.
void launch_column_sums(const float *in, float *out, size_t rows, size_t cols,
                        size_t ld, cudaStream_t stream);

// ---- layer norm (layernorm.cu) -------------------------------------------
// With `addend` (only for widths layer_norm_takes_addend accepts) the input
// is x + addend, which is also written to `sum`.
bool layer_norm_takes_addend(size_t cols);
void launch_layer_norm(const float *x, const float *gamma, const float *beta,
                       float epsilon, float *y, size_t rows, size_t cols,
                       cudaStream_t stream, const float *addend = nullptr,
                       float *sum = nullptr);
// dx += ...; dgamma += ...; dbeta += ...   (all accumulate)
void launch_layer_norm_backward(const float *x, const float *gamma,
                                float epsilon, const float *dy, float *dx,
                                float *dgamma, float *dbeta, size_t rows,
                                size_t cols, const float *base, float *dx_sums,
                                cudaStream_t stream);

// ---- attention (attention.cu) --------------------------------------------
// q, k, v, out: [groups * seq, head_dim]; probabilities: [groups * seq, seq].
// precision: a VITB200_PRECISION_* selector (FP32 kernels, or TF32 tensor
// cores in attention_mma.cu).
void launch_attention_forward(const float *q, const float *k, const float *v,
                              float *probabilities, float *out, size_t groups,
                              size_t seq, size_t head_dim, float scale,
                              int precision, cudaStream_t stream);
// out / dout: forward result and its gradient; row_dots: scratch of
// groups * seq floats.  dq, dk, dv accumulate.
void launch_attention_backward(const float *q, const float *k, const float *v,
                               const float *probabilities, const float *out,
                               const float *dout, float *dq, float *dk,
                               float *dv, float *row_dots, size_t groups,
                               size_t seq, size_t head_dim, float scale,
                               bool add_q, bool add_k, bool add_v,
                               int precision, cudaStream_t stream);

// Tensor-core kernels (attention_mma.cu); false = shape not covered.
bool attention_mma_supported(size_t head_dim);
bool launch_attention_mma_forward(const float *q, const float *k,
                                  const float *v, float *probabilities,
                                  float *out, size_t groups, size_t seq,
                                  size_t head_dim, float scale,
                                  cudaStream_t stream);
// One sweep, no probability matrix: writes O and the row log-sum-exp.
bool launch_attention_mma_flash_forward(const float *q, const float *k,
                                        const float *v, float *out, float *lse,
                                        size_t groups, size_t seq,
                                        size_t head_dim, float scale,
                                        cudaStream_t stream);
// lse == nullptr: read `probabilities`; otherwise rebuild them from Q, K, lse.
bool launch_attention_mma_backward(const float *q, const float *k,
                                   const float *v, const float *probabilities,
                                   const float *lse, const float *out,
                                   const float *dout, float *dq, float *dk,
                                   float *dv, float *row_dots, size_t groups,
                                   size_t seq, size_t head_dim, float scale,
                                   bool add_q, bool add_k, bool add_v,
                                   cudaStream_t stream);

// Short sequences with the whole (sample, head) group in shared memory
// (attention_small.cu).  The launchers return false when the shape is outside
// what they cover; the tiled kernels above take over then.
bool attention_small_supported(size_t seq, size_t head_dim);
// Where the rows of a (sample, head) group live.  Row t of group g starts
// (g / heads) * seq * ld + (g % heads) * head_dim + t * ld floats after the
// base pointer: {ld, heads} addresses one head's columns inside a token-major
// [batch*seq, ld] matrix (the base pointer already includes the first
// column), and the default {0, 1} means "stored group by group".
struct HeadLayout {
    int ld = 0;
    int heads = 1;
};
bool launch_attention_small_forward(const float *q, const float *k,
                                    const float *v, float *probabilities,
                                    float *out, size_t groups, size_t seq,
                                    size_t head_dim, float scale, bool write_p,
                                    bool write_o, cudaStream_t stream,
                                    HeadLayout in_layout = HeadLayout(),
                                    HeadLayout out_layout = HeadLayout());
// Tensor-core kernels for seq <= 64 and head_dim 16 or 32 (TF32 operands); P
// is neither written nor read.  With grad_layout = {3 * d_model, heads} (dq, dk,
// dv pointing at the three column blocks of the projected gradient),
// column_partials ([groups / heads, 3 * d_model]) receives per-sample column
// sums of that gradient: summed over its rows they are the bias gradient.
bool attention_warp_supported(size_t seq, size_t head_dim);
// Host copies of the shared-memory layout of the tensor-core attention
// kernels' staged tiles, for checking it without a device: the float offset of
// element (row, col) of a 64-row tile, and column e of the head-dimension
// slice that lane t of a quad contracts over.  -1 for other head dimensions.
int attention_tile_index(int head_dim, int row, int col);
int attention_lane_column(int head_dim, int t, int e);
bool launch_attention_warp_forward(const float *q, const float *k,
                                   const float *v, float *out, size_t groups,
                                   size_t seq, size_t head_dim, float scale,
                                   cudaStream_t stream,
                                   HeadLayout in_layout = HeadLayout(),
                                   HeadLayout out_layout = HeadLayout());
bool launch_attention_warp_backward(const float *q, const float *k,
                                    const float *v, const float *out,
                                    const float *dout, float *dq, float *dk,
                                    float *dv, size_t groups, size_t seq,
                                    size_t head_dim, float scale, bool add_q,
                                    bool add_k, bool add_v, cudaStream_t stream,
                                    HeadLayout in_layout = HeadLayout(),
                                    HeadLayout out_layout = HeadLayout(),
                                    HeadLayout dout_layout = HeadLayout(),
                                    HeadLayout grad_layout = HeadLayout(),
                                    float *column_partials = nullptr);
// The same register-resident products streamed over 64-row tiles, for any
// sequence length and head_dim 16, 32 or 64.  The forward pass saves each
// row's log-sum-exp (base 2, of the scaled scores; groups * seq floats) for
// the backward pass, which also wants groups * seq floats of scratch.
bool attention_stream_supported(size_t head_dim);
bool launch_attention_stream_forward(const float *q, const float *k,
                                     const float *v, float *out, float *lse,
                                     size_t groups, size_t seq, size_t head_dim,
                                     float scale, cudaStream_t stream,
                                     HeadLayout in_layout = HeadLayout(),
                                     HeadLayout out_layout = HeadLayout());
bool launch_attention_stream_backward(const float *q, const float *k,
                                      const float *v, const float *out,
                                      const float *dout, const float *lse,
                                      float *dq, float *dk, float *dv,
                                      float *row_dots, size_t groups, size_t seq,
                                      size_t head_dim, float scale, bool add_q,
                                      bool add_k, bool add_v,
                                      cudaStream_t stream,
                                      HeadLayout in_layout = HeadLayout(),
                                      HeadLayout out_layout = HeadLayout(),
                                      HeadLayout dout_layout = HeadLayout(),
                                      HeadLayout grad_layout = HeadLayout());
// The same computation on the tcgen05 tensor cores (attention_tc.cu): 128-row
// tiles, scores in tensor memory, operands by TMA; head_dim 32 or 64, any
// sequence length (meant for seq >= 128).  Same log-sum-exp convention as the
// streaming kernels, so either backward pass accepts either forward pass's
// rows.  False = shape, alignment or layout not covered (nothing launched).
bool attention_tc_supported(size_t seq, size_t head_dim);
bool launch_attention_tc_forward(const float *q, const float *k, const float *v,
                                 float *out, float *lse, size_t groups,
                                 size_t seq, size_t head_dim, float scale,
                                 cudaStream_t stream,
                                 HeadLayout in_layout = HeadLayout(),
                                 HeadLayout out_layout = HeadLayout());
bool launch_attention_tc_backward(const float *q, const float *k, const float *v,
                                  const float *out, const float *dout,
                                  const float *lse, float *dq, float *dk,
                                  float *dv, float *row_dots, size_t groups,
                                  size_t seq, size_t head_dim, float scale,
                                  bool add_q, bool add_k, bool add_v,
                                  cudaStream_t stream,
                                  HeadLayout in_layout = HeadLayout(),
                                  HeadLayout out_layout = HeadLayout(),
                                  HeadLayout dout_layout = HeadLayout(),
                                  HeadLayout grad_layout = HeadLayout(),
                                  float *column_partials = nullptr);
// column_partials (optional, token-major gradients that are overwritten): the
// kernels leave attention_tc_partial_rows() rows of 3 * heads * head_dim
// column sums of what they wrote, in the order [dQ | dK | dV] of the projected
// gradient; their column sums are the column sums of that gradient.
size_t attention_tc_partial_rows();
// recompute = true: `probabilities` is not read; P is rebuilt from Q and K.
bool launch_attention_small_backward(const float *q, const float *k,
                                     const float *v, const float *probabilities,
                                     const float *out, const float *dout,
                                     float *dq, float *dk, float *dv,
                                     size_t groups, size_t seq, size_t head_dim,
                                     float scale, bool add_q, bool add_k,
                                     bool add_v, bool recompute,
                                     cudaStream_t stream,
                                     HeadLayout in_layout = HeadLayout(),
                                     HeadLayout out_layout = HeadLayout(),
                                     HeadLayout dout_layout = HeadLayout(),
                                     HeadLayout grad_layout = HeadLayout());

// ---- loss (loss.cu) -------------------------------------------------------
// row_losses: scratch of `rows` floats.
void launch_softmax_cross_entropy(const float *logits, const float *targets,
                                  const float *class_weights,
                                  float label_smoothing, float *loss,
                                  float *logits_grad, float *row_losses,
                                  size_t rows, size_t cols,
                                  cudaStream_t stream);

// Same computation with the row-loss scratch in a fixed array inside the
// library (no allocation anywhere); at most kStaticLossMaxRows rows.
// Returns 0, -2 if rows exceeds the limit, -1 on other errors.
constexpr size_t kStaticLossMaxRows = 65536;
int launch_softmax_cross_entropy_static(const float *logits,
                                        const float *targets,
                                        const float *class_weights,
                                        float label_smoothing, float *loss,
                                        float *logits_grad, size_t rows,
                                        size_t cols, cudaStream_t stream);

// ---- optimiser (optimizer.cu) --------------------------------------------
struct ParameterSlice {
    float *value;
    float *grad;
    float *m;
    float *v;
    unsigned long long count;
    unsigned long long first_block;  // prefix sum of blocks before this slice
    float weight_decay;
    float correction1;
    float correction2;
    float pad;
};
constexpr unsigned kSliceBlockElements = 4096;

// partials: scratch of total_blocks floats; scale_out: 1 float.  The gradients
// are taken to be sums over 1/inverse_world ranks (1 for a single GPU).
void launch_gradient_clip_scale(const ParameterSlice *slices, unsigned slices_n,
                                unsigned total_blocks, float max_norm,
                                float inverse_world, float *partials,
                                float *scale_out, cudaStream_t stream);
void launch_scale_gradients(const ParameterSlice *slices, unsigned slices_n,
                            unsigned total_blocks, const float *scale,
                            cudaStream_t stream);
// scale may be nullptr (no clipping).  Zeroes the gradients afterwards.
void launch_adamw(const ParameterSlice *slices, unsigned slices_n,
                  unsigned total_blocks, const float *scale, float lr,
                  float beta1, float beta2, float epsilon, cudaStream_t stream);
void launch_adamw_single(float *value, float *grad, float *m, float *v,
                         size_t n, float lr, float beta1, float beta2,
                         float epsilon, float weight_decay, float correction1,
                         float correction2, cudaStream_t stream);

// ---- dense products (gemm_simt.cu, gemm_tc.cu) ---------------------------
// C[M,N] (+)= A[M,K] * B[K,N] with arbitrary element strides, FP32 FMA.
struct GemmOperands {
    const float *a;
    long long a_row, a_col;  // strides, in elements, of A(m,k)
    const float *b;
    long long b_row, b_col;  // strides of B(k,n)
    float *c;
    long long c_row;         // C is always unit stride along n
    int m, n, k;
    int accumulate;          // 0: C = AB, 1: C += AB
};
void launch_gemm_simt(const GemmOperands &operands, cudaStream_t stream);

}  // namespace vitb200
