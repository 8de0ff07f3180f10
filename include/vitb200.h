/*
 * vitb200 — a Blackwell (sm_100a) execution backend for the Vision Transformer
 * training step of transformer-in-c.
 *
 * Part 1 is the drop-in boundary: the five functions the reference's host code
 * already calls (reference include/cuda_backend.h:12-16, implemented there by
 * src/cuda_backend.cu:2015-2091).  A program that used to link
 * build/cuda_backend.o links this library instead and is otherwise unchanged;
 * ops.c keeps dispatching op by op through the table this backend installs
 * with ops_set_device_backend (reference src/ops.c:66-74), and tensors are
 * allocated through the hook installed with tensor_set_allocator
 * (reference src/autodiff.c:11-17).  Those two host functions are looked up
 * at run time, so the library loads on its own as well.
 *
 * Part 2 exposes individual device kernels on plain device pointers; it exists
 * for kernel-level parity tests and for timing a kernel against its roofline.
 *
 * Everything is single-threaded by contract, like the host code it serves
 * (reference include/ops.h:15).
 */
#ifndef VITB200_H
#define VITB200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ part 1 */

typedef struct CudaBackend CudaBackend;

/* Replaces cuda_backend_create (reference src/cuda_backend.cu:2015-2049).
 * 0 = ready; 1 = no usable device (callers treat this as "skip");
 * -1 = error.  The device is cuda:0 unless VITB200_DEVICE (or LOCAL_RANK when
 * VITB200_DEVICE_FROM_RANK=1) selects another one. */
int cuda_backend_create(CudaBackend **backend);

/* Replaces cuda_backend_free (reference src/cuda_backend.cu:2051-2065).
 * NULL-safe; disables device execution first.  Tensors allocated while the
 * backend was enabled stay valid and may be freed afterwards. */
void cuda_backend_free(CudaBackend *backend);

/* Replaces cuda_backend_available (reference src/cuda_backend.cu:2067-2069). */
int cuda_backend_available(const CudaBackend *backend);

/* Replaces cuda_backend_enable_device_execution (reference
 * src/cuda_backend.cu:2071-2081): installs the op table and the allocator.
 * 0 on success, -1 if the backend is unusable or the host's
 * ops_set_device_backend / tensor_set_allocator cannot be found. */
int cuda_backend_enable_device_execution(CudaBackend *backend);

/* Replaces cuda_backend_disable_device_execution (reference
 * src/cuda_backend.cu:2083-2091): synchronises, then uninstalls both hooks.
 * Idempotent. */
void cuda_backend_disable_device_execution(CudaBackend *backend);

/* ---- additions with no counterpart in the reference ---- */

/* Kernels launched by this library since it was loaded. */
unsigned long long vitb200_kernel_launches(void);

/* Coherence counters; any pointer may be NULL. */
void vitb200_memory_counters(size_t *live_allocations, size_t *mirror_bytes,
                             size_t *device_bytes, size_t *h2d_copies,
                             size_t *h2d_bytes, size_t *d2h_copies,
                             size_t *d2h_bytes, size_t *faults);

/* Work the backend avoided: gradient zero fills that became "first writer
 * stores" (or had to be issued after all because the zeros were read), and
 * tensors that were defined but never computed because nobody read them
 * before they were redefined (the attention probability matrix on the FP32
 * short-sequence path), or computed on demand.  Any pointer may be NULL. */
void vitb200_elision_counters(size_t *zero_fills_elided,
                              size_t *zero_fills_materialised,
                              size_t *lazy_defined, size_t *lazy_materialised,
                              size_t *lazy_dropped);

/* Zero fills that had to be written because a kernel needed the zeros in
 * memory: issued one by one as memset nodes in front of that kernel
 * (`memsets`), or found already done by the one launch per
 * ops_zero_gradients call that clears every small gradient buffer
 * (`batched`).  prefetched_reads: host reads served from a copy that was
 * started ahead of time (the loss of a step with the synchronize slot
 * deferred).  Any pointer may be NULL. */
void vitb200_zero_fill_counters(size_t *memsets, size_t *batched,
                                size_t *prefetched_reads);

/* Ops the backend merged into a neighbour since it was created: bias / GELU
 * ops carried by a product's epilogue, head split / merge ops absorbed by the
 * attention kernels, and bias gradients taken from column sums that the
 * producer of the matrix had already accumulated.  Any pointer may be NULL. */
void vitb200_fusion_counters(const CudaBackend *backend,
                             unsigned long long *epilogues,
                             unsigned long long *head_layouts,
                             unsigned long long *bias_gradients);

/* Op-table calls this backend declined since it was created (a slot returned
 * non-zero, so the host synchronised and ran its own CPU loop for that op:
 * reference src/ops.c:61-64).  Zero for any step that ran on the device. */
unsigned long long vitb200_declined_ops(const CudaBackend *backend);

/* Which kernels served the contractions: matrix products launched on the
 * tcgen05 tensor cores (and how many of those with the 128 x 256 tile) or on
 * the FP32 FMA kernel since the library was loaded, and long-sequence
 * attention passes served by the tcgen05 kernels or by the streaming
 * mma.sync kernels since the backend was created.  Any pointer may be NULL. */
void vitb200_kernel_path_counters(const CudaBackend *backend,
                                  unsigned long long *tensor_core_products,
                                  unsigned long long *wide_tile_products,
                                  unsigned long long *fma_products,
                                  unsigned long long *tensor_core_attention,
                                  unsigned long long *streaming_attention);

/* Checkpoints straight from and into device memory, in the host's own file
 * format ("CVITCKP" version 1: reference src/vit.c:1123-1215 writes it,
 * :1217-1268 reads it), so files are interchangeable with vit_model_save /
 * vit_model_load.  `config` is the host's ViTConfig as raw bytes (it is stored
 * verbatim, and on load it must equal the stored one byte for byte, as in the
 * reference's reader); `parameters` lists the model's parameters in the
 * reference's order (src/vit.c:1144-1172: patch projection and bias, class
 * token, positions, then per block the four matrices with their biases and
 * the four normalisation vectors, then final gamma, beta, head and its bias).
 * Values and both Adam moments go device -> page-locked staging -> file (and
 * back) without touching the tensors' host mirrors or their ownership; step
 * counters are host fields.  Loading leaves the tensors device-owned.
 * 0 = success, -1 = failure (I/O error, wrong magic / version /
 * configuration / element count).  vitb200_checkpoint_counters reports, for
 * the last save, the bytes that came from device buffers and from host
 * memory that held the current values. */
struct vitb200_parameter;   /* include/vitb200_host_abi.h; the host's Parameter */
int vitb200_checkpoint_save(CudaBackend *backend, const char *path,
                            const void *config, size_t config_bytes,
                            struct vitb200_parameter *const *parameters,
                            size_t count);
int vitb200_checkpoint_load(CudaBackend *backend, const char *path,
                            const void *config, size_t config_bytes,
                            struct vitb200_parameter *const *parameters,
                            size_t count);
void vitb200_checkpoint_counters(size_t *bytes_from_device,
                                 size_t *bytes_from_host_memory);

/* Makes a tensor buffer obtained through the backend allocator plainly
 * readable and writable by the host (copying it back from the device if
 * needed).  Required before passing it to read()/fread()/write()/fwrite(),
 * which fail with EFAULT on protected pages instead of faulting.  0 / -1. */
int vitb200_make_host_coherent(const void *tensor_memory);

/* Device timing of the work enqueued between begin and end, in milliseconds
 * (CUDA events on the backend's stream).  end() synchronises. */
int vitb200_timer_begin(CudaBackend *backend);
float vitb200_timer_end(CudaBackend *backend);

/* Data parallelism (no counterpart in the reference, which is single-GPU:
 * README.md:229).  One process per GPU, each with its own backend and its own
 * shard of the batch.  Rank 0 obtains 128 id bytes and passes them to the
 * other ranks by any means; every rank then calls vitb200_dp_init
 * (collective).  From then on the optimiser slot all-reduces the parameter
 * gradients (NCCL, FP32 sum, overlapped with the backward pass from the third
 * step on) and applies their mean; the loss each rank reports stays the mean
 * over its own shard.  NCCL (libnccl.so.2) is loaded at this point, not
 * before.  0 on success, -1 on failure. */
int vitb200_dp_unique_id(void *out128);
int vitb200_dp_init(CudaBackend *backend, int rank, int world,
                    const void *id128);
void vitb200_dp_shutdown(CudaBackend *backend);
void vitb200_dp_counters(CudaBackend *backend,
                         unsigned long long *all_reduce_calls,
                         unsigned long long *overlapped_tensors,
                         unsigned long long *late_tensors,
                         unsigned long long *bytes);
/* Contiguous ranges of the gradient arena all-reduced so far: from the third
 * optimiser step on the gradients live in one allocation, ordered as the
 * backward pass completes them, and leave in a few ranges of at least 4 MiB
 * (counted here and in all_reduce_calls) instead of one call per tensor. */
unsigned long long vitb200_dp_flat_ranges(CudaBackend *backend);
/* 0 while the exchange is healthy.  Every synchronise asks NCCL for
 * asynchronous errors (a peer that died, a transport failure); on the first
 * one the communicator is aborted, so this rank's stream drains instead of
 * waiting for the peer, the code is kept and returned here, and the optimiser
 * slot declines from then on (the host must stop training: its gradients are
 * incomplete).  What can be known on the host before a launch -- a rank that
 * never joined, left or stalled -- is the caller's to check first; see
 * ExchangeGroup in transformer-in-c_b200/vit_host.py and INTEGRATION.md. */
int vitb200_dp_status(CudaBackend *backend);

/* Gradient accumulation (no counterpart in the reference, whose train call
 * steps the optimiser after every batch).  Tells the backend that the next
 * ops_adamw_step_parameters calls consume gradients summed over
 * `micro_batches` forward/backward passes (the host zeroes the parameter
 * gradients once, runs the passes, then calls the optimiser once): the factor
 * 1 / micro_batches is folded into the clip scale, like 1 / world, so the norm
 * that is clipped and the update are those of the mean gradient.  With data
 * parallelism each gradient's all-reduce starts when the last micro-batch's
 * op has added to it (after a change of the count the exchange takes two
 * steps to learn the new schedule and runs at the optimiser call meanwhile).
 * To be called between optimiser steps, not between the micro-batches of one.
 * 1 restores plain steps.  0 on success, -1 on a bad argument. */
int vitb200_set_gradient_accumulation(CudaBackend *backend, int micro_batches);

/* What the op table's `synchronize` slot does.  0 (default): it waits for the
 * device, like cuda_backend_synchronize of the reference (src/cuda_backend.cu).
 * 1: it only launches what the backend was holding back and returns.  Results
 * stay correct either way, because every host access to a tensor the device
 * owns is caught (page protection) and waits for what it needs, and the loss
 * of a training step is copied back ahead of time; what changes is that the
 * host code after the slot (the end of one vit_model_train_batch_smoothed and
 * the start of the next: zeroing, the memcpy of the next batch) runs while the
 * device finishes the backward pass and the optimiser step.  A caller that
 * uses `synchronize` to time the device must leave this off or call
 * vitb200_device_busy_ms.  Returns the previous setting, -1 without a device. */
int vitb200_set_deferred_synchronize(CudaBackend *backend, int on);

/* Operand precision of the dense products issued through the op table:
 * VITB200_PRECISION_AUTO (default: TF32 tensor cores for products of at least
 * 16 Mi multiply-adds whose layout TMA can describe, FP32 FMA otherwise),
 * VITB200_PRECISION_FP32 (always FP32 FMA) or VITB200_PRECISION_TF32 (tensor
 * cores wherever the layout allows).  The environment variable VITB200_GEMM
 * (fp32 | tf32) sets the same thing at start-up; -1 returns to it. */
void vitb200_set_gemm_precision(int precision);

/* Every wait inside the tensor-core kernels is bounded; this returns 0, or the
 * code of the first wait that expired (1 producer, 2 MMA issuer, 3 epilogue).
 * Read it after synchronising.  The backend aborts on a non-zero code at its
 * next synchronise. */
int vitb200_tensor_core_status(void);

/* Milliseconds the backend's stream spent between the first kernel after a
 * synchronise and that next synchronise, summed since the last reset (CUDA
 * events; uploads issued before the first kernel are outside the spans).
 * Synchronises. */
double vitb200_device_busy_ms(CudaBackend *backend, int reset);

/* Per-op device timing.  While enabled every op is bracketed by a pair of
 * CUDA events on the backend's stream; entries accumulate per op name with
 * the op's algorithmic HBM bytes and floating-point operations, so a caller
 * can place each op on its roofline.  Enabling clears earlier entries. */
void vitb200_profile_enable(CudaBackend *backend, int on);
size_t vitb200_profile_entries(CudaBackend *backend);
int vitb200_profile_entry(CudaBackend *backend, size_t index, const char **name,
                          unsigned long long *calls, double *milliseconds,
                          double *bytes, double *flops);

/* ------------------------------------------------------------------ part 2 */
/* Every function below takes device pointers, enqueues on the given CUDA
 * stream handle (a cudaStream_t passed as void*, NULL = default stream) and
 * returns 0, or -1 for arguments the kernel does not support.  Semantics are
 * those of the like-named host op (reference src/ops.c), including "+=" into
 * gradient buffers. */

int vitb200_k_gemm(const float *x, const float *w, float *y, size_t m,
                   size_t k, size_t n, int precision, void *stream);
/* Forward product with what the host issues right after it folded into the
 * epilogue: y = x w (+ bias), and optionally gelu_out = gelu(y) or
 * residual_out = residual + y (not both).  Unused pointers are NULL. */
int vitb200_k_gemm_fused(const float *x, const float *w, float *y,
                         const float *bias, float *gelu_out,
                         const float *residual, float *residual_out, size_t m,
                         size_t k, size_t n, int precision, void *stream);
int vitb200_k_gemm_backward(const float *x, const float *w, const float *dy,
                            float *dx, float *dw, size_t m, size_t k, size_t n,
                            int precision, void *stream);
/* The input half of vitb200_k_gemm_backward followed by
 * vitb200_k_gelu_backward, for a layer whose input was gelu(gelu_input), as
 * one tensor-core kernel:
 *   d_gelu_input[m,k] = (dy[m,n] w[k,n]^T) * gelu'(gelu_input[m,k])
 * (stored, not added; the gradient of the layer's input itself is not
 * written).  column_partials, optional, receives
 * VITB200_GEMM_PARTIAL_ROWS rows of k floats whose column-wise sum is the
 * column sum of d_gelu_input (the bias gradient of the layer before the
 * GELU).  Returns -1, with nothing done, when the precision selector or the
 * shape keeps the product off the tensor cores. */
#define VITB200_GEMM_PARTIAL_ROWS 296
int vitb200_k_gemm_backward_gelu(const float *w, const float *dy,
                                 const float *gelu_input, float *d_gelu_input,
                                 float *column_partials, size_t m, size_t k,
                                 size_t n, int precision, void *stream);
int vitb200_k_bias_add(const float *in, const float *bias, float *out,
                       size_t rows, size_t cols, void *stream);
int vitb200_k_column_sums(const float *in, float *out, size_t rows,
                          size_t cols, void *stream);
int vitb200_k_layer_norm(const float *x, const float *gamma, const float *beta,
                         float epsilon, float *y, size_t rows, size_t cols,
                         void *stream);
int vitb200_k_layer_norm_backward(const float *x, const float *gamma,
                                  float epsilon, const float *dy, float *dx,
                                  float *dgamma, float *dbeta, size_t rows,
                                  size_t cols, void *stream);
int vitb200_k_gelu(const float *in, float *out, size_t n, void *stream);
int vitb200_k_gelu_backward(const float *x, const float *dy, float *dx,
                            size_t n, void *stream);
/* probabilities may be NULL for seq <= 128 (FP32; head_dim 8, 16, 32, 64) or
 * seq <= 64 (TF32; head_dim 16, 32): P then stays on chip in the forward pass
 * and is rebuilt from Q and K in the backward pass (row_dots unused).  -1 if
 * the shape has no such kernel. */
int vitb200_k_attention(const float *q, const float *k, const float *v,
                        float *probabilities, float *out, size_t groups,
                        size_t seq, size_t head_dim, float scale, int precision,
                        void *stream);
/* Flash attention on tensor cores (TF32 operands) for any sequence length and
 * head_dim 16, 32 or 64: P is never materialised.  The forward pass leaves
 * each row's log-sum-exp in `lse` (groups*seq floats, an opaque input of the
 * backward pass); row_dots is scratch of the same size.  The backward pass
 * adds into dq, dk, dv.  -1 if head_dim has no such kernel. */
int vitb200_k_attention_stream(const float *q, const float *k, const float *v,
                               float *out, float *lse, size_t groups,
                               size_t seq, size_t head_dim, float scale,
                               void *stream);
int vitb200_k_attention_stream_backward(const float *q, const float *k,
                                        const float *v, const float *out,
                                        const float *dout, const float *lse,
                                        float *dq, float *dk, float *dv,
                                        float *row_dots, size_t groups,
                                        size_t seq, size_t head_dim, float scale,
                                        void *stream);
/* The same flash attention on the tcgen05 tensor cores (128-row tiles, scores
 * and P in tensor memory, operands fetched by TMA; TF32 operands, FP32
 * accumulation and softmax), head_dim 32 or 64, any sequence length.  Replaces
 * attention_forward_flash / attention_backward_flash_{queries,keys} of the
 * reference backend (src/cuda_backend.cu:532-723; host loops src/ops.c:1297-1355,
 * 1381-1441).  `lse` and `row_dots` as above; the two families' `lse` rows are
 * interchangeable.  ld = 0: head-major tensors.  ld != 0: each operand is a block of
 * heads * head_dim columns of a token-major matrix with rows `ld` floats apart
 * (q, k, v: in_ld; out and dout: out_ld; dq, dk, dv: grad_ld), the pointer
 * naming the block's first column, groups = samples * heads.  The backward
 * pass adds into dq, dk, dv when `accumulate` is non-zero and overwrites them
 * otherwise.  -1: shape, alignment (16 bytes, ld a multiple of 4) or layout
 * not covered; nothing was launched. */
int vitb200_k_attention_tc(const float *q, const float *k, const float *v,
                           float *out, float *lse, size_t groups, size_t seq,
                           size_t head_dim, float scale, size_t in_ld,
                           size_t out_ld, size_t heads, void *stream);
int vitb200_k_attention_tc_backward(const float *q, const float *k,
                                    const float *v, const float *out,
                                    const float *dout, const float *lse,
                                    float *dq, float *dk, float *dv,
                                    float *row_dots, size_t groups, size_t seq,
                                    size_t head_dim, float scale, int accumulate,
                                    size_t in_ld, size_t out_ld, size_t grad_ld,
                                    size_t heads, void *stream);
/* row_dots: scratch, groups*seq floats. */
int vitb200_k_attention_backward(const float *q, const float *k, const float *v,
                                 const float *probabilities, const float *out,
                                 const float *dout, float *dq, float *dk,
                                 float *dv, float *row_dots, size_t groups,
                                 size_t seq, size_t head_dim, float scale,
                                 int precision, void *stream);
/* Shared-memory layout of the staged 64-row operand tiles of the tensor-core
 * attention kernels (head dimensions 16, 32, 64), computed on the host by the
 * code the kernels use: the float offset of element (row, col), and column e of
 * the head-dimension slice lane t (0..3) of a quad contracts over.  No device
 * needed; for checking that the layout is a bijection and that the kernels'
 * fragment loads meet no bank conflict.  -1 for arguments out of range. */
int vitb200_attention_tile_index(int head_dim, int row, int col);
int vitb200_attention_lane_column(int head_dim, int t, int e);
/* row_losses: scratch, rows floats. */
int vitb200_k_softmax_cross_entropy(const float *logits, const float *targets,
                                    const float *class_weights,
                                    float label_smoothing, float *loss,
                                    float *logits_grad, float *row_losses,
                                    size_t rows, size_t cols, void *stream);

/* No counterpart in the reference.  The same loss and gradient as
 * vitb200_k_softmax_cross_entropy, for callers that must not trigger a device
 * allocation: a latency-sensitive serving or training loop in which a
 * cudaMalloc would stall every stream of the device, a plug-in running under a
 * host that has handed out its whole memory budget up front, or code that is
 * not allowed to call the CUDA allocator at all.  The per-row scratch lives in
 * a fixed 256 KiB array inside the library (each GPU that loads the library
 * holds it until the process ends), so rows is limited to 65536; more rows
 * return -2 and print why.  The caller still owns every input and output.
 * The first call on a device looks the array's address up once
 * (cudaGetSymbolAddress); make that call outside any stream capture.  All
 * calls share the one array: two calls whose kernels may overlap on the GPU
 * (different streams without ordering) race on it.  The array keeps whatever
 * the previous call left, which is harmless: each call overwrites every entry
 * it later reads.  Never calls cudaMalloc, cudaFree or an allocating library
 * routine.  Returns 0 on success, -1 on other errors. */
int vitb200_k_softmax_cross_entropy_static(
    const float *logits, const float *targets, const float *class_weights,
    float label_smoothing, float *loss, float *logits_grad, size_t rows,
    size_t cols, void *stream);

/* GEMM operand precision selectors for part 2 and VITB200_GEMM. */
#define VITB200_PRECISION_AUTO 0  /* backend default for the shape          */
#define VITB200_PRECISION_FP32 1  /* FP32 FMA                                */
#define VITB200_PRECISION_TF32 2  /* tcgen05 kind::tf32, FP32 accumulate     */

#ifdef __cplusplus
}
#endif

#endif
