/*
 * Binary layout of the host structures that cross the backend boundary.
 *
 * The host program (the reference's unmodified ops.c / vit.c / autodiff.c)
 * hands the backend pointers to its own `Tensor` and `Parameter` objects and
 * copies a table of function pointers by value.  The backend is built without
 * the reference headers, so the layouts are restated here under different
 * names; tests/test_abi_layout.py compiles a translation unit that includes
 * both and compares every size and offset.
 *
 *   vitb200_tensor      <->  Tensor            (reference include/tensor.h:13-25)
 *   vitb200_parameter   <->  Parameter         (reference include/tensor.h:27-34)
 *   vitb200_op_table    <->  OpsDeviceBackend  (reference include/ops.h:21-105)
 *
 * Return convention of every op slot (reference src/ops.c:61-64): 0 = the
 * backend accepted the op (it may still be running), anything else = declined,
 * and the caller then synchronises and runs its own CPU loop.
 */
#ifndef VITB200_HOST_ABI_H
#define VITB200_HOST_ABI_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VITB200_TENSOR_MAX_DIMS 4

typedef void *(*vitb200_allocate_fn)(void *context, size_t bytes);
typedef void (*vitb200_release_fn)(void *context, void *memory);

/* A translation unit that has the host's own headers may define
 * VITB200_HOST_TYPES_ARE_THE_HOSTS after `typedef Tensor vitb200_tensor;
 * typedef Parameter vitb200_parameter;`: the op table below is then declared
 * over the host's types, which lets a compiler compare every slot's signature
 * with the host's (tests/abi_signature_check.c). */
#ifndef VITB200_HOST_TYPES_ARE_THE_HOSTS
typedef struct vitb200_tensor {
    float *data;                               /* values, row-major          */
    float *grad;                               /* same shape as data         */
    size_t ndim;
    size_t shape[VITB200_TENSOR_MAX_DIMS];
    size_t strides[VITB200_TENSOR_MAX_DIMS];
    int owns_memory;
    vitb200_release_fn release_memory;         /* captured at tensor_init    */
    void *release_context;
    size_t rows;                               /* 2-D aliases of shape[0..1] */
    size_t cols;
} vitb200_tensor;

typedef struct vitb200_parameter {
    vitb200_tensor value;
    vitb200_tensor first_moment;
    vitb200_tensor second_moment;
    float *m;                                  /* == first_moment.data       */
    float *v;                                  /* == second_moment.data      */
    size_t step;                               /* incremented by the host    */
} vitb200_parameter;
#endif

typedef struct vitb200_op_table {
    void *context;
    int (*gemm)(void *, const vitb200_tensor *left, const vitb200_tensor *right,
                vitb200_tensor *output);
    int (*gemm_backward)(void *, vitb200_tensor *left, vitb200_tensor *right,
                         const vitb200_tensor *output);
    int (*residual)(void *, const vitb200_tensor *left,
                    const vitb200_tensor *right, vitb200_tensor *output);
    int (*residual_backward)(void *, vitb200_tensor *left, vitb200_tensor *right,
                             const vitb200_tensor *output);
    int (*accumulate_gradient)(void *, vitb200_tensor *destination,
                               const vitb200_tensor *source);
    int (*bias_add)(void *, const vitb200_tensor *input,
                    const vitb200_tensor *bias, vitb200_tensor *output);
    int (*bias_add_backward)(void *, const vitb200_tensor *output,
                             vitb200_tensor *bias_grad);
    int (*layer_norm)(void *, const vitb200_tensor *input,
                      const vitb200_tensor *gamma, const vitb200_tensor *beta,
                      float epsilon, vitb200_tensor *output);
    int (*layer_norm_backward)(void *, const vitb200_tensor *input,
                               const vitb200_tensor *gamma, float epsilon,
                               const vitb200_tensor *output,
                               vitb200_tensor *input_grad,
                               vitb200_tensor *gamma_grad,
                               vitb200_tensor *beta_grad);
    int (*gelu)(void *, const vitb200_tensor *input, vitb200_tensor *output);
    int (*gelu_backward)(void *, const vitb200_tensor *input,
                         const vitb200_tensor *output);
    int (*split_heads)(void *, const vitb200_tensor *projected,
                       vitb200_tensor *query, vitb200_tensor *key,
                       vitb200_tensor *value, size_t batch,
                       size_t sequence_length, size_t d_model, size_t heads);
    int (*split_heads_backward)(void *, vitb200_tensor *projected,
                                const vitb200_tensor *query,
                                const vitb200_tensor *key,
                                const vitb200_tensor *value, size_t batch,
                                size_t sequence_length, size_t d_model,
                                size_t heads);
    int (*merge_heads)(void *, const vitb200_tensor *attended,
                       vitb200_tensor *merged, size_t batch,
                       size_t sequence_length, size_t d_model, size_t heads);
    int (*merge_heads_backward)(void *, vitb200_tensor *attended,
                                const vitb200_tensor *merged, size_t batch,
                                size_t sequence_length, size_t d_model,
                                size_t heads);
    int (*multi_head_attention)(void *, const vitb200_tensor *query,
                                const vitb200_tensor *key,
                                const vitb200_tensor *value, size_t batch,
                                size_t heads, size_t sequence_length,
                                float scale, vitb200_tensor *probabilities,
                                vitb200_tensor *output);
    int (*multi_head_attention_backward)(
        void *, const vitb200_tensor *query, const vitb200_tensor *key,
        const vitb200_tensor *value, size_t batch, size_t heads,
        size_t sequence_length, float scale,
        const vitb200_tensor *probabilities, const vitb200_tensor *output,
        vitb200_tensor *query_grad, vitb200_tensor *key_grad,
        vitb200_tensor *value_grad);
    int (*zero_gradient)(void *, vitb200_tensor *tensor);
    int (*extract_patches)(void *, const vitb200_tensor *images,
                           vitb200_tensor *patches, size_t channels,
                           size_t height, size_t width, size_t patch_size);
    int (*token_embedding)(void *, const vitb200_tensor *patch_tokens,
                           const vitb200_tensor *cls_token,
                           const vitb200_tensor *positional,
                           vitb200_tensor *tokens, size_t batch);
    int (*token_embedding_backward)(void *, vitb200_tensor *patch_tokens,
                                    vitb200_tensor *cls_token,
                                    vitb200_tensor *positional,
                                    const vitb200_tensor *tokens, size_t batch);
    int (*gather_rows)(void *, const vitb200_tensor *source,
                       vitb200_tensor *destination, size_t row_stride);
    int (*gather_rows_backward)(void *, vitb200_tensor *source,
                                const vitb200_tensor *destination,
                                size_t row_stride);
    int (*softmax_cross_entropy)(void *, const vitb200_tensor *logits,
                                 const vitb200_tensor *targets,
                                 const vitb200_tensor *class_weights,
                                 float label_smoothing, vitb200_tensor *loss,
                                 vitb200_tensor *logits_grad);
    int (*clip_gradient_norm)(void *, vitb200_parameter *const *parameters,
                              size_t parameter_count, float max_norm);
    int (*adamw_step)(void *, vitb200_parameter *parameter, float learning_rate,
                      float beta1, float beta2, float epsilon,
                      float weight_decay, float correction1,
                      float correction2);
    int (*zero_gradients)(void *, vitb200_tensor *const *tensors,
                          size_t tensor_count);
    int (*adamw_step_parameters)(void *, vitb200_parameter *const *parameters,
                                 const float *weight_decays,
                                 size_t parameter_count, float learning_rate,
                                 float beta1, float beta2, float epsilon,
                                 float max_gradient_norm);
    void (*synchronize)(void *);
} vitb200_op_table;

#ifdef __cplusplus
}
#endif

#endif
