/* Compiled by tests/test_abi_layout.py with -I<reference>/include -I<repo>/include.
 * The op table of include/vitb200_host_abi.h is declared here over the host's
 * own Tensor / Parameter types (whose layouts tests/abi_layout_check.c pins to
 * the mirrored structs), so each slot's function-pointer type can be compared
 * with the host's (reference include/ops.h:21-105) by the compiler itself:
 * any difference in arity, argument type, constness or return type fails. */
#include "ops.h"
#include "tensor.h"

typedef Tensor vitb200_tensor;
typedef Parameter vitb200_parameter;
#define VITB200_HOST_TYPES_ARE_THE_HOSTS
#include "vitb200_host_abi.h"

#define SAME_SIGNATURE(slot)                                                    \
    _Static_assert(__builtin_types_compatible_p(                                \
                       __typeof__(((OpsDeviceBackend *)0)->slot),               \
                       __typeof__(((vitb200_op_table *)0)->slot)),              \
                   "signature of " #slot)

SAME_SIGNATURE(context); SAME_SIGNATURE(gemm); SAME_SIGNATURE(gemm_backward);
SAME_SIGNATURE(residual); SAME_SIGNATURE(residual_backward);
SAME_SIGNATURE(accumulate_gradient); SAME_SIGNATURE(bias_add);
SAME_SIGNATURE(bias_add_backward); SAME_SIGNATURE(layer_norm);
SAME_SIGNATURE(layer_norm_backward); SAME_SIGNATURE(gelu);
SAME_SIGNATURE(gelu_backward); SAME_SIGNATURE(split_heads);
SAME_SIGNATURE(split_heads_backward); SAME_SIGNATURE(merge_heads);
SAME_SIGNATURE(merge_heads_backward); SAME_SIGNATURE(multi_head_attention);
SAME_SIGNATURE(multi_head_attention_backward); SAME_SIGNATURE(zero_gradient);
SAME_SIGNATURE(extract_patches); SAME_SIGNATURE(token_embedding);
SAME_SIGNATURE(token_embedding_backward); SAME_SIGNATURE(gather_rows);
SAME_SIGNATURE(gather_rows_backward); SAME_SIGNATURE(softmax_cross_entropy);
SAME_SIGNATURE(clip_gradient_norm); SAME_SIGNATURE(adamw_step);
SAME_SIGNATURE(zero_gradients); SAME_SIGNATURE(adamw_step_parameters);
SAME_SIGNATURE(synchronize);

/* The allocator hook pair (reference include/tensor.h:10-11, 36-37). */
_Static_assert(__builtin_types_compatible_p(TensorAllocateFunction,
                                            vitb200_allocate_fn),
               "allocator signature");
_Static_assert(__builtin_types_compatible_p(TensorReleaseFunction,
                                            vitb200_release_fn),
               "release signature");

int main(void) {
    return 0;
}
