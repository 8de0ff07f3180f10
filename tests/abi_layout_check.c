/* Compiled by tests/test_abi_layout.py with -I<reference>/include -I<repo>/include.
 * Fails to compile if the mirrored structures drift from the host's. */
#include "ops.h"
#include "tensor.h"
#include "vitb200_host_abi.h"
#include "augmentation.h"
#include "vitb200_augmentation.h"

#include <stddef.h>

#define SAME_SIZE(a, b) _Static_assert(sizeof(a) == sizeof(b), "size " #a)
#define SAME_FIELD(a, fa, b, fb) \
    _Static_assert(offsetof(a, fa) == offsetof(b, fb), "offset " #a "." #fa)

SAME_SIZE(Tensor, vitb200_tensor);
SAME_FIELD(Tensor, data, vitb200_tensor, data);
SAME_FIELD(Tensor, grad, vitb200_tensor, grad);
SAME_FIELD(Tensor, ndim, vitb200_tensor, ndim);
SAME_FIELD(Tensor, shape, vitb200_tensor, shape);
SAME_FIELD(Tensor, strides, vitb200_tensor, strides);
SAME_FIELD(Tensor, owns_memory, vitb200_tensor, owns_memory);
SAME_FIELD(Tensor, release_memory, vitb200_tensor, release_memory);
SAME_FIELD(Tensor, release_context, vitb200_tensor, release_context);
SAME_FIELD(Tensor, rows, vitb200_tensor, rows);
SAME_FIELD(Tensor, cols, vitb200_tensor, cols);

SAME_SIZE(Parameter, vitb200_parameter);
SAME_FIELD(Parameter, value, vitb200_parameter, value);
SAME_FIELD(Parameter, first_moment, vitb200_parameter, first_moment);
SAME_FIELD(Parameter, second_moment, vitb200_parameter, second_moment);
SAME_FIELD(Parameter, m, vitb200_parameter, m);
SAME_FIELD(Parameter, v, vitb200_parameter, v);
SAME_FIELD(Parameter, step, vitb200_parameter, step);

SAME_SIZE(OpsDeviceBackend, vitb200_op_table);
#define SLOT(name) SAME_FIELD(OpsDeviceBackend, name, vitb200_op_table, name)
SLOT(context); SLOT(gemm); SLOT(gemm_backward); SLOT(residual);
SLOT(residual_backward); SLOT(accumulate_gradient); SLOT(bias_add);
SLOT(bias_add_backward); SLOT(layer_norm); SLOT(layer_norm_backward);
SLOT(gelu); SLOT(gelu_backward); SLOT(split_heads); SLOT(split_heads_backward);
SLOT(merge_heads); SLOT(merge_heads_backward); SLOT(multi_head_attention);
SLOT(multi_head_attention_backward); SLOT(zero_gradient); SLOT(extract_patches);
SLOT(token_embedding); SLOT(token_embedding_backward); SLOT(gather_rows);
SLOT(gather_rows_backward); SLOT(softmax_cross_entropy);
SLOT(clip_gradient_norm); SLOT(adamw_step); SLOT(zero_gradients);
SLOT(adamw_step_parameters); SLOT(synchronize);

SAME_SIZE(DataAugmentation, vitb200_augmentation);
#define AUGMENTATION_FIELD(f) \
    SAME_FIELD(DataAugmentation, f, vitb200_augmentation, f)
AUGMENTATION_FIELD(max_shift_pixels); AUGMENTATION_FIELD(max_rotation_degrees);
AUGMENTATION_FIELD(max_scale_delta); AUGMENTATION_FIELD(max_brightness_delta);
AUGMENTATION_FIELD(max_contrast_delta);
AUGMENTATION_FIELD(noise_standard_deviation);
AUGMENTATION_FIELD(erasing_probability);
AUGMENTATION_FIELD(erasing_max_side_fraction);
AUGMENTATION_FIELD(erasing_value); AUGMENTATION_FIELD(minimum_value);
AUGMENTATION_FIELD(maximum_value);

/* The slots' signatures are compared in tests/abi_signature_check.c. */
int main(void) {
    return 0;
}
