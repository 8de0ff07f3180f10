/*
 * Batch augmentation on the B200: drop-in counterparts of the reference's
 * include/augmentation.h for callers that hold a vitb200 backend.
 *
 * Same arguments, same validation and return values, same sequence of random
 * draws (so *random_state ends where the reference leaves it and a run can
 * switch between the two implementations at any batch), same arithmetic; the
 * only values that can differ from the reference's are those that pass
 * through logf / cosf in the Gaussian noise (device libm instead of the
 * host's: about 1e-7 of the noise amplitude).
 *
 * `source` and `destination` may be ordinary host memory (copied to and from
 * the device inside the call, which then returns with the result in place) or
 * tensor memory obtained through the backend's allocator (used where it is,
 * the call returns with the work enqueued; ops_synchronize or a host access
 * makes the result visible, as for any other op).
 */
#ifndef VITB200_AUGMENTATION_H
#define VITB200_AUGMENTATION_H

#include <stddef.h>
#include <stdint.h>

#include "vitb200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Layout of the reference's DataAugmentation (include/augmentation.h:7-19). */
typedef struct {
    float max_shift_pixels;
    float max_rotation_degrees;
    float max_scale_delta;
    float max_brightness_delta;
    float max_contrast_delta;
    float noise_standard_deviation;
    float erasing_probability;
    float erasing_max_side_fraction;
    float erasing_value;
    float minimum_value;
    float maximum_value;
} vitb200_augmentation;

/* data_augmentation_enabled (include/augmentation.h:21). */
int vitb200_data_augmentation_enabled(const vitb200_augmentation *augmentation);

/* data_augmentation_apply (include/augmentation.h:23-26): 0 on success, -1 on
 * invalid arguments (the reference's checks, src/augmentation.c:182-198, plus
 * a NULL or disabled backend). */
int vitb200_data_augmentation_apply(CudaBackend *backend,
                                    const vitb200_augmentation *augmentation,
                                    uint64_t *random_state, const float *source,
                                    float *destination, size_t batch,
                                    size_t channels, size_t height,
                                    size_t width);

/* data_augmentation_translate (include/augmentation.h:28-30). */
int vitb200_data_augmentation_translate(CudaBackend *backend,
                                        const float *source, float *destination,
                                        size_t batch, size_t channels,
                                        size_t height, size_t width,
                                        float shift_y, float shift_x);

#ifdef __cplusplus
}
#endif

#endif
