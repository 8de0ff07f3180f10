// Batch augmentation on the device: the reference's data_augmentation_apply
// (reference src/augmentation.c:178-229) as three small kernels plus a host
// pass that lays the random stream out.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace vitb200 {

// Field for field the reference's DataAugmentation (include/augmentation.h:7-19).
struct AugmentationSettings {
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
};

// What the host pass decides for one sample: everything the reference draws
// per sample, and where in the random stream the sample's per-pixel noise
// draws start.
struct AugmentationSample {
    float inverse_cosine, inverse_sine, shift_y, shift_x;
    float contrast, brightness;
    unsigned erase_top, erase_left, erase_height, erase_width;   // height 0: none
    unsigned long long noise_state;   // stream state before the first noise draw
};

bool augmentation_enabled(const AugmentationSettings &settings);

// The reference's argument checks (src/augmentation.c:182-198).
bool augmentation_arguments_valid(const AugmentationSettings *settings,
                                  const uint64_t *random_state,
                                  const void *source, const void *destination,
                                  size_t batch, size_t channels, size_t height,
                                  size_t width);

// Plays the reference's sequence of draws for `batch` samples starting at
// *random_state, fills samples[0..batch) and leaves *random_state where the
// reference would.
void augmentation_plan(const AugmentationSettings &settings,
                       uint64_t *random_state, size_t batch, size_t channels,
                       size_t height, size_t width, AugmentationSample *samples);

// Applies a plan.  source / destination / samples are device pointers;
// `means` is scratch of batch * channels floats.  source == destination is
// allowed when no geometric transform is configured.
void launch_augmentation(const AugmentationSettings &settings,
                         const AugmentationSample *samples, const float *source,
                         float *destination, float *means, size_t batch,
                         size_t channels, size_t height, size_t width,
                         cudaStream_t stream);

// data_augmentation_translate (src/augmentation.c:231-245) on device buffers.
void launch_augmentation_translate(const float *source, float *destination,
                                   size_t batch, size_t channels, size_t height,
                                   size_t width, float shift_y, float shift_x,
                                   cudaStream_t stream);

}  // namespace vitb200
