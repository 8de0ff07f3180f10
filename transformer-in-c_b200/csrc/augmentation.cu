// Batch augmentation on the device (reference src/augmentation.c).
//
// The reference walks the batch sample by sample, pixel by pixel, drawing
// from one splitmix64 stream as it goes.  That generator advances its state
// by a constant per draw, so draw number k is mix(state + (k + 1) * step): a
// pure function of the start state.  The order of the draws is fixed except
// for random erasing, which takes four more draws only when its first draw
// says "erase".  A host pass over the batch (a dozen integer mixes per sample)
// therefore knows every per-sample parameter and where each sample's per-pixel
// noise draws start; after that every pixel is independent:
//
//   affine kernel   one thread per output pixel: inverse-map, bilinear sample
//                   with edge padding            (augmentation.c:36-90)
//   mean kernel     one warp per image plane: coalesced loads, additions in
//                   the reference's order by one lane (a float sum is
//                   order-dependent)                         (:118-122)
//   pixel kernel    contrast / brightness, Gaussian noise from the two draws
//                   that belong to the pixel, clamp, erase  (:123-166, :215-226)
//
// Arithmetic that the reference rounds step by step is written with the
// round-to-nearest intrinsics, which the compiler never contracts into fused
// multiply-adds; cos / sin of the rotation are taken on the host with the same
// libm as the reference.  What remains different is logf and cosf inside the
// Box-Muller noise (device libm, an ulp or two), i.e. errors of about 1e-7 of
// the noise amplitude; everything else is bit-identical.
#include "augmentation.h"
#include "kernels.h"
#include "device_util.cuh"

#include <cmath>

namespace vitb200 {
namespace {

constexpr unsigned long long kStep = 0x9E3779B97F4A7C15ull;
constexpr float kPi = 3.14159265358979323846f;

__host__ __device__ inline unsigned long long mix(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// ---- host side: the reference's draws, in its order ------------------------

struct Stream {
    uint64_t state;
    uint64_t bits() {
        state += kStep;
        return mix(state);
    }
    float unit() {   // augmentation.c:15-17
        return ((float)(bits() >> 40) + 0.5f) / 16777216.0f;
    }
    float symmetric(float magnitude) {   // :19-21
        return magnitude * (2.0f * unit() - 1.0f);
    }
    size_t index_below(size_t limit) {   // :28-30
        return (size_t)(bits() % (uint64_t)limit);
    }
};

bool geometric(const AugmentationSettings &s) {
    return s.max_shift_pixels > 0.0f || s.max_rotation_degrees > 0.0f ||
           s.max_scale_delta > 0.0f;
}

bool intensity(const AugmentationSettings &s) {
    return s.max_brightness_delta > 0.0f || s.max_contrast_delta > 0.0f;
}

// ---- device side -------------------------------------------------------------

__device__ __forceinline__ float clamp_value(float value, float minimum,
                                             float maximum) {
    return value < minimum ? minimum : value > maximum ? maximum : value;
}

// augmentation.c:36-55, every operation rounded on its own.
__device__ __forceinline__ float sample_bilinear(const float *plane, int height,
                                                 int width, float source_y,
                                                 float source_x) {
    const float clamped_y = clamp_value(source_y, 0.0f, float(height - 1));
    const float clamped_x = clamp_value(source_x, 0.0f, float(width - 1));
    const int top = int(clamped_y);
    const int left = int(clamped_x);
    const int bottom = top + 1 < height ? top + 1 : top;
    const int right = left + 1 < width ? left + 1 : left;
    const float wy = __fsub_rn(clamped_y, float(top));
    const float wx = __fsub_rn(clamped_x, float(left));
    const float one_minus_wx = __fsub_rn(1.0f, wx);
    const float upper =
        __fadd_rn(__fmul_rn(plane[top * width + left], one_minus_wx),
                  __fmul_rn(plane[top * width + right], wx));
    const float lower =
        __fadd_rn(__fmul_rn(plane[bottom * width + left], one_minus_wx),
                  __fmul_rn(plane[bottom * width + right], wx));
    return __fadd_rn(__fmul_rn(upper, __fsub_rn(1.0f, wy)),
                     __fmul_rn(lower, wy));
}

// augmentation.c:63-90.  `samples` == nullptr: one transform for all samples.
__global__ void augmentation_affine_kernel(
    const float *__restrict__ source, float *__restrict__ destination,
    const AugmentationSample *__restrict__ samples, AugmentationSample shared,
    size_t batch, int channels, int height, int width) {
    const size_t plane = size_t(height) * width;
    const size_t total = batch * channels * plane;
    const float center_y = __fmul_rn(0.5f, float(height - 1));
    const float center_x = __fmul_rn(0.5f, float(width - 1));
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t image_plane = i / plane;   // sample * channels + channel
        const int pixel = int(i % plane);
        const int y = pixel / width, x = pixel % width;
        const AugmentationSample &p =
            samples ? samples[image_plane / channels] : shared;
        const float centered_y =
            __fsub_rn(__fsub_rn(float(y), center_y), p.shift_y);
        const float centered_x =
            __fsub_rn(__fsub_rn(float(x), center_x), p.shift_x);
        const float source_x = __fadd_rn(
            __fadd_rn(__fmul_rn(p.inverse_cosine, centered_x),
                      __fmul_rn(p.inverse_sine, centered_y)),
            center_x);
        const float source_y = __fadd_rn(
            __fadd_rn(__fmul_rn(-p.inverse_sine, centered_x),
                      __fmul_rn(p.inverse_cosine, centered_y)),
            center_y);
        destination[i] = sample_bilinear(source + image_plane * plane, height,
                                         width, source_y, source_x);
    }
}

// augmentation.c:118-122: the plane mean, summed front to back.  A float sum
// depends on its order, so the additions stay sequential (lane 0 does them),
// but the loads are the warp's: 32 consecutive pixels at a time, handed to
// lane 0 by shuffles that do not wait for the running sum.
__global__ void augmentation_mean_kernel(const float *__restrict__ images,
                                         float *__restrict__ means,
                                         size_t planes, size_t plane_size) {
    const int lane = threadIdx.x & 31;
    const size_t warp = global_thread() >> 5;
    const size_t warps = grid_threads() >> 5;
    for (size_t p = warp; p < planes; p += warps) {
        const float *plane = images + p * plane_size;
        float sum = 0.0f;
        for (size_t base = 0; base < plane_size; base += 32) {
            const size_t index = base + lane;
            const float mine = index < plane_size ? plane[index] : 0.0f;
            const int live = int(min(size_t(32), plane_size - base));
            for (int l = 0; l < live; ++l) {
                sum = __fadd_rn(sum, __shfl_sync(kFullMask, mine, l));
            }
        }
        if (lane == 0) {
            means[p] = __fdiv_rn(sum, float(plane_size));
        }
    }
}

__device__ __forceinline__ float unit_from_state(unsigned long long state) {
    return __fdiv_rn(__fadd_rn(float(mix(state) >> 40), 0.5f), 16777216.0f);
}

// Everything after the geometric step, per pixel (augmentation.c:123-166 and
// the clamp of :219-223).
__global__ void augmentation_pixel_kernel(
    const float *__restrict__ input, float *__restrict__ destination,
    const AugmentationSample *__restrict__ samples,
    const float *__restrict__ means, AugmentationSettings settings,
    bool jitter, bool noise, bool clamps, bool erasing, size_t batch,
    int channels, int height, int width) {
    const size_t plane = size_t(height) * width;
    const size_t image = plane * channels;
    const size_t total = batch * image;
    for (size_t i = global_thread(); i < total; i += grid_threads()) {
        const size_t sample = i / image;
        const size_t within = i % image;   // the reference's noise loop index
        const AugmentationSample &p = samples[sample];
        float value = input[i];
        if (jitter) {
            const float mean = means[i / plane];
            value = __fadd_rn(
                __fadd_rn(mean, __fmul_rn(__fsub_rn(value, mean), p.contrast)),
                p.brightness);
        }
        if (noise) {
            // Draws 2k+1 and 2k+2 after the sample's noise start.
            const unsigned long long first =
                p.noise_state + (2ull * within + 1ull) * kStep;
            const float u1 = unit_from_state(first);
            const float u2 = unit_from_state(first + kStep);
            const float radius = __fsqrt_rn(__fmul_rn(-2.0f, logf(u1)));
            const float normal =
                __fmul_rn(radius, cosf(__fmul_rn(2.0f * kPi, u2)));
            value = __fadd_rn(
                value, __fmul_rn(settings.noise_standard_deviation, normal));
        }
        if (clamps) {
            value = clamp_value(value, settings.minimum_value,
                                settings.maximum_value);
        }
        if (erasing && p.erase_height) {
            const unsigned pixel = unsigned(within % plane);
            const unsigned y = pixel / unsigned(width);
            const unsigned x = pixel % unsigned(width);
            if (y >= p.erase_top && y < p.erase_top + p.erase_height &&
                x >= p.erase_left && x < p.erase_left + p.erase_width) {
                value = settings.erasing_value;
            }
        }
        destination[i] = value;
    }
}

}  // namespace

bool augmentation_enabled(const AugmentationSettings &s) {
    return geometric(s) || intensity(s) || s.noise_standard_deviation > 0.0f ||
           s.erasing_probability > 0.0f;
}

bool augmentation_arguments_valid(const AugmentationSettings *s,
                                  const uint64_t *random_state,
                                  const void *source, const void *destination,
                                  size_t batch, size_t channels, size_t height,
                                  size_t width) {
    return !(!s || !random_state || !source || !destination || batch == 0 ||
             channels == 0 || height == 0 || width == 0 ||
             s->max_shift_pixels < 0.0f || s->max_rotation_degrees < 0.0f ||
             s->max_scale_delta < 0.0f || s->max_scale_delta >= 1.0f ||
             s->max_brightness_delta < 0.0f || s->max_contrast_delta < 0.0f ||
             s->max_contrast_delta >= 1.0f ||
             s->noise_standard_deviation < 0.0f ||
             s->erasing_probability < 0.0f || s->erasing_probability > 1.0f ||
             s->erasing_max_side_fraction < 0.0f ||
             s->erasing_max_side_fraction > 1.0f ||
             (geometric(*s) && source == destination));
}

void augmentation_plan(const AugmentationSettings &s, uint64_t *random_state,
                       size_t batch, size_t channels, size_t height,
                       size_t width, AugmentationSample *samples) {
    Stream stream{*random_state};
    const size_t image_size = channels * height * width;
    for (size_t sample = 0; sample < batch; ++sample) {
        AugmentationSample &p = samples[sample];
        p = AugmentationSample{};
        p.inverse_cosine = 1.0f;
        p.contrast = 1.0f;
        if (geometric(s)) {   // augmentation.c:92-107, :67-68
            p.shift_y = stream.symmetric(s.max_shift_pixels);
            p.shift_x = stream.symmetric(s.max_shift_pixels);
            const float angle =
                stream.symmetric(s.max_rotation_degrees) * kPi / 180.0f;
            const float scale = 1.0f + stream.symmetric(s.max_scale_delta);
            p.inverse_cosine = cosf(angle) / scale;
            p.inverse_sine = sinf(angle) / scale;
        }
        if (intensity(s)) {   // :112-115
            p.contrast = 1.0f + stream.symmetric(s.max_contrast_delta);
            p.brightness = stream.symmetric(s.max_brightness_delta);
        }
        if (s.noise_standard_deviation > 0.0f) {   // :130-136, two draws a pixel
            p.noise_state = stream.state;
            stream.state += 2ull * image_size * kStep;
        }
        if (s.erasing_probability > 0.0f) {   // :141-166
            if (!(stream.unit() >= s.erasing_probability)) {
                const size_t max_height = (size_t)fmaxf(
                    1.0f, s.erasing_max_side_fraction * (float)height);
                const size_t max_width = (size_t)fmaxf(
                    1.0f, s.erasing_max_side_fraction * (float)width);
                const size_t erased_height = 1 + stream.index_below(max_height);
                const size_t erased_width = 1 + stream.index_below(max_width);
                p.erase_top = unsigned(stream.index_below(height - erased_height + 1));
                p.erase_left = unsigned(stream.index_below(width - erased_width + 1));
                p.erase_height = unsigned(erased_height);
                p.erase_width = unsigned(erased_width);
            }
        }
    }
    *random_state = stream.state;
}

void launch_augmentation(const AugmentationSettings &s,
                         const AugmentationSample *samples, const float *source,
                         float *destination, float *means, size_t batch,
                         size_t channels, size_t height, size_t width,
                         cudaStream_t stream) {
    const size_t total = batch * channels * height * width;
    const float *current = source;
    if (geometric(s)) {
        augmentation_affine_kernel<<<stream_grid(total), kStreamThreads, 0,
                                     stream>>>(
            source, destination, samples, AugmentationSample{}, batch,
            int(channels), int(height), int(width));
        ++g_kernel_launches;
        current = destination;
    }
    const bool jitter = intensity(s);
    const bool noise = s.noise_standard_deviation > 0.0f;
    const bool clamps = s.minimum_value < s.maximum_value;
    const bool erasing = s.erasing_probability > 0.0f;
    if (jitter) {
        augmentation_mean_kernel<<<stream_grid(batch * channels * 32),
                                   kStreamThreads, 0, stream>>>(
            current, means, batch * channels, height * width);
        ++g_kernel_launches;
    }
    if (jitter || noise || clamps || erasing || current != destination) {
        augmentation_pixel_kernel<<<stream_grid(total), kStreamThreads, 0,
                                    stream>>>(
            current, destination, samples, means, s, jitter, noise, clamps,
            erasing, batch, int(channels), int(height), int(width));
        ++g_kernel_launches;
    }
}

void launch_augmentation_translate(const float *source, float *destination,
                                   size_t batch, size_t channels, size_t height,
                                   size_t width, float shift_y, float shift_x,
                                   cudaStream_t stream) {
    AugmentationSample all{};
    all.inverse_cosine = cosf(0.0f) / 1.0f;
    all.inverse_sine = sinf(0.0f) / 1.0f;
    all.shift_y = shift_y;
    all.shift_x = shift_x;
    const size_t total = batch * channels * height * width;
    augmentation_affine_kernel<<<stream_grid(total), kStreamThreads, 0, stream>>>(
        source, destination, nullptr, all, batch, int(channels), int(height),
        int(width));
    ++g_kernel_launches;
}

}  // namespace vitb200
