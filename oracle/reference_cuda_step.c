/* Times the reference's own CUDA backend (src/cuda_backend.cu: cuBLAS SGEMM,
 * managed memory, its SIMT kernels) on the training step.
 *
 * TEST INFRASTRUCTURE ONLY: a secondary baseline for bench.py, built by
 * oracle/build_ref.py from the reference's unmodified sources compiled for
 * sm_100a.  Nothing of the shipped library is linked in.
 *
 * usage: reference_cuda_step channels height width patch d_model heads layers
 *                            classes batch warmup steps
 * prints one JSON object; exit code 77 when the backend reports no device.
 */
#define _POSIX_C_SOURCE 199309L
#include "cuda_backend.h"
#include "ops.h"
#include "vit.h"

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <time.h>

static uint64_t next_bits(uint64_t *state) {
    uint64_t z = (*state += 0x9E3779B97F4A7C15ULL);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

static double now_seconds(void) {
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return (double)t.tv_sec + 1e-9 * (double)t.tv_nsec;
}

int main(int argc, char **argv) {
    if (argc != 12) {
        fprintf(stderr, "usage: %s c h w patch d heads layers classes batch warmup steps\n",
                argv[0]);
        return 2;
    }
    size_t v[11];
    for (int i = 0; i < 11; ++i) {
        v[i] = (size_t)strtoull(argv[i + 1], NULL, 10);
    }
    const ViTConfig config = {v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7]};
    const size_t batch = v[8], warmup = v[9], steps = v[10];
    CudaBackend *backend = NULL;
    if (cuda_backend_create(&backend) != 0) {
        return 77;
    }
    if (cuda_backend_enable_device_execution(backend) != 0) {
        return 1;
    }
    ViTModel model;
    ViTModelCache cache;
    if (vit_model_init_seeded(&model, &config, 42) != 0 ||
        vit_model_cache_init(&cache, &model, batch) != 0) {
        fprintf(stderr, "model setup failed\n");
        return 1;
    }
    const size_t pixels = batch * v[0] * v[1] * v[2];
    float *images = malloc(pixels * sizeof(float));
    size_t *labels = malloc(batch * sizeof(size_t));
    uint64_t state = 1234;
    if (!images || !labels) {
        return 1;
    }
    for (size_t i = 0; i < pixels; ++i) {
        images[i] = (float)(next_bits(&state) >> 40) / 16777216.0f - 0.5f;
    }
    for (size_t i = 0; i < batch; ++i) {
        labels[i] = (size_t)(next_bits(&state) % v[7]);
    }
    float loss = 0.0f;
    for (size_t i = 0; i < warmup; ++i) {
        if (vit_model_train_batch_smoothed(&model, images, labels, batch, &cache,
                                           1e-3f, 0.05f, NULL, 0.1f, &loss) != 0) {
            return 1;
        }
    }
    const double start = now_seconds();
    for (size_t i = 0; i < steps; ++i) {
        if (vit_model_train_batch_smoothed(&model, images, labels, batch, &cache,
                                           1e-3f, 0.05f, NULL, 0.1f, &loss) != 0) {
            return 1;
        }
    }
    const double seconds = now_seconds() - start;
    printf("{\"ms_per_step\": %.4f, \"images_per_second\": %.2f, \"batch\": %zu, "
           "\"steps\": %zu, \"loss\": %.6f}\n",
           1e3 * seconds / (double)steps, (double)(batch * steps) / seconds,
           batch, steps, loss);
    vit_model_cache_free(&cache);
    vit_model_free(&model);
    cuda_backend_free(backend);
    free(images);
    free(labels);
    return 0;
}
