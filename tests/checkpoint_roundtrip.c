/* Checkpoint round trip through the reference's own vit_model_save /
 * vit_model_load (src/vit.c:1203-1259) with the device backend enabled.
 *
 * Built by oracle/build_ref.py against the reference's sources and
 * libvitb200.so (like the reference's tests/test_device.c) and run by
 * tests/test_checkpoint_gpu.py.  Exit code 0 = pass, 77 = no usable device.
 *
 *  1. train a device model for a few steps, save it while its parameters live
 *     on the device (the writer hands tensor memory to fwrite);
 *  2. load the file into a second device model (fread into tensor memory) and
 *     into a CPU model;
 *  3. every copy must hold bit-identical values, moments and step counters,
 *     and two device models with the same contents must produce the same
 *     loss on the next step;
 *  4. load a checkpoint into a device model whose parameters currently live
 *     on the device (fread into protected pages);
 *  5. the direct path (vitb200_checkpoint_save / _load: device buffers ->
 *     page-locked staging -> file and back): its file must be byte-identical
 *     to the one the reference's writer produces for the same model, every
 *     byte of it must have come straight from device buffers, the reference's
 *     reader must accept it into a CPU model, and a device model loaded from
 *     the reference's file through the direct reader must hold the same
 *     contents and give the same loss on the next step.
 */
#include "cuda_backend.h"
#include "vitb200.h"
#include "ops.h"
#include "tensor.h"
#include "vit.h"

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define BATCH 8
#define CHECK(condition)                                                     \
    do {                                                                     \
        if (!(condition)) {                                                  \
            fprintf(stderr, "checkpoint_roundtrip: %s failed (line %d)\n",   \
                    #condition, __LINE__);                                   \
            return 1;                                                        \
        }                                                                    \
    } while (0)

static uint64_t next_bits(uint64_t *state) {
    uint64_t z = (*state += 0x9E3779B97F4A7C15ULL);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

static size_t collect(ViTModel *model, Parameter **list) {
    size_t n = 0;
    list[n++] = &model->patch_projection.projection;
    list[n++] = &model->patch_projection.bias;
    list[n++] = &model->token_embedding.cls_token;
    list[n++] = &model->token_embedding.positional_embeddings;
    for (size_t layer = 0; layer < model->config.layers; ++layer) {
        ViTEncoderBlock *block = &model->blocks[layer];
        list[n++] = &block->query_key_value;
        list[n++] = &block->query_key_value_bias;
        list[n++] = &block->attention_output;
        list[n++] = &block->attention_output_bias;
        list[n++] = &block->mlp_input;
        list[n++] = &block->mlp_input_bias;
        list[n++] = &block->mlp_output;
        list[n++] = &block->mlp_output_bias;
        list[n++] = &block->attention_gamma;
        list[n++] = &block->attention_beta;
        list[n++] = &block->mlp_gamma;
        list[n++] = &block->mlp_beta;
    }
    list[n++] = &model->final_gamma;
    list[n++] = &model->final_beta;
    list[n++] = &model->classification_head.projection;
    list[n++] = &model->classification_head.bias;
    return n;
}

static int same_file(const char *a, const char *b) {
    FILE *fa = fopen(a, "rb"), *fb = fopen(b, "rb");
    int same = fa && fb;
    size_t bytes = 0;
    while (same) {
        const int ca = fgetc(fa), cb = fgetc(fb);
        same = ca == cb;
        if (ca == EOF || cb == EOF) {
            break;
        }
        ++bytes;
    }
    if (fa) fclose(fa);
    if (fb) fclose(fb);
    return same && bytes > 1000;
}

static int same_parameters(ViTModel *a, ViTModel *b) {
    Parameter *pa[8 + 12 * 4], *pb[8 + 12 * 4];
    const size_t count = collect(a, pa);
    if (collect(b, pb) != count) {
        return 0;
    }
    ops_synchronize();
    for (size_t i = 0; i < count; ++i) {
        const size_t bytes = tensor_numel(&pa[i]->value) * sizeof(float);
        const int same_step = pa[i]->step == pb[i]->step;
        const int same_value = memcmp(pa[i]->value.data, pb[i]->value.data, bytes) == 0;
        const int same_m = memcmp(pa[i]->m, pb[i]->m, bytes) == 0;
        const int same_v = memcmp(pa[i]->v, pb[i]->v, bytes) == 0;
        if (!same_step || !same_value || !same_m || !same_v) {
            fprintf(stderr,
                    "parameter %zu differs: step %d (%zu / %zu) value %d m %d v %d; "
                    "value[0] %.9g / %.9g, m[0] %.9g / %.9g\n",
                    i, same_step, pa[i]->step, pb[i]->step, same_value, same_m,
                    same_v, pa[i]->value.data[0], pb[i]->value.data[0],
                    pa[i]->m[0], pb[i]->m[0]);
            return 0;
        }
    }
    return 1;
}

int main(int argc, char **argv) {
    const char *path = argc > 1 ? argv[1] : "/tmp/vitb200_checkpoint.bin";
    CudaBackend *backend = NULL;
    if (cuda_backend_create(&backend) != 0) {
        return 77;
    }
    /* d_model 64: the QKV weights are 48 KiB, far beyond stdio's buffer, so
     * the writer goes to write(2) with the tensor's own pointer. */
    const ViTConfig config = {1, 28, 28, 4, 64, 4, 2, 11};
    float *images = malloc(BATCH * 28 * 28 * sizeof(float));
    size_t labels[BATCH];
    uint64_t state = 2024;
    CHECK(images != NULL);
    for (size_t i = 0; i < BATCH * 28 * 28; ++i) {
        images[i] = (float)(next_bits(&state) >> 40) / 16777216.0f - 0.5f;
    }
    for (size_t i = 0; i < BATCH; ++i) {
        labels[i] = (size_t)(next_bits(&state) % 11);
    }

    CHECK(cuda_backend_enable_device_execution(backend) == 0);
    ViTModel first, second;
    ViTModelCache first_cache, second_cache;
    CHECK(vit_model_init_seeded(&first, &config, 7) == 0);
    CHECK(vit_model_cache_init(&first_cache, &first, BATCH) == 0);
    CHECK(vit_model_init_seeded(&second, &config, 8) == 0);
    CHECK(vit_model_cache_init(&second_cache, &second, BATCH) == 0);
    float loss = 0.0f;
    for (int step = 0; step < 3; ++step) {
        CHECK(vit_model_train_batch_smoothed(&first, images, labels, BATCH,
                                             &first_cache, 1e-3f, 0.05f, NULL,
                                             0.1f, &loss) == 0);
    }
    CHECK(vit_model_save(&first, path) == 0);
    CHECK(vit_model_load(&second, path) == 0);
    CHECK(same_parameters(&first, &second));
    float loss_first = 0.0f, loss_second = 0.0f;
    CHECK(vit_model_train_batch_smoothed(&first, images, labels, BATCH,
                                         &first_cache, 1e-3f, 0.05f, NULL, 0.1f,
                                         &loss_first) == 0);
    CHECK(vit_model_train_batch_smoothed(&second, images, labels, BATCH,
                                         &second_cache, 1e-3f, 0.05f, NULL,
                                         0.1f, &loss_second) == 0);
    /* Same weights, same batch: the same loss (the forward pass has no
     * order-dependent reductions); the updated weights may differ in the last
     * bits because weight-gradient reductions are not ordered. */
    CHECK(loss_first == loss_second);
    /* Save again after the extra step, from the second model this time, and
     * read it into the first model while that model's parameters are on the
     * device: fread into memory whose pages are protected. */
    CHECK(vit_model_save(&second, path) == 0);
    CHECK(vit_model_load(&first, path) == 0);
    CHECK(same_parameters(&first, &second));
    /* The loaded values are what the device uses next. */
    CHECK(vit_model_train_batch_smoothed(&first, images, labels, BATCH,
                                         &first_cache, 1e-3f, 0.05f, NULL, 0.1f,
                                         &loss_first) == 0);
    CHECK(vit_model_train_batch_smoothed(&second, images, labels, BATCH,
                                         &second_cache, 1e-3f, 0.05f, NULL,
                                         0.1f, &loss_second) == 0);
    CHECK(loss_first == loss_second);
    CHECK(vit_model_save(&second, path) == 0);
    ops_synchronize();

    /* 5. The direct path.  One more step first, so that values and moments
     * are device-owned when the file is written. */
    char direct_path[1024];
    snprintf(direct_path, sizeof(direct_path), "%s.direct", path);
    CHECK(vit_model_train_batch_smoothed(&second, images, labels, BATCH,
                                         &second_cache, 1e-3f, 0.05f, NULL,
                                         0.1f, &loss_second) == 0);
    Parameter *list[8 + 12 * 4];
    const size_t listed = collect(&second, list);
    CHECK(vitb200_checkpoint_save(backend, direct_path, &second.config,
                                  sizeof(second.config),
                                  (struct vitb200_parameter *const *)list,
                                  listed) == 0);
    size_t from_device = 0, from_host = 0, parameter_bytes = 0;
    vitb200_checkpoint_counters(&from_device, &from_host);
    for (size_t i = 0; i < listed; ++i) {
        parameter_bytes += 3 * tensor_numel(&list[i]->value) * sizeof(float);
    }
    CHECK(from_device == parameter_bytes && from_host == 0);
    CHECK(vit_model_save(&second, path) == 0);   /* the reference's writer */
    CHECK(same_file(path, direct_path));
    /* The reference's file through the direct reader into the other device
     * model: same contents, same next loss. */
    const size_t first_listed = collect(&first, list);
    CHECK(vitb200_checkpoint_load(backend, path, &first.config,
                                  sizeof(first.config),
                                  (struct vitb200_parameter *const *)list,
                                  first_listed) == 0);
    CHECK(same_parameters(&first, &second));
    CHECK(vit_model_train_batch_smoothed(&first, images, labels, BATCH,
                                         &first_cache, 1e-3f, 0.05f, NULL, 0.1f,
                                         &loss_first) == 0);
    CHECK(vit_model_train_batch_smoothed(&second, images, labels, BATCH,
                                         &second_cache, 1e-3f, 0.05f, NULL,
                                         0.1f, &loss_second) == 0);
    CHECK(loss_first == loss_second);
    /* A file of the wrong configuration is refused. */
    ViTConfig other = second.config;
    other.layers += 1;
    CHECK(vitb200_checkpoint_load(backend, path, &other, sizeof(other),
                                  (struct vitb200_parameter *const *)list,
                                  first_listed) == -1);
    /* The direct writer's file of the current state, for the CPU model below. */
    const size_t second_listed = collect(&second, list);
    CHECK(vitb200_checkpoint_save(backend, path, &second.config,
                                  sizeof(second.config),
                                  (struct vitb200_parameter *const *)list,
                                  second_listed) == 0);
    remove(direct_path);
    ops_synchronize();
    cuda_backend_disable_device_execution(backend);

    ViTModel host_model;
    CHECK(vit_model_init_seeded(&host_model, &config, 9) == 0);
    CHECK(vit_model_load(&host_model, path) == 0);
    CHECK(same_parameters(&second, &host_model));

    vit_model_free(&host_model);
    vit_model_cache_free(&first_cache);
    vit_model_cache_free(&second_cache);
    vit_model_free(&first);
    vit_model_free(&second);
    cuda_backend_free(backend);
    free(images);
    remove(path);
    printf("checkpoint_roundtrip: ok (loss %.6f)\n", loss_first);
    return 0;
}
