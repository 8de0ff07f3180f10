/*
 * Flat C entry points over the reference's public ViT API, for drivers that
 * cannot spell its structs (the Python tests and bench.py go through ctypes).
 *
 * This file is host-side glue only: it is compiled against the reference's own
 * headers (include/vit.h, include/ops.h, include/tensor.h) together with the
 * reference's unmodified ops.c / vit.c / autodiff.c / arena.c, and every
 * numerical step is one of their functions.  Whether those run on the CPU or
 * on the B200 depends solely on whether a device backend is enabled when the
 * model and cache are created, exactly as in the reference's tests
 * (tests/test_device.c:141-170).
 */
#include "ops.h"
#include "tensor.h"
#include "vit.h"

#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    ViTModel model;
    ViTModelCache cache;
    size_t batch;
    size_t parameter_count;
    Parameter **parameters;
    const char **names;
    float *weight_decay_mask; /* 1 where AdamW decays (vit.c:793-815) */
} VitHost;

static void add_parameter(VitHost *host, size_t *count, Parameter *parameter,
                          const char *name, int decays) {
    host->parameters[*count] = parameter;
    host->names[*count] = name;
    host->weight_decay_mask[*count] = decays ? 1.0f : 0.0f;
    *count += 1;
}

/* Same order as the reference's optimiser list (vit.c:784-818). */
static int collect(VitHost *host) {
    ViTModel *model = &host->model;
    const size_t total = 8 + 12 * model->config.layers;
    host->parameters = calloc(total, sizeof(*host->parameters));
    host->names = calloc(total, sizeof(*host->names));
    host->weight_decay_mask = calloc(total, sizeof(float));
    if (!host->parameters || !host->names || !host->weight_decay_mask) {
        return -1;
    }
    size_t n = 0;
    add_parameter(host, &n, &model->patch_projection.projection, "patch_projection", 1);
    add_parameter(host, &n, &model->patch_projection.bias, "patch_bias", 0);
    add_parameter(host, &n, &model->token_embedding.cls_token, "cls_token", 0);
    add_parameter(host, &n, &model->token_embedding.positional_embeddings, "positional", 0);
    for (size_t layer = 0; layer < model->config.layers; ++layer) {
        ViTEncoderBlock *block = &model->blocks[layer];
        add_parameter(host, &n, &block->query_key_value, "query_key_value", 1);
        add_parameter(host, &n, &block->query_key_value_bias, "query_key_value_bias", 0);
        add_parameter(host, &n, &block->attention_output, "attention_output", 1);
        add_parameter(host, &n, &block->attention_output_bias, "attention_output_bias", 0);
        add_parameter(host, &n, &block->mlp_input, "mlp_input", 1);
        add_parameter(host, &n, &block->mlp_input_bias, "mlp_input_bias", 0);
        add_parameter(host, &n, &block->mlp_output, "mlp_output", 1);
        add_parameter(host, &n, &block->mlp_output_bias, "mlp_output_bias", 0);
        add_parameter(host, &n, &block->attention_gamma, "attention_gamma", 0);
        add_parameter(host, &n, &block->attention_beta, "attention_beta", 0);
        add_parameter(host, &n, &block->mlp_gamma, "mlp_gamma", 0);
        add_parameter(host, &n, &block->mlp_beta, "mlp_beta", 0);
    }
    add_parameter(host, &n, &model->final_gamma, "final_gamma", 0);
    add_parameter(host, &n, &model->final_beta, "final_beta", 0);
    add_parameter(host, &n, &model->classification_head.projection, "head", 1);
    add_parameter(host, &n, &model->classification_head.bias, "head_bias", 0);
    host->parameter_count = n;
    return 0;
}

void vithost_destroy(VitHost *host) {
    if (!host) {
        return;
    }
    vit_model_cache_free(&host->cache);
    vit_model_free(&host->model);
    free(host->parameters);
    free(host->names);
    free(host->weight_decay_mask);
    free(host);
}

VitHost *vithost_create(size_t channels, size_t height, size_t width,
                        size_t patch_size, size_t d_model, size_t heads,
                        size_t layers, size_t classes, size_t batch,
                        uint64_t seed) {
    VitHost *host = calloc(1, sizeof(*host));
    if (!host) {
        return NULL;
    }
    const ViTConfig config = {channels, height, width, patch_size,
                              d_model, heads, layers, classes};
    host->batch = batch;
    if (vit_model_init_seeded(&host->model, &config, seed) != 0 ||
        vit_model_cache_init(&host->cache, &host->model, batch) != 0 ||
        collect(host) != 0) {
        vithost_destroy(host);
        return NULL;
    }
    return host;
}

size_t vithost_parameter_count(const VitHost *host) {
    return host->parameter_count;
}

const char *vithost_parameter_name(const VitHost *host, size_t index) {
    return index < host->parameter_count ? host->names[index] : NULL;
}

/* what: 0 value, 1 gradient, 2 first moment, 3 second moment.  Returns the
 * element count and stores the host pointer; reading through it is legal once
 * ops_synchronize() has returned (ops.h memory-visibility rule). */
size_t vithost_parameter_view(VitHost *host, size_t index, int what,
                              float **data, size_t *rows, size_t *cols) {
    if (index >= host->parameter_count) {
        return 0;
    }
    Parameter *parameter = host->parameters[index];
    ops_synchronize();
    float *pointers[4] = {parameter->value.data, parameter->value.grad,
                          parameter->m, parameter->v};
    *data = pointers[what & 3];
    *rows = parameter->value.rows;
    *cols = parameter->value.cols;
    return tensor_numel(&parameter->value);
}

size_t vithost_parameter_step(const VitHost *host, size_t index) {
    return index < host->parameter_count ? host->parameters[index]->step : 0;
}

static int zero_cache_gradients(ViTModelCache *cache) {
    Tensor *fixed[] = {
        &cache->images, &cache->patches, &cache->patch_tokens, &cache->tokens,
        &cache->normalized_tokens, &cache->cls_tokens, &cache->logits,
        &cache->targets, &cache->class_weights, &cache->loss,
    };
    const size_t fixed_count = sizeof(fixed) / sizeof(*fixed);
    const size_t count = fixed_count + 15 * cache->layers;
    Tensor **list = malloc(count * sizeof(*list));
    if (!list) {
        return -1;
    }
    size_t n = 0;
    for (size_t i = 0; i < fixed_count; ++i) {
        list[n++] = fixed[i];
    }
    for (size_t layer = 0; layer < cache->layers; ++layer) {
        ViTEncoderBlockCache *b = &cache->block_caches[layer];
        Tensor *per_block[] = {
            &b->normalized_attention, &b->projected, &b->query, &b->key,
            &b->value, &b->probabilities, &b->attended, &b->merged,
            &b->attention_branch, &b->attention_residual, &b->normalized_mlp,
            &b->hidden, &b->activated, &b->mlp_branch, &b->output,
        };
        for (size_t i = 0; i < 15; ++i) {
            list[n++] = per_block[i];
        }
    }
    const int result = ops_zero_gradients(list, count);
    free(list);
    return result;
}

/* Loss and all parameter gradients for one batch, without the optimiser step:
 * the first half of vit_model_train_batch_smoothed (vit.c:1094-1112). */
int vithost_gradients(VitHost *host, const float *images, const size_t *labels,
                      const float *class_weights, float label_smoothing,
                      float *loss) {
    ViTModelCache *cache = &host->cache;
    vit_model_zero_grad(&host->model);
    int result = zero_cache_gradients(cache) ||
        ops_upload_labels(&cache->targets, labels) ||
        (class_weights &&
         ops_upload_values(&cache->class_weights, class_weights)) ||
        vit_model_forward(&host->model, images, host->batch, cache) ||
        ops_softmax_cross_entropy_tensor(
            &cache->logits, &cache->targets,
            class_weights ? &cache->class_weights : NULL, label_smoothing,
            &cache->loss, &cache->logits) ||
        vit_model_backward(&host->model, images, cache, NULL);
    ops_synchronize();
    if (result == 0) {
        *loss = cache->loss.data[0];
    }
    return result;
}

/* One full training step, straight through the reference's entry point. */
int vithost_train_step(VitHost *host, const float *images,
                       const size_t *labels, float learning_rate,
                       float weight_decay, const float *class_weights,
                       float label_smoothing, float *loss) {
    return vit_model_train_batch_smoothed(
        &host->model, images, labels, host->batch, &host->cache, learning_rate,
        weight_decay, class_weights, label_smoothing, loss);
}

/* One optimiser step over `micro_batches` consecutive batches of host->batch
 * images each (gradient accumulation), composed from the reference's public
 * pieces in the order of vit_model_train_batch_smoothed (vit.c:1094-1121): the
 * parameter gradients are zeroed once, every micro-batch runs zero-cache /
 * upload / forward / loss / backward and adds into them, and one
 * ops_adamw_step_parameters call with the reference's constants (vit.c:1085,
 * 1102) follows.  Each micro-batch loss is a mean over its rows
 * (ops.c:1067-1070), so the accumulated gradient is `micro_batches` times the
 * gradient of the mean loss over all images: with `scale_on_host` the
 * gradients are divided on the host before the optimiser (CPU models);
 * without it the device backend must have been told the count
 * (vitb200_set_gradient_accumulation), which folds the factor into its clip
 * scale.  *loss receives the mean of the micro-batch losses. */
int vithost_train_step_accumulated(VitHost *host, const float *images,
                                   const size_t *labels, size_t micro_batches,
                                   float learning_rate, float weight_decay,
                                   const float *class_weights,
                                   float label_smoothing, int scale_on_host,
                                   float *loss) {
    if (!host || !images || !labels || !loss || micro_batches == 0) {
        return -1;
    }
    ViTModelCache *cache = &host->cache;
    const ViTConfig *config = &host->model.config;
    const size_t image_floats =
        config->channels * config->height * config->width;
    double loss_sum = 0.0;
    vit_model_zero_grad(&host->model);
    for (size_t micro = 0; micro < micro_batches; ++micro) {
        const float *batch_images = images + micro * host->batch * image_floats;
        const int result = zero_cache_gradients(cache) ||
            ops_upload_labels(&cache->targets, labels + micro * host->batch) ||
            (class_weights &&
             ops_upload_values(&cache->class_weights, class_weights)) ||
            vit_model_forward(&host->model, batch_images, host->batch, cache) ||
            ops_softmax_cross_entropy_tensor(
                &cache->logits, &cache->targets,
                class_weights ? &cache->class_weights : NULL, label_smoothing,
                &cache->loss, &cache->logits) ||
            vit_model_backward(&host->model, batch_images, cache, NULL);
        if (result != 0) {
            ops_synchronize();
            return result;
        }
        if (micro + 1 < micro_batches) {
            /* The next micro-batch overwrites the loss tensor. */
            ops_synchronize();
            loss_sum += cache->loss.data[0];
        }
    }
    if (scale_on_host && micro_batches > 1) {
        ops_synchronize();
        const float inverse = 1.0f / (float)micro_batches;
        for (size_t p = 0; p < host->parameter_count; ++p) {
            Tensor *value = &host->parameters[p]->value;
            const size_t count = tensor_numel(value);
            for (size_t i = 0; i < count; ++i) {
                value->grad[i] *= inverse;
            }
        }
    }
    float *decays = malloc(host->parameter_count * sizeof(*decays));
    if (!decays) {
        return -1;
    }
    for (size_t p = 0; p < host->parameter_count; ++p) {
        decays[p] = host->weight_decay_mask[p] * weight_decay;
    }
    const int result = ops_adamw_step_parameters(
        host->parameters, decays, host->parameter_count, learning_rate, 0.9f,
        0.999f, 1e-8f, 1.0f);
    free(decays);
    ops_synchronize();
    if (result == 0) {
        loss_sum += cache->loss.data[0];
        *loss = (float)(loss_sum / (double)micro_batches);
    }
    return result;
}

/* Forward only; copies the [batch, classes] logits out. */
int vithost_forward(VitHost *host, const float *images, float *logits) {
    const int result =
        vit_model_forward(&host->model, images, host->batch, &host->cache);
    if (result == 0) {
        memcpy(logits, host->cache.logits.data,
               tensor_numel(&host->cache.logits) * sizeof(float));
    }
    return result;
}

/* The cache's image tensor ([batch, channels * height * width], vit.c:837-879):
 * memory from the tensor allocator, so with a backend enabled a device-side
 * producer (augmentation, dataset batches) can fill it where it lives. */
float *vithost_images_tensor(VitHost *host) {
    return host->cache.images.data;
}

/* Overwrites one parameter's values (host write; the next device op picks the
 * new contents up). */
int vithost_set_parameter(VitHost *host, size_t index, const float *values) {
    if (index >= host->parameter_count) {
        return -1;
    }
    return ops_upload_values(&host->parameters[index]->value, values);
}

/* Named activation of one encoder block (data or grad), for layer-by-layer
 * comparisons.  Returns the element count, 0 if unknown. */
size_t vithost_block_tensor(VitHost *host, size_t layer, const char *name,
                            int want_grad, float **data, size_t *rows,
                            size_t *cols) {
    if (layer >= host->cache.layers) {
        return 0;
    }
    ViTEncoderBlockCache *b = &host->cache.block_caches[layer];
    struct { const char *name; Tensor *tensor; } table[] = {
        {"normalized_attention", &b->normalized_attention},
        {"projected", &b->projected}, {"query", &b->query}, {"key", &b->key},
        {"value", &b->value}, {"probabilities", &b->probabilities},
        {"attended", &b->attended}, {"merged", &b->merged},
        {"attention_branch", &b->attention_branch},
        {"attention_residual", &b->attention_residual},
        {"normalized_mlp", &b->normalized_mlp}, {"hidden", &b->hidden},
        {"activated", &b->activated}, {"mlp_branch", &b->mlp_branch},
        {"output", &b->output},
    };
    for (size_t i = 0; i < sizeof(table) / sizeof(*table); ++i) {
        if (strcmp(table[i].name, name) == 0) {
            ops_synchronize();
            *data = want_grad ? table[i].tensor->grad : table[i].tensor->data;
            *rows = table[i].tensor->rows;
            *cols = table[i].tensor->cols;
            return tensor_numel(table[i].tensor);
        }
    }
    return 0;
}

/* Inference entry points of the reference, unchanged: chunked forward passes
 * with the softmax / loss / argmax on the host (vit.c:1325-1403).  With a
 * backend enabled the forward passes run on the device and the host reads
 * the logits after each chunk's synchronise. */
int vithost_evaluate(VitHost *host, const float *images, const size_t *labels,
                     size_t sample_count, float *accuracy, float *average_loss,
                     double *samples_per_second) {
    ViTEvaluationMetrics metrics = {0};
    const int result = vit_model_evaluate(&host->model, images, labels,
                                          sample_count, &metrics);
    if (result == 0) {
        *accuracy = metrics.accuracy;
        *average_loss = metrics.average_loss;
        *samples_per_second = metrics.samples_per_second;
    }
    return result;
}

int vithost_predict(VitHost *host, const float *images, size_t sample_count,
                    float *probabilities) {
    return vit_model_predict_probabilities(&host->model, images, sample_count,
                                           probabilities);
}

/* The reference's single-parameter optimiser entry point (ops.c:1102-1121,
 * used by its own tests, tests/test_vision.c:616-624) on a parameter created
 * here: `steps` calls of ops_adamw_step on a [rows, cols] parameter whose
 * value and gradient start from the given arrays (the gradient is restored
 * before every call: the update zeroes it).  Returns the value, both moments
 * and the step counter.  With a backend enabled the parameter lives in
 * backend memory and the update runs in the adamw_step slot. */
int vithost_adamw_single(const float *values, const float *gradient, size_t rows,
                         size_t cols, size_t steps, float learning_rate,
                         float beta1, float beta2, float epsilon,
                         float weight_decay, float *value_out, float *m_out,
                         float *v_out, size_t *step_out) {
    Parameter parameter;
    memset(&parameter, 0, sizeof(parameter));
    if (parameter_init(&parameter, rows, cols) != 0) {
        return -1;
    }
    const size_t count = rows * cols;
    int status = 0;
    ops_synchronize();
    memcpy(parameter.value.data, values, count * sizeof(float));
    for (size_t step = 0; step < steps && status == 0; ++step) {
        ops_synchronize();
        memcpy(parameter.value.grad, gradient, count * sizeof(float));
        status = ops_adamw_step(&parameter, learning_rate, beta1, beta2, epsilon,
                                weight_decay);
    }
    ops_synchronize();
    memcpy(value_out, parameter.value.data, count * sizeof(float));
    memcpy(m_out, parameter.m, count * sizeof(float));
    memcpy(v_out, parameter.v, count * sizeof(float));
    *step_out = parameter.step;
    parameter_free(&parameter);
    return status;
}

/* ops_clip_gradient_norm (ops.c:588-617) over freshly created parameters
 * whose gradients are the given arrays (one array of `counts[i]` floats
 * each); the clipped gradients are copied back. */
int vithost_clip_gradients(float *const *gradients, const size_t *counts,
                           size_t tensors, float max_norm) {
    Parameter *storage = calloc(tensors, sizeof(*storage));
    Parameter **list = calloc(tensors, sizeof(*list));
    int status = storage && list ? 0 : -1;
    size_t made = 0;
    for (; status == 0 && made < tensors; ++made) {
        status = parameter_init(&storage[made], 1, counts[made]);
        list[made] = &storage[made];
    }
    if (status == 0) {
        ops_synchronize();
        for (size_t i = 0; i < tensors; ++i) {
            memcpy(storage[i].value.grad, gradients[i], counts[i] * sizeof(float));
        }
        status = ops_clip_gradient_norm(list, tensors, max_norm);
        ops_synchronize();
        for (size_t i = 0; i < tensors; ++i) {
            memcpy(gradients[i], storage[i].value.grad, counts[i] * sizeof(float));
        }
    }
    for (size_t i = 0; i < made; ++i) {
        parameter_free(&storage[i]);
    }
    free(storage);
    free(list);
    return status;
}
