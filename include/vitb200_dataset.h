/*
 * Image datasets resident on the B200: counterparts of the reference's loader
 * (include/dataset.h) and of the three dataset passes of its trainer
 * (examples/organ_smnist.c:75-139: shuffle, pixel statistics, normalisation)
 * for callers that hold a vitb200 backend.
 *
 * The samples are uploaded once, as the integers the PGM files hold (one byte
 * per pixel, two when a file's maximum value needs them).  A shuffle permutes
 * a table of 4-byte indices with the trainer's own sequence of random draws
 * instead of moving images, and a batch is gathered, converted and normalised
 * by one kernel straight into the caller's buffer.  Every value is
 * bit-identical to what the reference's host pipeline
 * (vision_dataset_load_pgm_csv -> normalize_dataset -> shuffle_dataset ->
 * batch slice) holds at the same place.
 */
#ifndef VITB200_DATASET_H
#define VITB200_DATASET_H

#include <stddef.h>

#include "vitb200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct vitb200_dataset vitb200_dataset;

/* vision_dataset_load_pgm_csv (include/dataset.h:23-24, src/dataset.c:136-226)
 * with the result on the backend's device: same manifest syntax, same PGM
 * dialects (P2 / P5, 8 and 16 bit), same failures.  0 on success; -1 on
 * invalid arguments, an unusable backend, or any input the reference rejects
 * (*dataset is then NULL). */
int vitb200_dataset_load_pgm_csv(CudaBackend *backend, const char *manifest_path,
                                 vitb200_dataset **dataset);

/* The same object from samples that are already in memory: `pixels` holds
 * sample_count x height x width integers (row-major, one channel),
 * `max_values` each sample's PGM maximum (1..65535; NULL = 255 for all),
 * `labels` one class index per sample. */
int vitb200_dataset_from_integers(CudaBackend *backend,
                                  const unsigned short *pixels,
                                  const unsigned short *max_values,
                                  const size_t *labels, size_t sample_count,
                                  size_t height, size_t width,
                                  vitb200_dataset **dataset);

/* vision_dataset_free (include/dataset.h:25).  NULL-safe.  A dataset uses its
 * backend's stream: free it before cuda_backend_free. */
void vitb200_dataset_free(vitb200_dataset *dataset);

/* The fields of the reference's VisionDataset. */
size_t vitb200_dataset_sample_count(const vitb200_dataset *dataset);
size_t vitb200_dataset_height(const vitb200_dataset *dataset);
size_t vitb200_dataset_width(const vitb200_dataset *dataset);
size_t vitb200_dataset_channels(const vitb200_dataset *dataset);

/* compute_pixel_statistics (examples/organ_smnist.c:108-127): mean and
 * 1 / standard deviation of the loader's [0, 1] pixels, accumulated in double
 * in storage order on the host when the dataset is created. */
int vitb200_dataset_statistics(const vitb200_dataset *dataset, float *mean,
                               float *inverse_standard_deviation);

/* shuffle_dataset (examples/organ_smnist.c:75-101): advances *state through
 * the same draws and leaves the samples in the order the reference's
 * dataset would have; successive calls compose, as they do there. */
int vitb200_dataset_shuffle(vitb200_dataset *dataset, unsigned long *state);

/* Samples [offset, offset + batch) of the current order:
 * images[b][p] = (pixel / max_value - mean) * inverse_standard_deviation
 * (the loader's conversion, src/dataset.c:104, then normalize_pixel,
 * examples/organ_smnist.c:129-131; pass mean = 0, inverse = 1 for the
 * loader's own values) and labels[b].  `images` may be ordinary host memory
 * (the call returns with the batch in place) or tensor memory obtained through
 * the backend's allocator, such as the model cache's image tensor (the kernel
 * writes it where it lives on the device and the call returns with the work
 * enqueued; the tensor must hold exactly batch x height x width floats, since
 * all of it is declared overwritten).  `labels` may be NULL.  -1 when the range leaves the dataset. */
int vitb200_dataset_batch(vitb200_dataset *dataset, size_t offset, size_t batch,
                          float mean, float inverse_standard_deviation,
                          float *images, size_t *labels);

/* Loader only, no device: fills *pixels / *max_values / *labels with malloc'ed
 * arrays (free them with free()).  For tools and for checking the parser
 * against the reference's without a GPU. */
int vitb200_dataset_parse_pgm_csv(const char *manifest_path,
                                  unsigned short **pixels,
                                  unsigned short **max_values, size_t **labels,
                                  size_t *sample_count, size_t *height,
                                  size_t *width);

/* compute_pixel_statistics on integers in memory (no device); max_values NULL
 * = 255 for all. */
int vitb200_dataset_pixel_statistics(const unsigned short *pixels,
                                     const unsigned short *max_values,
                                     size_t sample_count, size_t image_size,
                                     float *mean,
                                     float *inverse_standard_deviation);

/* The index-table shuffle on its own (no device): order[0..count) is permuted
 * exactly as shuffle_dataset permutes its samples. */
void vitb200_dataset_shuffle_order(unsigned int *order, size_t count,
                                   unsigned long *state);

#ifdef __cplusplus
}
#endif

#endif
