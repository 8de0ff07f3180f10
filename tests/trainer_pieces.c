/*
 * TEST INFRASTRUCTURE.  Exposes three static functions of the reference's
 * trainer (examples/organ_smnist.c: shuffle_dataset :75-101,
 * compute_pixel_statistics :108-127, normalize_dataset :132-139) so that the
 * device-resident dataset can be checked against them.  The trainer's source is
 * compiled where it lies (oracle/build_ref.py passes its directory with -I and
 * renames its main); nothing of it is copied here.
 */
#define main organ_smnist_main
#include "organ_smnist.c"
#undef main

int trainer_shuffle(VisionDataset *dataset, unsigned long *state) {
    return shuffle_dataset(dataset, state);
}

void trainer_statistics(const VisionDataset *dataset, float *mean,
                        float *inverse_standard_deviation) {
    const PixelStatistics statistics = compute_pixel_statistics(dataset);
    *mean = statistics.mean;
    *inverse_standard_deviation = statistics.inverse_standard_deviation;
}

void trainer_normalize(VisionDataset *dataset, float mean,
                       float inverse_standard_deviation) {
    const PixelStatistics statistics = {mean, inverse_standard_deviation};
    normalize_dataset(dataset, &statistics);
}
