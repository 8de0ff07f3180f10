// Image dataset kept on the device: the reference's PGM + CSV loader
// (reference src/dataset.c:55-226), its in-place shuffle and its pixel
// normalisation (reference examples/organ_smnist.c:75-139) for a trainer whose
// batches are consumed on the GPU.
//
// The samples stay in HBM as the integers the files hold (8 or 16 bits per
// pixel plus each file's maximum value).  A batch is produced by one kernel
// that gathers the samples of the current order, converts them as the
// reference's loader does (value / max, one rounding) and normalises them as
// its trainer does ((x - mean) * inverse_std, two roundings), so a batch is
// bit-identical to the reference's host pipeline while the per-epoch shuffle
// moves 4-byte indices instead of whole images.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>
#include <vector>

namespace vitb200 {

// What the loader extracts from the files, on the host.
struct ParsedDataset {
    std::vector<uint16_t> pixels;      // [samples][height * width]
    std::vector<uint16_t> max_values;  // per sample (PGM header)
    std::vector<size_t> labels;
    size_t height = 0, width = 0, channels = 1;
    size_t samples() const { return labels.size(); }
    size_t image_size() const { return height * width * channels; }
};

// vision_dataset_load_pgm_csv (src/dataset.c:136-226): same manifest syntax
// (`path,label` lines; '#', empty lines skipped), same PGM dialects (P2 / P5,
// comments, 8- and 16-bit samples), same failures (-1: unreadable file, bad
// header, value above the maximum, mixed sizes, empty manifest).
int dataset_parse_pgm_csv(const char *manifest_path, ParsedDataset *out);

// The float the reference's loader stores for one sample value.
inline float dataset_pixel_value(uint16_t value, uint16_t max_value) {
    return float(value) / float(max_value);
}

// compute_pixel_statistics (examples/organ_smnist.c:108-127): double sums over
// the loader's floats in storage order.
void dataset_statistics(const ParsedDataset &dataset, float *mean,
                        float *inverse_standard_deviation);

// shuffle_dataset (examples/organ_smnist.c:75-101) applied to an index table:
// the same draws from *state (the trainer's linear congruential generator,
// :70-73) and the same swaps, so order[i] is the loaded position of the sample
// the reference would now hold at position i.
void dataset_shuffle(std::vector<uint32_t> &order, unsigned long *state);

// destination[b][p] = ((pixels[order[first + b]][p] / max) - mean) * inverse_std
// for b in [0, batch).  All pointers are device pointers; `wide` selects 16-bit
// storage.  `order` may be null (identity).
void launch_dataset_batch(const void *pixels, bool wide,
                          const uint16_t *max_values, const uint32_t *order,
                          size_t first, size_t batch, size_t image_size,
                          float mean, float inverse_standard_deviation,
                          float *destination, cudaStream_t stream);

}  // namespace vitb200
