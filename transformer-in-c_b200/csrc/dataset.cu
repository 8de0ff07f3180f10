#include "dataset.h"

#include "device_util.cuh"
#include "kernels.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

namespace vitb200 {
namespace {

// A file held in memory with a read cursor; get() plays the role of fgetc.
class Bytes {
public:
    bool open(const char *path) {
        FILE *file = fopen(path, "rb");
        if (!file) {
            return false;
        }
        char chunk[1 << 16];
        size_t got;
        while ((got = fread(chunk, 1, sizeof(chunk), file)) > 0) {
            data_.append(chunk, got);
        }
        fclose(file);
        return true;
    }
    int get() {
        return cursor_ < data_.size() ? static_cast<unsigned char>(data_[cursor_++])
                                      : EOF;
    }
private:
    std::string data_;
    size_t cursor_ = 0;
};

bool is_blank(int c) {
    return c == ' ' || c == '\n' || c == '\r' || c == '\t';
}

// One header or raster token (src/dataset.c:7-33): blanks are skipped, a '#'
// where a token would start opens a comment that runs to the end of the line,
// the blank that ends the token is consumed, and a token of 64 characters or
// more is an error.
bool next_token(Bytes &file, std::string *token) {
    int c;
    for (;;) {
        do {
            c = file.get();
        } while (c != EOF && is_blank(c));
        if (c != '#') {
            break;
        }
        do {
            c = file.get();
        } while (c != EOF && c != '\n');
    }
    if (c == EOF) {
        return false;
    }
    token->clear();
    while (c != EOF && !is_blank(c)) {
        if (token->size() + 1 >= 64) {
            return false;
        }
        token->push_back(char(c));
        c = file.get();
    }
    return true;
}

// src/dataset.c:35-53: the whole token must be a base-10 number as strtoul
// reads it; sizes must not be zero.
bool parse_number(const std::string &token, bool allow_zero, size_t *value) {
    char *end = nullptr;
    const unsigned long parsed = strtoul(token.c_str(), &end, 10);
    if (token.empty() || *end != '\0' || (!allow_zero && parsed == 0)) {
        return false;
    }
    *value = size_t(parsed);
    return true;
}

// One PGM image (src/dataset.c:55-125), appended to `pixels`.
bool read_pgm(const char *path, std::vector<uint16_t> *pixels, size_t *height,
              size_t *width, uint16_t *max_value) {
    Bytes file;
    std::string token;
    if (!file.open(path) || !next_token(file, &token) ||
        (token != "P2" && token != "P5")) {
        return false;
    }
    const bool binary = token == "P5";
    size_t maximum = 0;
    if (!next_token(file, &token) || !parse_number(token, false, width) ||
        !next_token(file, &token) || !parse_number(token, false, height) ||
        !next_token(file, &token) || !parse_number(token, false, &maximum) ||
        maximum > 65535) {
        return false;
    }
    const size_t count = *width * *height;
    const size_t start = pixels->size();
    pixels->resize(start + count);
    uint16_t *out = pixels->data() + start;
    for (size_t i = 0; i < count; ++i) {
        size_t value;
        if (binary) {
            // One byte per sample below 256, else two, most significant first;
            // values above the header's maximum are not rejected here.
            const int high = file.get();
            if (high == EOF) {
                return false;
            }
            value = size_t(high);
            if (maximum >= 256) {
                const int low = file.get();
                if (low == EOF) {
                    return false;
                }
                value = (value << 8) | size_t(low);
            }
        } else if (!next_token(file, &token) ||
                   !parse_number(token, true, &value) || value > maximum) {
            return false;
        }
        out[i] = uint16_t(value);
    }
    *max_value = uint16_t(maximum);
    return true;
}

}  // namespace

int dataset_parse_pgm_csv(const char *manifest_path, ParsedDataset *out) {
    if (!manifest_path || !out) {
        return -1;
    }
    *out = ParsedDataset();
    FILE *manifest = fopen(manifest_path, "r");
    if (!manifest) {
        return -1;
    }
    char line[4096];
    bool ok = true;
    while (ok && fgets(line, sizeof(line), manifest)) {
        if (line[0] == '#' || line[0] == '\n' || line[0] == '\r') {
            continue;
        }
        // `path,label`: leading blanks dropped, the path runs to the first
        // comma (src/dataset.c:163).
        char path[2048];
        unsigned long label = 0;
        size_t height = 0, width = 0;
        uint16_t max_value = 0;
        ok = sscanf(line, " %2047[^,],%lu", path, &label) == 2 &&
             read_pgm(path, &out->pixels, &height, &width, &max_value);
        if (ok && out->labels.empty()) {
            out->height = height;
            out->width = width;
        }
        ok = ok && out->height == height && out->width == width;
        if (ok) {
            out->labels.push_back(size_t(label));
            out->max_values.push_back(max_value);
        }
    }
    fclose(manifest);
    if (!ok || out->labels.empty()) {
        *out = ParsedDataset();
        return -1;
    }
    return 0;
}

void dataset_statistics(const ParsedDataset &dataset, float *mean,
                        float *inverse_standard_deviation) {
    const size_t image_size = dataset.image_size();
    const size_t count = dataset.samples() * image_size;
    double sum = 0.0, squared_sum = 0.0;
    for (size_t sample = 0; sample < dataset.samples(); ++sample) {
        const uint16_t *pixels = dataset.pixels.data() + sample * image_size;
        const uint16_t max_value = dataset.max_values[sample];
        for (size_t i = 0; i < image_size; ++i) {
            const float pixel = dataset_pixel_value(pixels[i], max_value);
            sum += pixel;
            squared_sum += double(pixel) * pixel;
        }
    }
    const double average = sum / double(count);
    const double variance = squared_sum / double(count) - average * average;
    const double floor = 1e-12;
    *mean = float(average);
    *inverse_standard_deviation =
        float(1.0 / std::sqrt(variance > floor ? variance : floor));
}

void dataset_shuffle(std::vector<uint32_t> &order, unsigned long *state) {
    for (size_t index = order.size(); index > 1; --index) {
        *state = *state * 1664525UL + 1013904223UL;
        const size_t other = *state % index;
        if (other != index - 1) {
            const uint32_t held = order[index - 1];
            order[index - 1] = order[other];
            order[other] = held;
        }
    }
}

namespace {

constexpr int kBatchThreads = 256;

// V sample values per thread (4 when the image size allows 32-/64-bit loads
// of the stored integers and 128-bit stores of the floats).  Each of the three
// operations rounds once, like the host code it stands for.
template <typename T, int V>
__global__ void __launch_bounds__(kBatchThreads)
dataset_batch_kernel(const T *__restrict__ pixels,
                     const uint16_t *__restrict__ max_values,
                     const uint32_t *__restrict__ order, size_t first,
                     size_t batch, size_t image_size, float mean,
                     float inverse_std, float *__restrict__ destination) {
    const size_t per_image = image_size / V;
    const size_t total = batch * per_image;
    for (size_t i = size_t(blockIdx.x) * kBatchThreads + threadIdx.x; i < total;
         i += size_t(gridDim.x) * kBatchThreads) {
        const size_t slot = i / per_image;
        const size_t offset = (i % per_image) * V;
        const size_t sample = order ? order[first + slot] : first + slot;
        const float scale = float(max_values[sample]);
        const T *source = pixels + sample * image_size + offset;
        float values[V];
        if (V == 4) {
            alignas(8) T raw[4];
            if (sizeof(T) == 1) {
                *reinterpret_cast<uint32_t *>(raw) =
                    *reinterpret_cast<const uint32_t *>(source);
            } else {
                *reinterpret_cast<uint2 *>(raw) =
                    *reinterpret_cast<const uint2 *>(source);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                values[e] = float(raw[e]);
            }
        } else {
            values[0] = float(source[0]);
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
            values[e] = __fmul_rn(
                __fsub_rn(__fdiv_rn(values[e], scale), mean), inverse_std);
        }
        float *target = destination + slot * image_size + offset;
        if (V == 4) {
            __stcs(reinterpret_cast<float4 *>(target),
                   make_float4(values[0], values[1], values[2], values[3]));
        } else {
            target[0] = values[0];
        }
    }
}

template <typename T>
void launch_batch(const void *pixels, const uint16_t *max_values,
                  const uint32_t *order, size_t first, size_t batch,
                  size_t image_size, float mean, float inverse_std,
                  float *destination, cudaStream_t stream) {
    const T *typed = static_cast<const T *>(pixels);
    // 16-byte stores need the destination rows aligned as well.
    const bool vector = image_size % 4 == 0 &&
                        reinterpret_cast<uintptr_t>(destination) % 16 == 0 &&
                        reinterpret_cast<uintptr_t>(pixels) % 8 == 0;
    const size_t work = batch * (vector ? image_size / 4 : image_size);
    size_t blocks = (work + kBatchThreads - 1) / kBatchThreads;
    const size_t wave = size_t(kSmCount) * 8;
    blocks = blocks < wave ? (blocks ? blocks : 1) : wave;
    if (vector) {
        dataset_batch_kernel<T, 4><<<unsigned(blocks), kBatchThreads, 0, stream>>>(
            typed, max_values, order, first, batch, image_size, mean,
            inverse_std, destination);
    } else {
        dataset_batch_kernel<T, 1><<<unsigned(blocks), kBatchThreads, 0, stream>>>(
            typed, max_values, order, first, batch, image_size, mean,
            inverse_std, destination);
    }
    ++g_kernel_launches;
}

}  // namespace

void launch_dataset_batch(const void *pixels, bool wide,
                          const uint16_t *max_values, const uint32_t *order,
                          size_t first, size_t batch, size_t image_size,
                          float mean, float inverse_standard_deviation,
                          float *destination, cudaStream_t stream) {
    if (batch == 0 || image_size == 0) {
        return;
    }
    if (wide) {
        launch_batch<uint16_t>(pixels, max_values, order, first, batch,
                               image_size, mean, inverse_standard_deviation,
                               destination, stream);
    } else {
        launch_batch<uint8_t>(pixels, max_values, order, first, batch,
                              image_size, mean, inverse_standard_deviation,
                              destination, stream);
    }
}

}  // namespace vitb200
