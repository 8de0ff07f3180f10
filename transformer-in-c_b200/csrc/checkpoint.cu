// Checkpoints written from and read into device memory directly.
//
// The host's own writer (reference src/vit.c:1123-1215) hands every tensor to
// fwrite, which pulls each parameter, first moment and second moment back
// through its host mirror (page faults, mirror pages repopulated, ownership
// changes) before the bytes reach the file.  Here the same file -- format
// "CVITCKP" version 1: magic[8], uint32 version, the host's configuration
// structure as raw bytes, then per parameter { size_t count; size_t step;
// float value[count]; float m[count]; float v[count]; } in the optimiser's
// parameter order (reference src/vit.c:1144-1172) -- is produced from the
// device buffers through two page-locked staging blocks, one being filled by
// the copy engine while the other is written out; ownership and mirrors stay
// as they are.  Loading goes the other way and leaves the tensors
// device-owned.  Tensors whose current contents are on the host side are
// written from (read into) their mirrors.
#include "checkpoint.h"
#include "coherence.h"

#include <cstdint>
#include <cstdio>
#include <cstring>

namespace vitb200 {
namespace {

constexpr char kMagic[8] = {'C', 'V', 'I', 'T', 'C', 'K', 'P', '\0'};
constexpr uint32_t kVersion = 1;
constexpr size_t kBlockBytes = size_t(8) << 20;

struct Staging {
    char *block[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    bool busy[2] = {false, false};   // an upload from the block may be in flight
    int next = 0;                    // block the next upload stages in
    bool ok = false;
    Staging() {
        ok = cudaHostAlloc(reinterpret_cast<void **>(&block[0]), kBlockBytes,
                           cudaHostAllocDefault) == cudaSuccess &&
             cudaHostAlloc(reinterpret_cast<void **>(&block[1]), kBlockBytes,
                           cudaHostAllocDefault) == cudaSuccess &&
             cudaEventCreateWithFlags(&done[0], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&done[1], cudaEventDisableTiming) == cudaSuccess;
    }
    ~Staging() {
        for (int i = 0; i < 2; ++i) {
            if (block[i]) cudaFreeHost(block[i]);
            if (done[i]) cudaEventDestroy(done[i]);
        }
    }
};

// Writes `bytes` of one tensor.  `device` is where its current contents are,
// or nullptr when the mirror (`host`) holds them.
bool write_tensor(FILE *file, const float *device, const void *host, size_t bytes,
                  Staging &staging, cudaStream_t stream, CheckpointCounters *counters) {
    if (!device) {
        counters->from_mirrors += bytes;
        return fwrite(host, 1, bytes, file) == bytes;
    }
    counters->from_device += bytes;
    const char *source = reinterpret_cast<const char *>(device);
    size_t issued = 0, written = 0;
    int slot = 0;
    size_t in_flight[2] = {0, 0};
    // Two blocks in flight: copy block i + 1 while block i goes to the file.
    while (written < bytes) {
        while (issued < bytes && in_flight[slot] == 0) {
            const size_t chunk = bytes - issued < kBlockBytes ? bytes - issued : kBlockBytes;
            if (cudaMemcpyAsync(staging.block[slot], source + issued, chunk,
                                cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
                cudaEventRecord(staging.done[slot], stream) != cudaSuccess) {
                return false;
            }
            in_flight[slot] = chunk;
            issued += chunk;
            slot ^= 1;
        }
        const int oldest = in_flight[slot] ? slot : slot ^ 1;
        if (cudaEventSynchronize(staging.done[oldest]) != cudaSuccess ||
            fwrite(staging.block[oldest], 1, in_flight[oldest], file) !=
                in_flight[oldest]) {
            return false;
        }
        written += in_flight[oldest];
        in_flight[oldest] = 0;
        slot = oldest;
    }
    return true;
}

bool read_tensor(FILE *file, float *device, size_t bytes, Staging &staging,
                 cudaStream_t stream) {
    // The two blocks alternate across tensors as well: the file is read into
    // one while the copy engine still empties the other.
    char *target = reinterpret_cast<char *>(device);
    size_t done = 0;
    while (done < bytes) {
        const size_t chunk = bytes - done < kBlockBytes ? bytes - done : kBlockBytes;
        const int slot = staging.next;
        if (staging.busy[slot] &&
            cudaEventSynchronize(staging.done[slot]) != cudaSuccess) {
            return false;
        }
        if (fread(staging.block[slot], 1, chunk, file) != chunk ||
            cudaMemcpyAsync(target + done, staging.block[slot], chunk,
                            cudaMemcpyHostToDevice, stream) != cudaSuccess ||
            cudaEventRecord(staging.done[slot], stream) != cudaSuccess) {
            return false;
        }
        staging.busy[slot] = true;
        staging.next = slot ^ 1;
        done += chunk;
    }
    return true;
}

}  // namespace

int checkpoint_save(const char *path, const void *config, size_t config_bytes,
                    vitb200_parameter *const *parameters, size_t count,
                    cudaStream_t stream, CheckpointCounters *counters) {
    CheckpointCounters local = {};
    if (!counters) {
        counters = &local;
    }
    Staging staging;
    if (!staging.ok || !path || !config || (!parameters && count)) {
        return -1;
    }
    FILE *file = fopen(path, "wb");
    if (!file) {
        return -1;
    }
    bool ok = fwrite(kMagic, sizeof(kMagic), 1, file) == 1 &&
              fwrite(&kVersion, sizeof(kVersion), 1, file) == 1 &&
              fwrite(config, config_bytes, 1, file) == 1;
    for (size_t i = 0; ok && i < count; ++i) {
        const vitb200_parameter *parameter = parameters[i];
        size_t elements = parameter->value.ndim ? 1 : 0;
        for (size_t d = 0; d < parameter->value.ndim; ++d) {
            elements *= parameter->value.shape[d];
        }
        const size_t bytes = elements * sizeof(float);
        ok = fwrite(&elements, sizeof(elements), 1, file) == 1 &&
             fwrite(&parameter->step, sizeof(parameter->step), 1, file) == 1;
        const void *tensors[3] = {parameter->value.data, parameter->m, parameter->v};
        for (int t = 0; ok && t < 3; ++t) {
            if (!coherent_owns(tensors[t])) {
                // Plain host memory (a model created before the backend was
                // enabled): written as it is.
                ok = fwrite(tensors[t], 1, bytes, file) == bytes;
                counters->from_mirrors += bytes;
                continue;
            }
            const float *device = coherent_current_device(tensors[t], stream);
            ok = write_tensor(file, device, tensors[t], bytes, staging, stream, counters);
        }
    }
    if (fclose(file) != 0) {
        ok = false;
    }
    return ok ? 0 : -1;
}

int checkpoint_load(const char *path, const void *config, size_t config_bytes,
                    vitb200_parameter *const *parameters, size_t count,
                    cudaStream_t stream) {
    Staging staging;
    if (!staging.ok || !path || !config || (!parameters && count)) {
        return -1;
    }
    FILE *file = fopen(path, "rb");
    if (!file) {
        return -1;
    }
    char magic[sizeof(kMagic)];
    uint32_t version = 0;
    // The configuration must be the model's own, byte for byte, as in the
    // reference's reader (src/vit.c:1257-1258).
    char stored[256];
    bool ok = config_bytes <= sizeof(stored) &&
              fread(magic, sizeof(magic), 1, file) == 1 &&
              memcmp(magic, kMagic, sizeof(kMagic)) == 0 &&
              fread(&version, sizeof(version), 1, file) == 1 && version == kVersion &&
              fread(stored, config_bytes, 1, file) == 1 &&
              memcmp(stored, config, config_bytes) == 0;
    for (size_t i = 0; ok && i < count; ++i) {
        vitb200_parameter *parameter = parameters[i];
        size_t expected = parameter->value.ndim ? 1 : 0;
        for (size_t d = 0; d < parameter->value.ndim; ++d) {
            expected *= parameter->value.shape[d];
        }
        size_t elements = 0, step = 0;
        ok = fread(&elements, sizeof(elements), 1, file) == 1 && elements == expected &&
             fread(&step, sizeof(step), 1, file) == 1;
        const size_t bytes = elements * sizeof(float);
        void *tensors[3] = {parameter->value.data, parameter->m, parameter->v};
        for (int t = 0; ok && t < 3; ++t) {
            if (!coherent_owns(tensors[t])) {
                ok = fread(tensors[t], 1, bytes, file) == bytes;
                continue;
            }
            float *device = device_view(tensors[t], Access::Overwrite, stream);
            ok = device && read_tensor(file, device, bytes, staging, stream);
        }
        if (ok) {
            parameter->step = step;
        }
    }
    fclose(file);
    // The staging blocks go away with this call: the copies must be done.
    if (cudaStreamSynchronize(stream) != cudaSuccess) {
        ok = false;
    }
    return ok ? 0 : -1;
}

}  // namespace vitb200
