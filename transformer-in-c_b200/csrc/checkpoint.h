// Device-to-file and file-to-device checkpoints in the host's own format
// (checkpoint.cu).
#pragma once

#include "../../include/vitb200_host_abi.h"

#include <cstddef>
#include <cuda_runtime.h>

namespace vitb200 {

struct CheckpointCounters {
    size_t from_device;    // bytes that went device -> staging -> file
    size_t from_mirrors;   // bytes written from host memory that was current
};

// 0 on success, -1 on any failure (the file may be incomplete then).
int checkpoint_save(const char *path, const void *config, size_t config_bytes,
                    vitb200_parameter *const *parameters, size_t count,
                    cudaStream_t stream, CheckpointCounters *counters);
int checkpoint_load(const char *path, const void *config, size_t config_bytes,
                    vitb200_parameter *const *parameters, size_t count,
                    cudaStream_t stream);

}  // namespace vitb200
