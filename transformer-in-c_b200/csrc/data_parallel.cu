#include "data_parallel.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <unordered_map>
#include <vector>

namespace vitb200 {
namespace {

// The handful of NCCL declarations used here (NCCL's public C API), so the
// library builds and loads without NCCL installed.
struct ncclComm;
typedef ncclComm *NcclComm;
struct NcclUniqueId {
    char internal[128];
};
constexpr int kNcclSuccess = 0;
constexpr int kNcclFloat32 = 7;
constexpr int kNcclSum = 0;

struct NcclApi {
    int (*get_unique_id)(NcclUniqueId *) = nullptr;
    int (*comm_init_rank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
    int (*comm_destroy)(NcclComm) = nullptr;
    int (*all_reduce)(const void *, void *, size_t, int, int, NcclComm,
                      cudaStream_t) = nullptr;
    int (*group_start)() = nullptr;
    int (*group_end)() = nullptr;
    const char *(*error_string)(int) = nullptr;
    bool loaded = false;
};

NcclApi &nccl() {
    static NcclApi api = []() {
        NcclApi a;
        void *handle = nullptr;
        for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
            handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (handle) {
                break;
            }
        }
        if (!handle) {
            return a;
        }
        auto find = [&](const char *symbol) { return dlsym(handle, symbol); };
        a.get_unique_id = reinterpret_cast<decltype(a.get_unique_id)>(find("ncclGetUniqueId"));
        a.comm_init_rank = reinterpret_cast<decltype(a.comm_init_rank)>(find("ncclCommInitRank"));
        a.comm_destroy = reinterpret_cast<decltype(a.comm_destroy)>(find("ncclCommDestroy"));
        a.all_reduce = reinterpret_cast<decltype(a.all_reduce)>(find("ncclAllReduce"));
        a.group_start = reinterpret_cast<decltype(a.group_start)>(find("ncclGroupStart"));
        a.group_end = reinterpret_cast<decltype(a.group_end)>(find("ncclGroupEnd"));
        a.error_string = reinterpret_cast<decltype(a.error_string)>(find("ncclGetErrorString"));
        a.loaded = a.get_unique_id && a.comm_init_rank && a.comm_destroy &&
                   a.all_reduce && a.group_start && a.group_end;
        return a;
    }();
    return api;
}

void check_nccl(int status, const char *what) {
    if (status != kNcclSuccess) {
        fprintf(stderr, "vitb200: %s failed: %s\n", what,
                nccl().error_string ? nccl().error_string(status) : "NCCL error");
        abort();
    }
}

void check_cuda(cudaError_t status, const char *what) {
    if (status != cudaSuccess) {
        fprintf(stderr, "vitb200: %s failed: %s\n", what,
                cudaGetErrorString(status));
        abort();
    }
}

struct Gradient {
    float *device = nullptr;
    size_t count = 0;
    int producers_this_step = 0;
    int expected_producers = 0;  // producers seen in the previous step
    bool overlap = false;   // the producer count is known: safe to reduce early
    bool reduced = false;
};

struct Pending {
    float *device;
    size_t count;
};

// Buckets are flushed once they hold this much, so the exchange starts while
// the backward pass is still running but launch overheads stay amortised.
constexpr size_t kBucketBytes = size_t(2) << 20;

}  // namespace

struct DataParallel {
    int rank = 0;
    int world = 1;
    NcclComm comm = nullptr;
    cudaStream_t compute = nullptr;
    cudaStream_t exchange = nullptr;
    cudaEvent_t produced = nullptr;
    cudaEvent_t exchanged = nullptr;
    std::unordered_map<const void *, Gradient> gradients;
    std::vector<Pending> pending;
    size_t pending_bytes = 0;
    unsigned long long optimizer_calls = 0;
    unsigned long long all_reduce_calls = 0;
    unsigned long long overlapped = 0;
    unsigned long long late = 0;
    unsigned long long bytes = 0;
};

namespace {

void flush(DataParallel *dp) {
    if (dp->pending.empty()) {
        return;
    }
    check_cuda(cudaEventRecord(dp->produced, dp->compute), "cudaEventRecord");
    check_cuda(cudaStreamWaitEvent(dp->exchange, dp->produced, 0),
               "cudaStreamWaitEvent");
    check_nccl(nccl().group_start(), "ncclGroupStart");
    for (const Pending &item : dp->pending) {
        check_nccl(nccl().all_reduce(item.device, item.device, item.count,
                                     kNcclFloat32, kNcclSum, dp->comm,
                                     dp->exchange),
                   "ncclAllReduce");
        dp->all_reduce_calls += 1;
        dp->bytes += item.count * sizeof(float);
    }
    check_nccl(nccl().group_end(), "ncclGroupEnd");
    dp->pending.clear();
    dp->pending_bytes = 0;
}

void enqueue(DataParallel *dp, float *device, size_t count) {
    dp->pending.push_back(Pending{device, count});
    dp->pending_bytes += count * sizeof(float);
    if (dp->pending_bytes >= kBucketBytes) {
        flush(dp);
    }
}

}  // namespace

int dp_unique_id(void *out128) {
    if (!nccl().loaded || !out128) {
        return -1;
    }
    NcclUniqueId id;
    if (nccl().get_unique_id(&id) != kNcclSuccess) {
        return -1;
    }
    memcpy(out128, id.internal, sizeof(id.internal));
    return 0;
}

DataParallel *dp_create(int rank, int world, const void *id128,
                        cudaStream_t compute_stream) {
    if (!nccl().loaded || world < 1 || rank < 0 || rank >= world || !id128) {
        return nullptr;
    }
    DataParallel *dp = new DataParallel();
    dp->rank = rank;
    dp->world = world;
    dp->compute = compute_stream;
    NcclUniqueId id;
    memcpy(id.internal, id128, sizeof(id.internal));
    if (nccl().comm_init_rank(&dp->comm, world, id, rank) != kNcclSuccess ||
        cudaStreamCreateWithFlags(&dp->exchange, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&dp->produced, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&dp->exchanged, cudaEventDisableTiming) != cudaSuccess) {
        dp_destroy(dp);
        return nullptr;
    }
    return dp;
}

void dp_destroy(DataParallel *dp) {
    if (!dp) {
        return;
    }
    if (dp->exchange) {
        cudaStreamSynchronize(dp->exchange);
    }
    if (dp->comm) {
        nccl().comm_destroy(dp->comm);
    }
    if (dp->produced) {
        cudaEventDestroy(dp->produced);
    }
    if (dp->exchanged) {
        cudaEventDestroy(dp->exchanged);
    }
    if (dp->exchange) {
        cudaStreamDestroy(dp->exchange);
    }
    delete dp;
}

int dp_world(const DataParallel *dp) {
    return dp ? dp->world : 1;
}

void dp_gradient_produced(DataParallel *dp, const void *host_grad,
                          float *device_grad, size_t count) {
    if (!dp || dp->world == 1) {
        return;
    }
    auto found = dp->gradients.find(host_grad);
    if (found == dp->gradients.end()) {
        return;
    }
    Gradient &gradient = found->second;
    gradient.producers_this_step += 1;
    if (gradient.overlap && !gradient.reduced && gradient.count == count &&
        gradient.producers_this_step == gradient.expected_producers) {
        gradient.device = device_grad;
        gradient.reduced = true;
        dp->overlapped += 1;
        enqueue(dp, device_grad, count);
    }
}

float dp_before_optimizer(DataParallel *dp, const void *const *host_grads,
                          float *const *device_grads, const size_t *counts,
                          size_t parameters) {
    if (!dp || dp->world == 1) {
        return 1.0f;
    }
    dp->optimizer_calls += 1;
    for (size_t i = 0; i < parameters; ++i) {
        Gradient &gradient = dp->gradients[host_grads[i]];
        if (gradient.reduced &&
            gradient.producers_this_step > gradient.expected_producers) {
            // Another op added to a gradient after it had been exchanged: the
            // sum on the wire is incomplete.  This model never does it; refuse
            // to continue rather than train on wrong gradients.
            fprintf(stderr,
                    "vitb200: a parameter gradient was written again after its "
                    "all-reduce had started\n");
            abort();
        }
        if (!gradient.reduced) {
            dp->late += 1;
            enqueue(dp, device_grads[i], counts[i]);
        }
        // Once two steps in a row have written a gradient the same number of
        // times (one op per micro-batch), it is exchanged as soon as the last
        // of those ops has been enqueued.
        gradient.overlap = dp->optimizer_calls >= 2 &&
                           gradient.producers_this_step >= 1 &&
                           gradient.producers_this_step ==
                               gradient.expected_producers;
        gradient.expected_producers = gradient.producers_this_step;
        gradient.device = device_grads[i];
        gradient.count = counts[i];
        gradient.producers_this_step = 0;
        gradient.reduced = false;
    }
    flush(dp);
    check_cuda(cudaEventRecord(dp->exchanged, dp->exchange), "cudaEventRecord");
    check_cuda(cudaStreamWaitEvent(dp->compute, dp->exchanged, 0),
               "cudaStreamWaitEvent");
    return 1.0f / float(dp->world);
}

void dp_forget_schedule(DataParallel *dp) {
    if (!dp) {
        return;
    }
    dp->optimizer_calls = 0;
    for (auto &entry : dp->gradients) {
        entry.second.overlap = false;
        entry.second.expected_producers = 0;
    }
}

void dp_counters(const DataParallel *dp, unsigned long long *all_reduce_calls,
                 unsigned long long *overlapped_tensors,
                 unsigned long long *late_tensors, unsigned long long *bytes) {
    if (all_reduce_calls) *all_reduce_calls = dp ? dp->all_reduce_calls : 0;
    if (overlapped_tensors) *overlapped_tensors = dp ? dp->overlapped : 0;
    if (late_tensors) *late_tensors = dp ? dp->late : 0;
    if (bytes) *bytes = dp ? dp->bytes : 0;
}

}  // namespace vitb200
