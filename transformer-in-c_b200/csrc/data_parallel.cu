#include "data_parallel.h"
#include "coherence.h"

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
    int (*comm_get_async_error)(NcclComm, int *) = nullptr;
    int (*comm_abort)(NcclComm) = nullptr;
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
        a.comm_get_async_error = reinterpret_cast<decltype(a.comm_get_async_error)>(
            find("ncclCommGetAsyncError"));
        a.comm_abort = reinterpret_cast<decltype(a.comm_abort)>(find("ncclCommAbort"));
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
    bool reduced = false;   // handed to NCCL, or complete inside the arena, this step
    // Written by an op that does not report through dp_gradient_produced: its
    // writers cannot be counted, so it is exchanged at the optimiser call.
    bool other_writers = false;
    size_t offset = 0;      // arena mode: position inside the arena, in floats
    size_t slot = 0;        // arena mode: floats reserved (a multiple of a page)
};

struct Pending {
    float *device;
    size_t count;
};

// Ranges are handed to NCCL once they hold this much, so the exchange starts
// while the backward pass is still running but launch overheads stay
// amortised; the last range goes out as soon as the last gradient is complete.
constexpr size_t kBucketBytes = size_t(4) << 20;

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
    // Flat exchange.  Step 2 records the order in which the gradients become
    // complete; at its optimiser call their device buffers move, in that
    // order, into one allocation (the arena), and from then on contiguous
    // ranges of it are all-reduced as their last gradient becomes complete:
    // a handful of NCCL calls per step instead of one per tensor.
    std::vector<const void *> completion_order;   // being recorded this step
    std::vector<const void *> arena_order;
    float *arena = nullptr;
    size_t arena_floats = 0;
    bool arena_failed = false;   // do not try again
    size_t complete_prefix = 0;  // gradients of arena_order complete this step
    size_t complete_floats = 0;  // arena floats they cover
    size_t sent_floats = 0;      // arena floats handed to NCCL this step
    unsigned long long arena_ranges = 0;
    int error = 0;   // first asynchronous NCCL error seen; the exchange is over then
};

namespace {

constexpr size_t kPageFloats = 1024;

void wait_for_compute(DataParallel *dp) {
    check_cuda(cudaEventRecord(dp->produced, dp->compute), "cudaEventRecord");
    check_cuda(cudaStreamWaitEvent(dp->exchange, dp->produced, 0),
               "cudaStreamWaitEvent");
}

void flush(DataParallel *dp) {
    if (dp->pending.empty()) {
        return;
    }
    wait_for_compute(dp);
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

// All-reduces arena floats [sent, upto) in one call.
void send_range(DataParallel *dp, size_t upto) {
    if (upto <= dp->sent_floats) {
        return;
    }
    wait_for_compute(dp);
    float *range = dp->arena + dp->sent_floats;
    const size_t count = upto - dp->sent_floats;
    check_nccl(nccl().all_reduce(range, range, count, kNcclFloat32, kNcclSum,
                                 dp->comm, dp->exchange),
               "ncclAllReduce");
    dp->all_reduce_calls += 1;
    dp->arena_ranges += 1;
    dp->bytes += count * sizeof(float);
    dp->sent_floats = upto;
}

// Gives every gradient its own device buffer back and frees the arena.
void drop_arena(DataParallel *dp) {
    if (!dp->arena) {
        return;
    }
    for (const void *host : dp->arena_order) {
        // False for tensors that are gone already: nothing to move.
        coherent_place_device_buffer(host, nullptr, dp->compute);
    }
    check_cuda(cudaStreamSynchronize(dp->compute), "cudaStreamSynchronize");
    check_cuda(cudaStreamSynchronize(dp->exchange), "cudaStreamSynchronize");
    coherent_external_range(dp->arena, dp->arena_floats * sizeof(float), false);
    cudaFree(dp->arena);
    dp->arena = nullptr;
    dp->arena_floats = 0;
    dp->arena_order.clear();
}

// Step 2's optimiser call: the completion order is known for every
// parameter exactly once -> move the gradients into one allocation.
void build_arena(DataParallel *dp, const void *const *host_grads, size_t parameters) {
    if (dp->arena || dp->arena_failed ||
        dp->completion_order.size() != parameters) {
        return;
    }
    size_t total = 0;
    for (const void *host : dp->completion_order) {
        auto found = dp->gradients.find(host);
        const size_t bytes = coherent_device_bytes(host);
        if (found == dp->gradients.end() || found->second.slot != 0 || bytes == 0) {
            for (auto &entry : dp->gradients) {
                entry.second.slot = 0;
            }
            return;   // not a permutation of the parameter list
        }
        found->second.slot =
            (bytes / sizeof(float) + kPageFloats - 1) / kPageFloats * kPageFloats;
        found->second.offset = total;
        total += found->second.slot;
    }
    (void)host_grads;
    void *memory = nullptr;
    if (cudaMalloc(&memory, total * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        dp->arena_failed = true;
        return;
    }
    dp->arena = static_cast<float *>(memory);
    dp->arena_floats = total;
    check_cuda(cudaMemsetAsync(dp->arena, 0, total * sizeof(float), dp->compute),
               "cudaMemsetAsync");
    coherent_external_range(dp->arena, total * sizeof(float), true);
    dp->arena_order = dp->completion_order;
    for (const void *host : dp->arena_order) {
        Gradient &gradient = dp->gradients[host];
        if (!coherent_place_device_buffer(host, dp->arena + gradient.offset,
                                          dp->compute)) {
            drop_arena(dp);
            dp->arena_failed = true;
            return;
        }
        gradient.device = dp->arena + gradient.offset;
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
    const char *flat = getenv("VITB200_DP_FLAT");
    dp->arena_failed = flat && atoi(flat) == 0;   // per-tensor exchange only
    return dp;
}

void dp_destroy(DataParallel *dp) {
    if (!dp) {
        return;
    }
    if (dp->exchange) {
        cudaStreamSynchronize(dp->exchange);
    }
    if (dp->compute && dp->exchange) {
        drop_arena(dp);
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

int dp_poll(DataParallel *dp) {
    if (!dp || dp->error || !dp->comm || !nccl().comm_get_async_error) {
        return dp ? dp->error : 0;
    }
    int status = kNcclSuccess;
    if (nccl().comm_get_async_error(dp->comm, &status) != kNcclSuccess) {
        status = 1;   // unhandled error querying the communicator
    }
    if (status != kNcclSuccess) {
        fprintf(stderr, "vitb200: the gradient exchange failed: %s\n",
                nccl().error_string ? nccl().error_string(status) : "NCCL error");
        dp->error = status;
        // Frees the communicator's resources and ends its kernels, so that
        // this rank's stream drains instead of waiting for a peer for ever.
        if (nccl().comm_abort) {
            nccl().comm_abort(dp->comm);
        }
        dp->comm = nullptr;
    }
    return dp->error;
}

int dp_status(const DataParallel *dp) {
    return dp ? dp->error : 0;
}

void dp_gradient_touched(DataParallel *dp, const void *host_grad) {
    if (!dp || dp->world == 1) {
        return;
    }
    auto found = dp->gradients.find(host_grad);
    if (found == dp->gradients.end()) {
        return;
    }
    Gradient &gradient = found->second;
    if (gradient.reduced) {
        // Its sum is already on the wire without this contribution.
        fprintf(stderr,
                "vitb200: a parameter gradient was written by an op outside the "
                "exchange's bookkeeping after its all-reduce had started\n");
        abort();
    }
    gradient.other_writers = true;
    gradient.overlap = false;
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
    const bool complete = gradient.expected_producers > 0 &&
                          gradient.producers_this_step == gradient.expected_producers;
    if (complete && !dp->arena) {
        dp->completion_order.push_back(host_grad);
    }
    if (!complete || !gradient.overlap || gradient.reduced ||
        gradient.count != count) {
        return;
    }
    if (dp->arena) {
        if (device_grad != dp->arena + gradient.offset) {
            // The buffer has left the arena (it should not): the optimiser
            // call notices and falls back to the per-tensor exchange.
            return;
        }
        gradient.reduced = true;
        dp->overlapped += 1;
        // Extend the prefix of complete gradients; ranges go out whole.
        while (dp->complete_prefix < dp->arena_order.size()) {
            const Gradient &next = dp->gradients[dp->arena_order[dp->complete_prefix]];
            if (!next.reduced) {
                break;
            }
            dp->complete_floats = next.offset + next.slot;
            dp->complete_prefix += 1;
        }
        const bool everything = dp->complete_prefix == dp->arena_order.size();
        if (everything || (dp->complete_floats - dp->sent_floats) * sizeof(float) >=
                              kBucketBytes) {
            send_range(dp, dp->complete_floats);
        }
        return;
    }
    gradient.device = device_grad;
    gradient.reduced = true;
    dp->overlapped += 1;
    enqueue(dp, device_grad, count);
}

float dp_before_optimizer(DataParallel *dp, const void *const *host_grads,
                          float *const *device_grads, const size_t *counts,
                          size_t parameters) {
    if (!dp || dp->world == 1) {
        return 1.0f;
    }
    dp->optimizer_calls += 1;
    // The arena serves exactly the parameter list it was built for, with
    // every buffer still inside it.
    if (dp->arena) {
        bool intact = parameters == dp->arena_order.size();
        for (size_t i = 0; intact && i < parameters; ++i) {
            auto found = dp->gradients.find(host_grads[i]);
            intact = found != dp->gradients.end() && found->second.slot != 0 &&
                     device_grads[i] == dp->arena + found->second.offset;
        }
        if (!intact) {
            if (dp->sent_floats != 0) {
                fprintf(stderr, "vitb200: the parameter list changed after part of "
                                "its gradients had been exchanged\n");
                abort();
            }
            drop_arena(dp);
            dp->gradients.clear();
            dp->optimizer_calls = 1;
        }
    }
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
            if (!dp->arena) {
                enqueue(dp, device_grads[i], counts[i]);
            }
        }
        // Once two steps in a row have written a gradient the same number of
        // times (one op per micro-batch), it is exchanged as soon as the last
        // of those ops has been enqueued.
        gradient.overlap = dp->optimizer_calls >= 2 && !gradient.other_writers &&
                           gradient.producers_this_step >= 1 &&
                           gradient.producers_this_step ==
                               gradient.expected_producers;
        gradient.expected_producers = gradient.producers_this_step;
        if (!dp->arena) {
            gradient.device = device_grads[i];
        }
        gradient.count = counts[i];
        gradient.producers_this_step = 0;
        gradient.reduced = false;
    }
    if (dp->arena) {
        send_range(dp, dp->arena_floats);   // whatever has not gone out yet
        dp->complete_prefix = 0;
        dp->complete_floats = 0;
        dp->sent_floats = 0;
    } else {
        flush(dp);
    }
    check_cuda(cudaEventRecord(dp->exchanged, dp->exchange), "cudaEventRecord");
    check_cuda(cudaStreamWaitEvent(dp->compute, dp->exchanged, 0),
               "cudaStreamWaitEvent");
    if (!dp->arena && dp->optimizer_calls >= 2) {
        build_arena(dp, host_grads, parameters);
    }
    dp->completion_order.clear();
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

void dp_tensor_released(DataParallel *dp, const void *host_pointer) {
    if (!dp || dp->gradients.find(host_pointer) == dp->gradients.end()) {
        return;
    }
    // A parameter is going away: this model's schedule and arena are over.
    drop_arena(dp);
    dp->gradients.clear();
    dp->completion_order.clear();
    dp->optimizer_calls = 0;
    dp->complete_prefix = 0;
    dp->complete_floats = 0;
    dp->sent_floats = 0;
}

void dp_counters(const DataParallel *dp, unsigned long long *all_reduce_calls,
                 unsigned long long *overlapped_tensors,
                 unsigned long long *late_tensors, unsigned long long *bytes) {
    if (all_reduce_calls) *all_reduce_calls = dp ? dp->all_reduce_calls : 0;
    if (overlapped_tensors) *overlapped_tensors = dp ? dp->overlapped : 0;
    if (late_tensors) *late_tensors = dp ? dp->late : 0;
    if (bytes) *bytes = dp ? dp->bytes : 0;
}

unsigned long long dp_flat_ranges(const DataParallel *dp) {
    return dp ? dp->arena_ranges : 0;
}

}  // namespace vitb200
