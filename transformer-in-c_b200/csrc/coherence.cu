#include "coherence.h"

#include <atomic>

#include <cerrno>
#include <csignal>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>

#include <sys/mman.h>
#include <ucontext.h>
#include <unistd.h>

namespace vitb200 {
namespace {

enum class Owner { Host, Shared, Device };

struct LazyDefinition;

struct Region {
    LazyDefinition *lazy = nullptr;    // this buffer's contents are defined lazily
    LazyDefinition *feeds = nullptr;   // first of the definitions reading this buffer
    char *mirror = nullptr;
    size_t bytes = 0;         // size the host asked for
    size_t mapped = 0;        // page-rounded size of the mapping
    float *device = nullptr;  // created on first device use
    Owner owner = Owner::Host;
    bool zero_pending = false;  // device contents are an unmaterialised zero fill
    // The device buffer a batched fill (coherent_zero_fill_batch) has already
    // zeroed for the pending fill; materialising it then costs nothing.
    float *zeroed = nullptr;
    unsigned uploads = 0;       // host-to-device copies so far
    bool pinned = false;        // mirror registered with the driver
    // A page-locked mirror is uploaded by DMA that may still be reading it
    // after the call returns: recorded behind the copy, waited for before the
    // host gets to write the mirror again.
    cudaEvent_t uploaded = nullptr;
    bool upload_in_flight = false;
    // Copy of the device contents on its way to page-locked staging memory
    // (coherent_prefetch_host); valid until the device writes the buffer again.
    void *staging = nullptr;
    cudaEvent_t fetched = nullptr;
    bool prefetched = false;
    // Overlapped uploads (see upload_beside_compute): the device buffer the
    // previous upload went to, and the point of the compute stream after
    // which nothing reads it any more.
    float *spare = nullptr;
    cudaEvent_t spare_free = nullptr;
};

// Process-global on purpose: the host keeps the release function inside every
// tensor and may call it long after the backend object is gone.
std::map<uintptr_t, Region> &registry() {
    static std::map<uintptr_t, Region> *regions =
        new std::map<uintptr_t, Region>();
    return *regions;
}

CoherenceStats g_stats = {};
cudaStream_t g_stream = nullptr;
cudaStream_t g_copy_stream = nullptr;   // device-to-host prefetches
cudaEvent_t g_produced = nullptr;       // orders a prefetch behind its producer
void (*g_flush)(void) = nullptr;
int (*g_wait_poll)(void) = nullptr;
bool g_overlap_uploads = false;
struct sigaction g_previous_action;
bool g_handler_installed = false;
size_t g_page = 4096;

// Mirrors at least this large give their pages back to the kernel while the
// device owns the contents; they are re-populated on copy-back.
constexpr size_t kDropPagesThreshold = size_t(1) << 21;

// Largest buffer coherent_prefetch_host stages (it is meant for scalars and
// short vectors the host is known to read next).
constexpr size_t kPrefetchLimitBytes = 4096;

// Smallest input an upload beside the compute stream is set up for.
constexpr size_t kOverlapUploadBytes = size_t(1) << 18;

[[noreturn]] void die(const char *what, const char *detail) {
    fprintf(stderr, "vitb200: %s failed: %s\n", what, detail);
    abort();
}

void check(cudaError_t status, const char *what) {
    if (status != cudaSuccess) {
        die(what, cudaGetErrorString(status));
    }
}

void protect(Region &region, int protection) {
    if (mprotect(region.mirror, region.mapped, protection) != 0) {
        die("mprotect", strerror(errno));
    }
}

Region *find_base(const void *pointer) {
    auto &regions = registry();
    auto it = regions.find(reinterpret_cast<uintptr_t>(pointer));
    return it == regions.end() ? nullptr : &it->second;
}

Region *find_containing(uintptr_t address) {
    auto &regions = registry();
    auto it = regions.upper_bound(address);
    if (it == regions.begin()) {
        return nullptr;
    }
    --it;
    Region &region = it->second;
    return address < it->first + region.mapped ? &region : nullptr;
}

// Lowest and highest mirror addresses ever handed out.  Read without the
// single-thread assumption of the rest of this file: the stdio hooks are
// entered from any thread that writes a log line, and must be able to tell
// "not ours" without touching the registry.
std::atomic<uintptr_t> g_lowest_mirror{~uintptr_t(0)};
std::atomic<uintptr_t> g_highest_mirror{0};

void note_mirror_range(const void *mirror, size_t bytes) {
    const uintptr_t begin = reinterpret_cast<uintptr_t>(mirror);
    uintptr_t seen = g_lowest_mirror.load(std::memory_order_relaxed);
    while (begin < seen &&
           !g_lowest_mirror.compare_exchange_weak(seen, begin)) {
    }
    seen = g_highest_mirror.load(std::memory_order_relaxed);
    while (begin + bytes > seen &&
           !g_highest_mirror.compare_exchange_weak(seen, begin + bytes)) {
    }
}

// Device buffers of released tensors, kept for reuse by size: the host's
// evaluation entry points allocate and free a whole activation cache per call
// (reference src/vit.c:1371-1375), and cudaMalloc / cudaFree would otherwise
// dominate them.  Every kernel runs on one stream, so a recycled buffer cannot
// be touched by work enqueued before its previous owner was released.
std::multimap<size_t, float *> &buffer_pool() {
    static std::multimap<size_t, float *> *pool =
        new std::multimap<size_t, float *>();
    return *pool;
}
size_t g_pooled_bytes = 0;
constexpr size_t kPoolLimitBytes = size_t(8) << 30;

void ensure_device_buffer(Region &region) {
    if (region.device) {
        return;
    }
    auto &pool = buffer_pool();
    auto found = pool.find(region.mapped);
    if (found != pool.end()) {
        region.device = found->second;
        pool.erase(found);
        g_pooled_bytes -= region.mapped;
    } else {
        void *memory = nullptr;
        check(cudaMalloc(&memory, region.mapped), "cudaMalloc");
        region.device = static_cast<float *>(memory);
    }
    g_stats.device_bytes += region.mapped;
}

// A device buffer that outlived its region's use of it because pending
// definitions still read the old contents; shared by all of them.
struct Snapshot {
    float *device = nullptr;
    size_t bytes = 0;
    int references = 0;
};

// A buffer whose contents are a known function of (at most two) other
// buffers and have not been computed.  All definitions reading one source are
// chained from the source's `feeds` through `next_reader`.  If a source is
// about to be overwritten while definitions are still pending, its old device
// buffer moves into a Snapshot they share and the source continues with a
// fresh buffer.
struct LazyDefinition {
    LazyMaterialise function = nullptr;
    unsigned char arguments[64] = {};
    Region *output = nullptr;
    int sources = 0;
    Region *source[2] = {nullptr, nullptr};
    Snapshot *snapshot[2] = {nullptr, nullptr};
    LazyDefinition *next_reader[2] = {nullptr, nullptr};
};

// Device memory owned by somebody else (the gradient-exchange arena) that
// buffers may be placed in: never pooled, never freed here.
struct ExternalRange {
    uintptr_t begin, end;
};
std::vector<ExternalRange> &external_ranges() {
    static std::vector<ExternalRange> *ranges = new std::vector<ExternalRange>();
    return *ranges;
}

bool is_external(const void *device) {
    const uintptr_t address = reinterpret_cast<uintptr_t>(device);
    for (const ExternalRange &range : external_ranges()) {
        if (address >= range.begin && address < range.end) {
            return true;
        }
    }
    return false;
}

void recycle(float *device, size_t bytes) {
    if (is_external(device)) {
        return;
    }
    if (bytes > kPoolLimitBytes) {
        cudaFree(device);
        return;
    }
    // Over the limit the pool gives up buffers of other sizes first: what is
    // being released now is what the running workload allocates and will ask
    // for again, while the rest may be left over from a model that is gone.
    auto &pool = buffer_pool();
    while (g_pooled_bytes + bytes > kPoolLimitBytes && !pool.empty()) {
        auto victim = pool.begin();
        if (victim->first == bytes) {
            victim = pool.upper_bound(bytes);
            if (victim == pool.end()) {
                victim = pool.begin();
            }
        }
        cudaFree(victim->second);
        g_pooled_bytes -= victim->first;
        pool.erase(victim);
    }
    pool.emplace(bytes, device);
    g_pooled_bytes += bytes;
}

int reader_slot(const LazyDefinition *lazy, const Region *region) {
    return lazy->source[0] == region ? 0 : 1;
}

void unlink_reader(LazyDefinition *lazy, int slot) {
    Region *region = lazy->source[slot];
    LazyDefinition **link = &region->feeds;
    while (*link && *link != lazy) {
        link = &(*link)->next_reader[reader_slot(*link, region)];
    }
    if (*link) {
        *link = lazy->next_reader[slot];
    }
    lazy->source[slot] = nullptr;
    lazy->next_reader[slot] = nullptr;
}

// Forgets a definition without computing it (its output is being redefined).
void drop_lazy(LazyDefinition *lazy) {
    for (int i = 0; i < lazy->sources; ++i) {
        if (lazy->source[i]) {
            unlink_reader(lazy, i);
        }
        if (lazy->snapshot[i] && --lazy->snapshot[i]->references == 0) {
            recycle(lazy->snapshot[i]->device, lazy->snapshot[i]->bytes);
            delete lazy->snapshot[i];
        }
    }
    if (lazy->output) {
        lazy->output->lazy = nullptr;
    }
    delete lazy;
    g_stats.lazy_dropped += 1;
}

const float *source_device(const LazyDefinition *lazy, int slot) {
    return lazy->snapshot[slot] ? lazy->snapshot[slot]->device
                                : lazy->source[slot]->device;
}

// Computes a pending definition into its output buffer.
void materialise_lazy(LazyDefinition *lazy, cudaStream_t stream) {
    ensure_device_buffer(*lazy->output);
    float *inputs[2] = {nullptr, nullptr};
    for (int i = 0; i < lazy->sources; ++i) {
        inputs[i] = const_cast<float *>(source_device(lazy, i));
    }
    lazy->function(lazy->arguments, lazy->output->device, inputs, stream);
    g_stats.lazy_materialised += 1;
    g_stats.lazy_dropped -= 1;   // drop_lazy below counts it again
    drop_lazy(lazy);
}

// Computes every definition that reads `region` (it is about to be modified
// in place).
void materialise_readers(Region &region, cudaStream_t stream) {
    while (region.feeds) {
        materialise_lazy(region.feeds, stream);
    }
}

// True when copying `region` costs much less memory traffic than computing the
// definitions that read it.
bool copy_beats_readers(const Region &region) {
    size_t readers = 0;
    for (const LazyDefinition *lazy = region.feeds; lazy;
         lazy = lazy->next_reader[reader_slot(lazy, &region)]) {
        readers += lazy->output ? lazy->output->bytes : 0;
    }
    return readers / 8 >= region.bytes;
}

// The source is about to be replaced wholesale: the pending readers keep the
// old buffer, the region goes on without one.
void detach_source(Region &region) {
    Snapshot *snapshot = new Snapshot();
    snapshot->device = region.device;
    snapshot->bytes = region.mapped;
    for (LazyDefinition *lazy = region.feeds; lazy;) {
        const int slot = reader_slot(lazy, &region);
        LazyDefinition *next = lazy->next_reader[slot];
        lazy->snapshot[slot] = snapshot;
        lazy->source[slot] = nullptr;
        lazy->next_reader[slot] = nullptr;
        snapshot->references += 1;
        lazy = next;
    }
    region.feeds = nullptr;
    g_stats.device_bytes -= region.mapped;
    region.device = nullptr;
}

// Definition of an alias: the output is a plain copy of its source.
void materialise_copy(const void *arguments, float *output,
                      float *const *sources, cudaStream_t stream) {
    size_t bytes = 0;
    memcpy(&bytes, arguments, sizeof(bytes));
    check(cudaMemcpyAsync(output, sources[0], bytes, cudaMemcpyDeviceToDevice,
                          stream),
          "cudaMemcpyAsync(device to device)");
}

bool is_alias(const Region &region) {
    return region.lazy && region.lazy->function == materialise_copy;
}

void materialise_zero(Region &region, cudaStream_t stream) {
    if (region.zero_pending) {
        if (region.zeroed && region.zeroed == region.device) {
            g_stats.zero_fills_batched += 1;
        } else {
            check(cudaMemsetAsync(region.device, 0, region.bytes, stream),
                  "cudaMemsetAsync");
            g_stats.zero_fills_materialised += 1;
        }
        region.zero_pending = false;
        region.zeroed = nullptr;
    }
}

// Up to kZeroBatch buffers cleared by one launch: a block per 4096 floats.
constexpr int kZeroBatch = 120;
constexpr unsigned kZeroFloatsPerBlock = 4096;

struct ZeroBatch {
    float *buffer[kZeroBatch];
    unsigned floats[kZeroBatch];
};

__global__ void __launch_bounds__(256) zero_batch_kernel(const ZeroBatch batch) {
    float *buffer = batch.buffer[blockIdx.y];
    const unsigned floats = batch.floats[blockIdx.y];
    const unsigned begin = blockIdx.x * kZeroFloatsPerBlock;
    const unsigned end = min(floats, begin + kZeroFloatsPerBlock);
    for (unsigned i = begin + threadIdx.x; i < end; i += blockDim.x) {
        buffer[i] = 0.0f;
    }
}

// Brings the mirror up to date and hands ownership back to the host side.
// `for_write` selects HOST (exclusive) over SHARED (both valid).
// Blocks until the event has happened.  With a poll hook installed the wait
// spins and gives the hook a chance to notice that the event can never happen
// (a dead peer of a gradient exchange); the hook's non-zero answer ends it.
void wait_for(cudaEvent_t event) {
    if (g_wait_poll) {
        unsigned spins = 0;
        while (cudaEventQuery(event) == cudaErrorNotReady) {
            if ((++spins & 1023u) == 0 && g_wait_poll() != 0) {
                break;
            }
        }
        cudaGetLastError();
    }
    check(cudaEventSynchronize(event), "cudaEventSynchronize");
}

void wait_for_upload(Region &region) {
    if (region.upload_in_flight) {
        wait_for(region.uploaded);
        region.upload_in_flight = false;
    }
}

void serve_host_access(Region &region, bool for_write) {
    if (region.feeds && for_write) {
        materialise_readers(region, g_stream);
    }
    if (region.owner == Owner::Device) {
        if (g_flush) {
            g_flush();
        }
        if (region.prefetched && !region.lazy && !region.zero_pending) {
            // The contents are already on their way: wait for that copy alone,
            // not for everything queued behind the kernel that produced them.
            wait_for(region.fetched);
            region.prefetched = false;
            protect(region, PROT_READ | PROT_WRITE);
            memcpy(region.mirror, region.staging, region.bytes);
            g_stats.device_to_host_copies += 1;
            g_stats.device_to_host_bytes += region.bytes;
            g_stats.prefetched_reads += 1;
            if (for_write) {
                region.owner = Owner::Host;
            } else {
                protect(region, PROT_READ);
                region.owner = Owner::Shared;
            }
            return;
        }
        if (region.lazy) {
            materialise_lazy(region.lazy, g_stream);
        }
        ensure_device_buffer(region);
        materialise_zero(region, g_stream);
        check(cudaStreamSynchronize(g_stream), "cudaStreamSynchronize");
        protect(region, PROT_READ | PROT_WRITE);
        check(cudaMemcpy(region.mirror, region.device, region.bytes,
                         cudaMemcpyDeviceToHost),
              "cudaMemcpy(device to host)");
        g_stats.device_to_host_copies += 1;
        g_stats.device_to_host_bytes += region.bytes;
        if (for_write) {
            region.owner = Owner::Host;
        } else {
            protect(region, PROT_READ);
            region.owner = Owner::Shared;
        }
        return;
    }
    if (region.owner == Owner::Shared && for_write) {
        // Queued kernels may still want the device copy as it is now; they
        // read device memory, which a host write to the mirror cannot disturb,
        // but anything not yet launched must go out before the next upload.
        if (g_flush) {
            g_flush();
        }
        wait_for_upload(region);
        protect(region, PROT_READ | PROT_WRITE);
        region.owner = Owner::Host;
    }
}

void on_fault(int signal_number, siginfo_t *info, void *context) {
    const uintptr_t address = reinterpret_cast<uintptr_t>(info->si_addr);
    Region *region = find_containing(address);
    if (region && region->owner != Owner::Host) {
        bool is_write = true;
#if defined(__x86_64__)
        const ucontext_t *machine = static_cast<const ucontext_t *>(context);
        is_write = (machine->uc_mcontext.gregs[REG_ERR] & 0x2) != 0;
#endif
        g_stats.faults_served += 1;
        serve_host_access(*region, is_write);
        return;
    }
    // Not ours: behave as if we had never been installed.
    if (g_previous_action.sa_flags & SA_SIGINFO) {
        if (g_previous_action.sa_sigaction) {
            g_previous_action.sa_sigaction(signal_number, info, context);
            return;
        }
    } else if (g_previous_action.sa_handler != SIG_DFL &&
               g_previous_action.sa_handler != SIG_IGN) {
        g_previous_action.sa_handler(signal_number);
        return;
    }
    signal(signal_number, SIG_DFL);
}

}  // namespace

void coherence_install_fault_handler() {
    if (g_handler_installed) {
        return;
    }
    g_page = static_cast<size_t>(sysconf(_SC_PAGESIZE));
    struct sigaction action;
    memset(&action, 0, sizeof(action));
    action.sa_sigaction = on_fault;
    action.sa_flags = SA_SIGINFO | SA_NODEFER;
    sigemptyset(&action.sa_mask);
    if (sigaction(SIGSEGV, &action, &g_previous_action) != 0) {
        die("sigaction", strerror(errno));
    }
    g_handler_installed = true;
}

void coherence_set_stream(cudaStream_t stream, void (*flush)(void)) {
    g_stream = stream;
    g_flush = flush;
}

void (*g_released)(const void *) = nullptr;

void coherence_set_release_hook(void (*released)(const void *)) {
    g_released = released;
}

void *coherent_allocate(void *context, size_t bytes) {
    (void)context;
    if (bytes == 0) {
        return nullptr;
    }
    coherence_install_fault_handler();
    const size_t mapped = (bytes + g_page - 1) / g_page * g_page;
    void *mirror = mmap(nullptr, mapped, PROT_READ | PROT_WRITE,
                        MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (mirror == MAP_FAILED) {
        return nullptr;
    }
    Region region;
    region.mirror = static_cast<char *>(mirror);
    region.bytes = bytes;
    region.mapped = mapped;
    registry()[reinterpret_cast<uintptr_t>(mirror)] = region;
    note_mirror_range(mirror, mapped);
    g_stats.live_allocations += 1;
    g_stats.mirror_bytes += mapped;
    return mirror;
}

void coherent_release(void *context, void *memory) {
    (void)context;
    if (g_released && memory) {
        // While the region still exists: work that was recorded against it
        // but not launched yet has to go out (or be dropped) first.
        g_released(memory);
    }
    auto &regions = registry();
    auto it = regions.find(reinterpret_cast<uintptr_t>(memory));
    if (it == regions.end()) {
        return;
    }
    if (it->second.lazy) {
        drop_lazy(it->second.lazy);
    }
    if (it->second.feeds) {
        // The pending reader inherits the buffer.
        detach_source(it->second);
    }
    Region region = it->second;
    regions.erase(it);
    wait_for_upload(region);
    if (region.uploaded) {
        cudaEventDestroy(region.uploaded);
    }
    if (region.fetched) {
        cudaEventSynchronize(region.fetched);
        cudaEventDestroy(region.fetched);
    }
    if (region.staging) {
        cudaFreeHost(region.staging);
    }
    if (region.spare) {
        // Its last readers are in the compute stream, which is also where a
        // pooled buffer's next user will be.
        recycle(region.spare, region.mapped);
        g_stats.device_bytes -= region.mapped;
        cudaEventDestroy(region.spare_free);
    }
    if (region.pinned) {
        cudaHostUnregister(region.mirror);
    }
    if (region.device) {
        recycle(region.device, region.mapped);
        g_stats.device_bytes -= region.mapped;
    }
    munmap(region.mirror, region.mapped);
    g_stats.live_allocations -= 1;
    g_stats.mirror_bytes -= region.mapped;
}

void coherent_external_range(const void *base, size_t bytes, bool add) {
    auto &ranges = external_ranges();
    const uintptr_t begin = reinterpret_cast<uintptr_t>(base);
    if (add) {
        ranges.push_back(ExternalRange{begin, begin + bytes});
        return;
    }
    for (size_t i = 0; i < ranges.size(); ++i) {
        if (ranges[i].begin == begin) {
            ranges.erase(ranges.begin() + long(i));
            return;
        }
    }
}

size_t coherent_device_bytes(const void *host_pointer) {
    const Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    return region ? region->mapped : 0;
}

bool coherent_place_device_buffer(const void *host_pointer, float *device,
                                  cudaStream_t stream) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    if (!region || region->lazy || region->feeds) {
        return false;
    }
    if (region->device == device && device) {
        return true;
    }
    float *old = region->device;
    if (!device) {
        if (!old || !is_external(old)) {
            return true;   // already in memory of its own (or nowhere yet)
        }
        region->device = nullptr;
        g_stats.device_bytes -= region->mapped;
        ensure_device_buffer(*region);
        device = region->device;
    } else {
        if (!old) {
            g_stats.device_bytes += region->mapped;
        }
        region->device = device;
    }
    if (old) {
        // Whatever the old buffer holds that is current moves along; a
        // pending zero fill or host-owned contents need no copy.
        if (region->owner != Owner::Host && !region->zero_pending) {
            check(cudaMemcpyAsync(device, old, region->bytes,
                                  cudaMemcpyDeviceToDevice, stream),
                  "cudaMemcpyAsync(device to device)");
        }
        recycle(old, region->mapped);
    }
    return true;
}

const float *coherent_current_device(const void *host_pointer,
                                     cudaStream_t stream) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    if (!region || region->owner != Owner::Device) {
        return nullptr;   // not ours, or the mirror holds the current values
    }
    if (region->lazy) {
        if (is_alias(*region)) {
            return source_device(region->lazy, 0);
        }
        materialise_lazy(region->lazy, stream);
    }
    ensure_device_buffer(*region);
    materialise_zero(*region, stream);
    return region->device;
}

bool coherent_owns(const void *host_pointer) {
    return host_pointer && find_base(host_pointer) != nullptr;
}

void ensure_copy_stream() {
    if (!g_copy_stream) {
        check(cudaStreamCreateWithFlags(&g_copy_stream, cudaStreamNonBlocking),
              "cudaStreamCreate");
        check(cudaEventCreateWithFlags(&g_produced, cudaEventDisableTiming),
              "cudaEventCreate");
    }
}

// The upload of a large, repeatedly rewritten input (the image batch) taken off
// the compute stream: with the host running ahead of the device, the copy then
// happens while the previous step's backward pass runs instead of between the
// optimiser and the next forward pass.  The input gets two device buffers used
// in turn.  The one written now held the batch before last; its readers were
// all enqueued before the previous upload, which left an event behind them on
// the compute stream (spare_free) that the copy waits for.  The compute stream
// waits for the copy, and leaves the same kind of event for the buffer that has
// just been retired.
void upload_beside_compute(Region &region, cudaStream_t stream) {
    ensure_copy_stream();
    if (!region.spare) {
        void *memory = nullptr;
        check(cudaMalloc(&memory, region.mapped), "cudaMalloc");
        region.spare = static_cast<float *>(memory);
        g_stats.device_bytes += region.mapped;
        check(cudaEventCreateWithFlags(&region.spare_free, cudaEventDisableTiming),
              "cudaEventCreate");
    } else {
        check(cudaStreamWaitEvent(g_copy_stream, region.spare_free, 0),
              "cudaStreamWaitEvent");
    }
    float *retired = region.device;
    region.device = region.spare;
    region.spare = retired;
    check(cudaMemcpyAsync(region.device, region.mirror, region.bytes,
                          cudaMemcpyHostToDevice, g_copy_stream),
          "cudaMemcpyAsync(host to device)");
    if (!region.uploaded) {
        check(cudaEventCreateWithFlags(&region.uploaded, cudaEventDisableTiming),
              "cudaEventCreate");
    }
    check(cudaEventRecord(region.uploaded, g_copy_stream), "cudaEventRecord");
    region.upload_in_flight = true;
    check(cudaStreamWaitEvent(stream, region.uploaded, 0), "cudaStreamWaitEvent");
    // Everything that reads the retired buffer is in the stream by now.
    check(cudaEventRecord(region.spare_free, stream), "cudaEventRecord");
}

float *device_view(const void *host_pointer, Access access,
                   cudaStream_t stream) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    if (!region) {
        return nullptr;
    }
    if (region->lazy) {
        if (access == Access::Read && is_alias(*region)) {
            // A reader of an alias is served from the source's buffer.
            g_stats.alias_reads += 1;
            return const_cast<float *>(source_device(region->lazy, 0));
        }
        if (access == Access::Overwrite) {
            drop_lazy(region->lazy);
        } else {
            materialise_lazy(region->lazy, stream);
        }
    }
    if (region->feeds && access != Access::Read) {
        if (access == Access::Overwrite && region->device) {
            detach_source(*region);
        } else if (region->device && region->owner != Owner::Host &&
                   copy_beats_readers(*region)) {
            // An in-place update of a small source with large definitions
            // pending on it (a weight matrix under the optimizer): the
            // readers keep the old buffer, the update runs on a copy.
            float *old = region->device;
            detach_source(*region);
            ensure_device_buffer(*region);
            check(cudaMemcpyAsync(region->device, old, region->bytes,
                                  cudaMemcpyDeviceToDevice, stream),
                  "cudaMemcpyAsync(device to device)");
            g_stats.sources_copied += 1;
        } else {
            materialise_readers(*region, stream);
        }
    }
    ensure_device_buffer(*region);
    if (region->zero_pending) {
        if (access == Access::Overwrite) {
            region->zero_pending = false;
            region->zeroed = nullptr;
            g_stats.zero_fills_elided += 1;
        } else {
            materialise_zero(*region, stream);
        }
    }
    if (region->owner == Owner::Host && access != Access::Overwrite) {
        // Launch everything recorded so far first: the upload must not
        // overtake kernels that were recorded against the old contents.
        if (g_flush) {
            g_flush();
        }
        // A mirror that is uploaded again and again (the image batch, the
        // labels) is page-locked once, so its copies become plain DMA instead
        // of going through the driver's staging buffer.
        if (++region->uploads == 2 && !region->pinned) {
            if (cudaHostRegister(region->mirror, region->mapped,
                                 cudaHostRegisterDefault) == cudaSuccess) {
                region->pinned = true;
            } else {
                cudaGetLastError();   // stay pageable; clear the error state
            }
        }
        if (g_overlap_uploads && region->pinned && access == Access::Read &&
            region->bytes >= kOverlapUploadBytes && !region->lazy &&
            !region->feeds && !region->zero_pending && !is_external(region->device)) {
            upload_beside_compute(*region, stream);
        } else {
            check(cudaMemcpyAsync(region->device, region->mirror, region->bytes,
                                  cudaMemcpyHostToDevice, stream),
                  "cudaMemcpyAsync(host to device)");
            if (region->pinned) {
                if (!region->uploaded) {
                    check(cudaEventCreateWithFlags(&region->uploaded,
                                                   cudaEventDisableTiming),
                          "cudaEventCreate");
                }
                check(cudaEventRecord(region->uploaded, stream), "cudaEventRecord");
                region->upload_in_flight = true;
            }
        }
        g_stats.host_to_device_copies += 1;
        g_stats.host_to_device_bytes += region->bytes;
    }
    if (access != Access::Read) {
        region->prefetched = false;
    }
    if (access == Access::Read) {
        if (region->owner == Owner::Host) {
            protect(*region, PROT_READ);
            region->owner = Owner::Shared;
        }
    } else if (region->owner != Owner::Device) {
        protect(*region, PROT_NONE);
        region->owner = Owner::Device;
        if (region->mapped >= kDropPagesThreshold && !region->pinned) {
            madvise(region->mirror, region->mapped, MADV_DONTNEED);
        }
    }
    return region->device;
}

bool coherent_mark_zero(const void *host_pointer, cudaStream_t stream) {
    (void)stream;
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    if (!region) {
        return false;
    }
    if (region->lazy) {
        drop_lazy(region->lazy);
    }
    if (region->feeds) {
        detach_source(*region);   // pending readers keep the old contents
    }
    // No device buffer is created here: a gradient that nobody writes in a
    // step (the probability matrix's, the images') never needs one.
    if (region->owner != Owner::Device) {
        protect(*region, PROT_NONE);
        region->owner = Owner::Device;
        if (region->mapped >= kDropPagesThreshold && !region->pinned) {
            madvise(region->mirror, region->mapped, MADV_DONTNEED);
        }
    }
    region->zero_pending = true;
    region->zeroed = nullptr;
    region->prefetched = false;
    return true;
}

bool coherent_prefetch_host(const void *host_pointer, cudaStream_t stream) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    if (!region || region->owner != Owner::Device || !region->device ||
        region->lazy || region->zero_pending || region->bytes == 0 ||
        region->bytes > kPrefetchLimitBytes) {
        return false;
    }
    ensure_copy_stream();
    if (!region->staging) {
        check(cudaMallocHost(&region->staging, region->bytes), "cudaMallocHost");
        check(cudaEventCreateWithFlags(&region->fetched, cudaEventDisableTiming),
              "cudaEventCreate");
    }
    check(cudaEventRecord(g_produced, stream), "cudaEventRecord");
    check(cudaStreamWaitEvent(g_copy_stream, g_produced, 0), "cudaStreamWaitEvent");
    check(cudaMemcpyAsync(region->staging, region->device, region->bytes,
                          cudaMemcpyDeviceToHost, g_copy_stream),
          "cudaMemcpyAsync(device to host)");
    check(cudaEventRecord(region->fetched, g_copy_stream), "cudaEventRecord");
    region->prefetched = true;
    return true;
}

void coherent_set_wait_poll(int (*poll)(void)) {
    g_wait_poll = poll;
}

void coherent_set_overlapped_uploads(bool on) {
    g_overlap_uploads = on;
}

size_t coherent_zero_fill_batch(const void *const *host_pointers, size_t count,
                                size_t max_bytes, cudaStream_t stream) {
    ZeroBatch batch;
    Region *members[kZeroBatch];
    int filled = 0;
    unsigned longest = 0;
    size_t cleared = 0;
    auto launch = [&]() {
        if (filled == 0) {
            return;
        }
        const dim3 grid((longest + kZeroFloatsPerBlock - 1) / kZeroFloatsPerBlock,
                        unsigned(filled));
        zero_batch_kernel<<<grid, 256, 0, stream>>>(batch);
        check(cudaGetLastError(), "zero_batch_kernel");
        for (int i = 0; i < filled; ++i) {
            members[i]->zeroed = members[i]->device;
        }
        cleared += size_t(filled);
        filled = 0;
        longest = 0;
    };
    for (size_t i = 0; i < count; ++i) {
        Region *region = host_pointers[i] ? find_base(host_pointers[i]) : nullptr;
        // Only a plain pending fill over a buffer that already exists: no
        // buffer is created for a gradient that nobody may write this step.
        if (!region || !region->zero_pending || region->lazy || region->feeds ||
            !region->device || region->zeroed == region->device ||
            region->bytes == 0 || region->bytes > max_bytes) {
            continue;
        }
        bool listed = false;   // the caller may name a buffer twice
        for (int j = 0; j < filled; ++j) {
            listed = listed || members[j] == region;
        }
        if (listed) {
            continue;
        }
        members[filled] = region;
        batch.buffer[filled] = region->device;
        batch.floats[filled] = unsigned(region->bytes / sizeof(float));
        longest = batch.floats[filled] > longest ? batch.floats[filled] : longest;
        if (++filled == kZeroBatch) {
            launch();
        }
    }
    launch();
    return cleared;
}

bool coherent_define_lazy(const void *output_host,
                          const void *const *source_hosts, int sources,
                          LazyMaterialise function, const void *arguments,
                          size_t argument_bytes, cudaStream_t stream) {
    Region *output = output_host ? find_base(output_host) : nullptr;
    if (!output || sources < 0 || sources > 2 ||
        argument_bytes > sizeof(LazyDefinition::arguments)) {
        return false;
    }
    Region *inputs[2] = {nullptr, nullptr};
    for (int i = 0; i < sources; ++i) {
        inputs[i] = find_base(source_hosts[i]);
        // A source must hold its current contents on the device.
        if (!inputs[i] || inputs[i] == output || inputs[i]->lazy ||
            !inputs[i]->device || inputs[i]->owner == Owner::Host ||
            inputs[i]->zero_pending || (i == 1 && inputs[1] == inputs[0])) {
            return false;
        }
    }
    if (output->lazy) {
        drop_lazy(output->lazy);
    }
    if (output->feeds) {
        if (output->device) {
            detach_source(*output);
        } else {
            materialise_readers(*output, stream);
        }
    }
    LazyDefinition *lazy = new LazyDefinition();
    lazy->function = function;
    memcpy(lazy->arguments, arguments, argument_bytes);
    lazy->output = output;
    lazy->sources = sources;
    for (int i = 0; i < sources; ++i) {
        lazy->source[i] = inputs[i];
        lazy->next_reader[i] = inputs[i]->feeds;
        inputs[i]->feeds = lazy;
    }
    output->lazy = lazy;
    output->zero_pending = false;
    output->zeroed = nullptr;
    if (output->owner != Owner::Device) {
        protect(*output, PROT_NONE);
        output->owner = Owner::Device;
        if (output->mapped >= kDropPagesThreshold && !output->pinned) {
            madvise(output->mirror, output->mapped, MADV_DONTNEED);
        }
    }
    g_stats.lazy_defined += 1;
    return true;
}

bool coherent_define_alias(const void *output_host, const void *source_host,
                           cudaStream_t stream) {
    Region *output = output_host ? find_base(output_host) : nullptr;
    Region *source = source_host ? find_base(source_host) : nullptr;
    if (!output || !source || output->bytes != source->bytes) {
        return false;
    }
    const size_t bytes = source->bytes;
    const void *sources[1] = {source_host};
    return coherent_define_lazy(output_host, sources, 1, materialise_copy,
                                &bytes, sizeof(bytes), stream);
}

float *device_view_accumulate_based(const void *host_pointer,
                                    cudaStream_t stream, const float **base) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    *base = nullptr;
    if (!region) {
        return nullptr;
    }
    if (is_alias(*region)) {
        // The sum replaces the alias: read the source, write our own buffer.
        // (If the source buffer is recycled into this very region the two
        // pointers coincide and the update is in place, element by element.)
        const float *source = source_device(region->lazy, 0);
        drop_lazy(region->lazy);
        float *own = device_view(host_pointer, Access::Overwrite, stream);
        *base = source;
        return own;
    }
    bool was_zero = false;
    float *own = device_view_accumulate(host_pointer, stream, &was_zero);
    *base = was_zero ? nullptr : own;
    return own;
}

bool coherent_is_lazy(const void *host_pointer) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    return region && region->lazy != nullptr;
}

bool coherent_lazy_source(const void *output_host, LazyMaterialise function,
                          void *arguments, size_t argument_bytes,
                          const float **source, const void **source_host) {
    Region *region = output_host ? find_base(output_host) : nullptr;
    if (!region || !region->lazy || region->lazy->function != function ||
        region->lazy->sources != 1 ||
        argument_bytes > sizeof(LazyDefinition::arguments)) {
        return false;
    }
    memcpy(arguments, region->lazy->arguments, argument_bytes);
    *source = source_device(region->lazy, 0);
    *source_host = region->lazy->source[0] ? region->lazy->source[0]->mirror
                                           : nullptr;
    return true;
}

const void *coherent_alias_root(const void *host_pointer) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    if (!region || !is_alias(*region)) {
        return host_pointer;
    }
    return region->lazy->source[0] ? region->lazy->source[0]->mirror : nullptr;
}

bool coherent_is_zero_pending(const void *host_pointer) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    return region && region->zero_pending && !region->lazy;
}

float *device_view_accumulate(const void *host_pointer, cudaStream_t stream,
                              bool *was_zero) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    *was_zero = false;
    if (!region) {
        return nullptr;
    }
    if (region->zero_pending) {
        // Same transition as a full overwrite.
        *was_zero = true;
        return device_view(host_pointer, Access::Overwrite, stream);
    }
    return device_view(host_pointer, Access::ReadWrite, stream);
}

int coherent_make_host_owned(const void *host_pointer) {
    Region *region = host_pointer ? find_base(host_pointer) : nullptr;
    if (!region) {
        return -1;
    }
    serve_host_access(*region, true);
    return 0;
}

int coherent_prepare_host_io(const void *pointer, size_t bytes,
                             bool host_writes) {
    const uintptr_t begin = reinterpret_cast<uintptr_t>(pointer);
    if (!pointer || bytes == 0 ||
        begin >= g_highest_mirror.load(std::memory_order_relaxed) ||
        begin + bytes <= g_lowest_mirror.load(std::memory_order_relaxed)) {
        return 0;
    }
    int touched = 0;
    for (uintptr_t address = begin; address < begin + bytes;) {
        Region *region = find_containing(address);
        if (!region) {
            // Not ours: step to the next mirror, if any starts inside the range.
            auto next = registry().upper_bound(address);
            if (next == registry().end() || next->first >= begin + bytes) {
                break;
            }
            address = next->first;
            continue;
        }
        serve_host_access(*region, host_writes);
        touched += 1;
        address = reinterpret_cast<uintptr_t>(region->mirror) + region->mapped;
    }
    return touched;
}

CoherenceStats coherence_stats() {
    return g_stats;
}

}  // namespace vitb200
