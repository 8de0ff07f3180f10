// The drop-in boundary: the five cuda_backend_* functions, the op table that
// ops.c dispatches through, and the argument checks in front of each kernel.
//
// Every slot follows the host's convention (reference src/ops.c:61-64): return
// 0 once the work is enqueued, non-zero to decline, in which case the host
// synchronises and runs its own loop.  A slot declines when a buffer was not
// allocated by this backend (tensors created before device execution was
// enabled live in plain calloc memory) or when a shape is outside what the
// kernels index; it never declines half-way through.
#include "../../include/vitb200.h"
#include "../../include/vitb200_host_abi.h"
#include "../../include/vitb200_augmentation.h"
#include "../../include/vitb200_dataset.h"

#include "augmentation.h"
#include "checkpoint.h"
#include "coherence.h"
#include "data_parallel.h"
#include "dataset.h"
#include "gemm.h"
#include "gemm_tc.h"
#include "kernels.h"

#include <cfloat>
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <unordered_map>
#include <vector>

// Host functions this backend calls into.  They live in the host program
// (reference src/ops.c:66, src/autodiff.c:11); weak references keep this
// library loadable on its own, and a dlsym lookup covers hosts that were
// loaded after it.
extern "C" {
void ops_set_device_backend(const vitb200_op_table *table)
    __attribute__((weak));
void tensor_set_allocator(vitb200_allocate_fn allocate,
                          vitb200_release_fn release, void *context)
    __attribute__((weak));
}

using namespace vitb200;

namespace {

struct Scratch {
    void *memory = nullptr;
    size_t bytes = 0;
};

struct OpStat {
    const char *name;
    unsigned long long calls;
    double ms;
    double bytes;   // algorithmic HBM bytes
    double flops;   // algorithmic floating-point operations
};

struct PendingOp {
    int stat;
    cudaEvent_t begin, end;
};

// A forward product whose launch is held back for one or two ops so that the
// bias add, and then a GELU or a residual add, that the host issues right
// after it (reference src/vit.c:493-535) can ride on its epilogue.
struct PendingGemm {
    bool active = false;
    const float *x = nullptr, *w = nullptr;
    float *y = nullptr;
    const void *y_host = nullptr;   // host address of the output values
    int m = 0, k = 0, n = 0;
    GemmEpilogue epilogue;
    double bytes = 0.0, flops = 0.0;
};

// A short-sequence attention forward pass held back for one op: if the host
// merges the heads next (reference src/vit.c:489-491) the kernel writes its
// result in the merged layout and the head-major tensor becomes a pending
// view of it.  Input pointers are resolved when the op is recorded.
struct PendingAttention {
    bool active = false;
    int kind = 0;            // see attention_kind()
    float *lse = nullptr;    // kind 3: where the rows' log-sum-exp goes
    const float *q = nullptr, *k = nullptr, *v = nullptr;
    HeadLayout in_layout;
    const void *output_host = nullptr;
    size_t batch = 0, heads = 0, seq = 0, head_dim = 0;
    float scale = 0.0f;
    double bytes = 0.0, flops = 0.0;
};

// The matching backward pass, held back in case the host scatters the three
// gradients into the projected gradient next (reference src/vit.c:618-626).
struct PendingAttentionBackward {
    bool active = false;
    int kind = 0;
    const float *lse = nullptr;   // kind 3
    const float *q = nullptr, *k = nullptr, *v = nullptr, *out = nullptr,
                *dout = nullptr;
    HeadLayout in_layout, out_layout, dout_layout;
    const void *dq_host = nullptr, *dk_host = nullptr, *dv_host = nullptr;
    size_t batch = 0, heads = 0, seq = 0, head_dim = 0;
    float scale = 0.0f;
    double bytes = 0.0, flops = 0.0;
};

// Column sums of a gradient matrix that its producer computed on the way,
// kept for the bias_add_backward the host issues next on the same values
// (possibly through aliases of them).  Valid only while no other op has
// launched anything and nothing has been uploaded since.
struct ColumnSumMemo {
    bool valid = false;
    const float *data = nullptr;
    size_t rows = 0, cols = 0;
    unsigned long long epoch = 0;
    size_t uploads = 0;
    // Where the sums are: one row of `cols` floats in the zero-kept scratch
    // (partial_rows == 0), or that many rows of partial sums.
    const float *partials = nullptr;
    size_t partial_rows = 0;
};

// Device memory that column sums are gathered in: `clean` = known to be all
// zero.  The buffers circulate between the two current ones of the backend
// (the running sums a producer adds into, the per-CTA partial rows), the
// bias-gradient reductions that wait for their batched launch, and a free list.
struct SumBuffer {
    float *memory = nullptr;
    size_t floats = 0;
    bool clean = false;
};

// A bias gradient whose column sums exist (as one running row, or as a few
// hundred partial rows) and which only has to be folded into the gradient
// buffer: held back so that up to kColumnSumBatch of them share a launch.
struct PendingColumnSum {
    SumBuffer source;
    bool running = false;   // one running row (cleared by the launch), not partial rows
    size_t rows = 0, cols = 0;
    float *destination = nullptr;
    bool add = false;
    const void *host_gradient = nullptr;
    size_t count = 0;
};

// A residual add held back for one op: the layer norm that the host applies
// to the sum next (reference src/vit.c:520-523, and the next block's first
// layer norm after :534) computes the sum itself.
struct PendingResidual {
    bool active = false;
    const float *a = nullptr, *b = nullptr;
    float *sum = nullptr;
    const void *sum_host = nullptr;
    size_t count = 0;
};

// The input half of a product's backward pass, dX = dY W^T, held back while
// dX is still a pending zero fill: when the next op is the GELU backward pass
// that consumes dX (reference src/vit.c:552-554), the two run as one kernel
// and dX itself is never stored.
struct PendingInputGradient {
    bool active = false;
    const void *dx_host = nullptr, *w_host = nullptr, *dy_host = nullptr;
    int m = 0, k = 0, n = 0;
};

// Arguments of a gradient that was skipped that way, should somebody read it.
struct InputGradientShape {
    int m, k, n;
};

constexpr int kStagingSlots = 8;
constexpr size_t kStagingBytes = 64 * 1024;

}  // namespace

struct CudaBackend {
    int device = 0;
    cudaStream_t stream = nullptr;
    vitb200_op_table table = {};
    int enabled = 0;
    Scratch rows_scratch;      // per-row floats: CE row losses, attention dots
    Scratch norm_partials;
    Scratch clip_scale;
    Scratch slice_table;
    // Pinned ring for small host-to-device tables (the optimiser's slices).
    char *staging[kStagingSlots] = {};
    cudaEvent_t staging_done[kStagingSlots] = {};
    int staging_next = 0;
    cudaEvent_t timer_begin = nullptr, timer_end = nullptr;
    // Device-busy accounting: a span opens at the first kernel after a
    // synchronise and closes at the next synchronise.
    cudaEvent_t span_begin = nullptr, span_end = nullptr;
    bool span_open = false;
    double busy_ms = 0.0;
    // Optional per-op timing (vitb200_profile_enable).
    bool profiling = false;
    bool deferred_synchronize = false;   // see vitb200_set_deferred_synchronize
    std::vector<OpStat> op_stats;
    std::vector<PendingOp> pending_ops;
    std::vector<cudaEvent_t> free_events;
    DataParallel *dp = nullptr;
    // 1 / (micro-batches whose gradients one optimiser step consumes).
    float accumulation_inverse = 1.0f;
    // Ops that launched work so far (see ColumnSumMemo).
    unsigned long long epoch = 0;
    ColumnSumMemo column_memo;
    SumBuffer running_sums;    // what a producer adds its column sums into
    SumBuffer partial_sums;    // per-CTA / per-sample partial rows
    std::vector<SumBuffer> free_running, free_partial;
    std::vector<PendingColumnSum> pending_sums;
    // Batch augmentation: device staging for plain host buffers, the
    // per-sample table (pinned host copy + device copy) and the plane means.
    Scratch augment_source, augment_destination, augment_table, augment_means;
    void *augment_host_table = nullptr;
    size_t augment_host_bytes = 0;
    cudaEvent_t augment_table_read = nullptr;
    unsigned long long memo_hits = 0;
    PendingGemm pending;
    PendingAttention pending_attention;
    PendingAttentionBackward pending_attention_backward;
    PendingResidual pending_residual;
    PendingInputGradient pending_input_gradient;
    unsigned long long fused_residuals = 0;
    unsigned long long fused_head_layouts = 0;
    // Row log-sum-exp of flash attention, one buffer per probability tensor
    // (keyed by the tensor's host address), kept from forward to backward.
    std::unordered_map<const void *, Scratch> lse_buffers;
    std::unordered_map<const void *, bool> lse_streamed;
    unsigned long long fused_epilogues = 0;
    // Op slots that returned non-zero (the host then runs its CPU loop), and
    // which attention family served the long sequences.
    unsigned long long declined_ops = 0;
    unsigned long long tc_attention_launches = 0;
    unsigned long long streaming_attention_launches = 0;
    void (*set_table)(const vitb200_op_table *) = nullptr;
    void (*set_allocator)(vitb200_allocate_fn, vitb200_release_fn,
                          void *) = nullptr;
};

namespace {

[[noreturn]] void die(const char *what, cudaError_t status) {
    fprintf(stderr, "vitb200: %s failed: %s\n", what,
            cudaGetErrorString(status));
    abort();
}

void check(cudaError_t status, const char *what) {
    if (status != cudaSuccess) {
        die(what, status);
    }
}

void check_launch(const char *what) {
    check(cudaGetLastError(), what);
}

cudaEvent_t take_event(CudaBackend *backend) {
    if (!backend->free_events.empty()) {
        cudaEvent_t event = backend->free_events.back();
        backend->free_events.pop_back();
        return event;
    }
    cudaEvent_t event = nullptr;
    check(cudaEventCreate(&event), "cudaEventCreate");
    return event;
}

int stat_index(CudaBackend *backend, const char *name) {
    for (size_t i = 0; i < backend->op_stats.size(); ++i) {
        if (backend->op_stats[i].name == name) {  // string literals: same pointer
            return int(i);
        }
    }
    backend->op_stats.push_back(OpStat{name, 0, 0.0, 0.0, 0.0});
    return int(backend->op_stats.size() - 1);
}

// Brackets the launches of one op: opens the device-busy span, and when
// profiling is on, times the op with a pair of events on the backend stream.
// `bytes` and `flops` are the op's algorithmic traffic and arithmetic.
class OpScope {
public:
    OpScope(CudaBackend *backend, const char *name, double bytes, double flops)
        : backend_(backend), name_(name) {
        backend->epoch += 1;
        if (!backend->span_open) {
            check(cudaEventRecord(backend->span_begin, backend->stream),
                  "cudaEventRecord");
            backend->span_open = true;
        }
        if (backend->profiling) {
            pending_.stat = stat_index(backend, name);
            OpStat &stat = backend->op_stats[pending_.stat];
            stat.calls += 1;
            stat.bytes += bytes;
            stat.flops += flops;
            pending_.begin = take_event(backend);
            pending_.end = take_event(backend);
            check(cudaEventRecord(pending_.begin, backend->stream),
                  "cudaEventRecord");
        }
    }
    ~OpScope() {
        check_launch(name_);
        if (backend_->profiling) {
            check(cudaEventRecord(pending_.end, backend_->stream),
                  "cudaEventRecord");
            backend_->pending_ops.push_back(pending_);
        }
    }
private:
    CudaBackend *backend_;
    const char *name_;
    PendingOp pending_ = {};
};

void flush_attention(CudaBackend *backend);

void flush_input_gradient(CudaBackend *backend);
void flush_column_sums(CudaBackend *backend);

// Launches the held-back product, with whatever was attached to it.
// keep_column_sums: the caller is an op of the backward pass that neither
// reads nor writes a bias gradient, so bias-gradient reductions that are
// waiting for their batched launch may go on waiting.
void flush_pending(CudaBackend *backend, bool keep_column_sums = false) {
    if (!keep_column_sums) {
        flush_column_sums(backend);
    }
    // Every op starts here: whatever it does may change the matrix a memo
    // describes.  The few ops that provably do not put the memo back.
    backend->column_memo.valid = false;
    if (backend->pending_attention.active ||
        backend->pending_attention_backward.active) {
        flush_attention(backend);
    }
    if (backend->pending_residual.active) {
        const PendingResidual held = backend->pending_residual;
        backend->pending_residual.active = false;
        OpScope scope(backend, "residual", 12.0 * double(held.count), 0.0);
        launch_add(held.a, held.b, held.sum, held.count, backend->stream);
    }
    if (backend->pending_input_gradient.active) {
        flush_input_gradient(backend);
    }
    PendingGemm &pending = backend->pending;
    if (!pending.active) {
        return;
    }
    pending.active = false;
    OpScope scope(backend, "gemm", pending.bytes, pending.flops);
    gemm_forward_fused(pending.x, pending.w, pending.y, pending.m, pending.k,
                       pending.n, pending.epilogue, VITB200_PRECISION_AUTO,
                       backend->stream);
}

CudaBackend *g_flush_backend = nullptr;

// Hook for the coherence layer: called before an upload is enqueued and
// before a host access to device-owned memory is served.
void flush_hook() {
    if (g_flush_backend) {
        flush_pending(g_flush_backend);
    }
}

void settle_timers(CudaBackend *backend) {
    flush_pending(backend);
    if (backend->span_open) {
        check(cudaEventRecord(backend->span_end, backend->stream),
              "cudaEventRecord");
    }
    if (backend->dp && dp_world(backend->dp) > 1) {
        // With an exchange in flight the wait also watches the communicator:
        // a failed peer shows up as an asynchronous NCCL error, and aborting
        // the communicator then lets this stream drain.
        unsigned spins = 0;
        while (cudaStreamQuery(backend->stream) == cudaErrorNotReady) {
            if ((++spins & 1023u) == 0 && dp_poll(backend->dp) != 0) {
                break;
            }
        }
        cudaGetLastError();
    }
    check(cudaStreamSynchronize(backend->stream), "cudaStreamSynchronize");
    if (const int code = gemm_tc_status()) {
        fprintf(stderr,
                "vitb200: a tensor-core kernel gave up waiting (code %d)\n",
                code);
        abort();
    }
    if (backend->span_open) {
        float ms = 0.0f;
        check(cudaEventElapsedTime(&ms, backend->span_begin, backend->span_end),
              "cudaEventElapsedTime");
        backend->busy_ms += ms;
        backend->span_open = false;
    }
    for (const PendingOp &op : backend->pending_ops) {
        float ms = 0.0f;
        check(cudaEventElapsedTime(&ms, op.begin, op.end),
              "cudaEventElapsedTime");
        backend->op_stats[op.stat].ms += ms;
        backend->free_events.push_back(op.begin);
        backend->free_events.push_back(op.end);
    }
    backend->pending_ops.clear();
}

template <typename T>
T *scratch(CudaBackend *backend, Scratch &buffer, size_t count) {
    const size_t bytes = (count ? count : 1) * sizeof(T);
    if (buffer.bytes < bytes) {
        if (buffer.memory) {
            check(cudaStreamSynchronize(backend->stream), "cudaStreamSynchronize");
            check(cudaFree(buffer.memory), "cudaFree");
        }
        const size_t grown = bytes + bytes / 2;
        check(cudaMalloc(&buffer.memory, grown), "cudaMalloc");
        buffer.bytes = grown;
    }
    return static_cast<T *>(buffer.memory);
}

void free_scratch(Scratch &buffer) {
    if (buffer.memory) {
        cudaFree(buffer.memory);
    }
    buffer = Scratch{};
}

// A tensor is about to go (its region still exists).  Ops that were recorded
// but held back keep raw pointers into tensors, so they are launched now,
// while every buffer they name is still there; then the log-sum-exp buffer
// kept for the tensor, if any, is forgotten (the host's evaluation entry
// points create and free a cache per call).
void release_hook(const void *host_pointer) {
    CudaBackend *backend = g_flush_backend;
    if (!backend) {
        return;
    }
    if (backend->pending.active || backend->pending_attention.active ||
        backend->pending_attention_backward.active ||
        backend->pending_residual.active ||
        backend->pending_input_gradient.active ||
        !backend->pending_sums.empty()) {
        flush_pending(backend);
    }
    dp_tensor_released(backend->dp, host_pointer);
    auto found = backend->lse_buffers.find(host_pointer);
    if (found != backend->lse_buffers.end()) {
        // The buffer may still be read by enqueued work.
        cudaStreamSynchronize(backend->stream);
        free_scratch(found->second);
        backend->lse_buffers.erase(found);
    }
    backend->lse_streamed.erase(host_pointer);
}

size_t numel(const vitb200_tensor *tensor) {
    size_t count = 1;
    for (size_t i = 0; i < tensor->ndim; ++i) {
        count *= tensor->shape[i];
    }
    return tensor->ndim ? count : 0;
}

bool ours(std::initializer_list<const void *> pointers) {
    for (const void *pointer : pointers) {
        if (!coherent_owns(pointer)) {
            return false;
        }
    }
    return true;
}

bool fits_int(size_t value) {
    return value > 0 && value <= size_t(INT_MAX);
}

CudaBackend *self(void *context) {
    return static_cast<CudaBackend *>(context);
}

float *view(CudaBackend *backend, const void *pointer, Access access) {
    return device_view(pointer, access, backend->stream);
}

// View of a buffer about to be added into; *add comes back false when the
// buffer is a pending zero fill, in which case the kernel must store.
float *accumulate_view(CudaBackend *backend, const void *pointer, bool *add) {
    bool was_zero = false;
    float *device = device_view_accumulate(pointer, backend->stream, &was_zero);
    *add = !was_zero;
    return device;
}

// dX = dY W^T on its own: the op after the product's backward pass was not
// the GELU backward pass the product was held back for.
void flush_input_gradient(CudaBackend *backend) {
    const PendingInputGradient held = backend->pending_input_gradient;
    backend->pending_input_gradient.active = false;
    const float *w = view(backend, held.w_host, Access::Read);
    const float *dy = view(backend, held.dy_host, Access::Read);
    bool add = true;
    float *dx = accumulate_view(backend, held.dx_host, &add);
    OpScope scope(backend, "gemm_backward",
                  4.0 * (double(held.m) * held.n + double(held.k) * held.n +
                         (add ? 2.0 : 1.0) * double(held.m) * held.k),
                  2.0 * double(held.m) * held.k * held.n);
    gemm_backward_input(w, dy, dx, held.m, held.k, held.n,
                        VITB200_PRECISION_AUTO, add, backend->stream);
}


// Long sequences: the tcgen05 kernels where they apply (head_dim 32 or 64, at
// least a tile's worth of rows; VITB200_ATTENTION=stream switches them off),
// otherwise the register-resident streaming kernels.  Both keep the same
// log-sum-exp rows.
bool tc_attention_wanted(size_t seq, size_t head_dim) {
    static const bool disabled = []() {
        const char *choice = getenv("VITB200_ATTENTION");
        return choice && strcmp(choice, "stream") == 0;
    }();
    return !disabled && seq >= 96 && attention_tc_supported(seq, head_dim);
}

bool long_attention_forward(CudaBackend *backend, const float *q, const float *k,
                            const float *v, float *out, float *lse, size_t groups,
                            size_t seq, size_t head_dim, float scale,
                            HeadLayout in_layout = HeadLayout(),
                            HeadLayout out_layout = HeadLayout()) {
    if (tc_attention_wanted(seq, head_dim) &&
        launch_attention_tc_forward(q, k, v, out, lse, groups, seq, head_dim, scale,
                                    backend->stream, in_layout, out_layout)) {
        backend->tc_attention_launches += 1;
        return true;
    }
    if (launch_attention_stream_forward(q, k, v, out, lse, groups, seq, head_dim,
                                        scale, backend->stream, in_layout,
                                        out_layout)) {
        backend->streaming_attention_launches += 1;
        return true;
    }
    return false;
}

bool long_attention_backward(CudaBackend *backend, const float *q, const float *k,
                             const float *v, const float *out, const float *dout,
                             const float *lse, float *dq, float *dk, float *dv,
                             float *row_dots, size_t groups, size_t seq,
                             size_t head_dim, float scale, bool add_q, bool add_k,
                             bool add_v, HeadLayout in_layout = HeadLayout(),
                             HeadLayout out_layout = HeadLayout(),
                             HeadLayout dout_layout = HeadLayout(),
                             HeadLayout grad_layout = HeadLayout(),
                             float *column_partials = nullptr,
                             bool *partials_written = nullptr) {
    if (partials_written) {
        *partials_written = false;
    }
    if (tc_attention_wanted(seq, head_dim) &&
        launch_attention_tc_backward(q, k, v, out, dout, lse, dq, dk, dv, row_dots,
                                     groups, seq, head_dim, scale, add_q, add_k,
                                     add_v, backend->stream, in_layout, out_layout,
                                     dout_layout, grad_layout, column_partials)) {
        backend->tc_attention_launches += 1;
        if (partials_written) {
            *partials_written = column_partials != nullptr;
        }
        return true;
    }
    if (launch_attention_stream_backward(q, k, v, out, dout, lse, dq, dk, dv,
                                         row_dots, groups, seq, head_dim, scale,
                                         add_q, add_k, add_v, backend->stream,
                                         in_layout, out_layout, dout_layout,
                                         grad_layout)) {
        backend->streaming_attention_launches += 1;
        return true;
    }
    return false;
}

void run_attention(CudaBackend *backend, const PendingAttention &pending,
                   float *out, HeadLayout out_layout) {
    OpScope scope(backend, "multi_head_attention", pending.bytes,
                  pending.flops);
    const size_t groups = pending.batch * pending.heads;
    if (pending.kind == 3) {
        long_attention_forward(backend, pending.q, pending.k, pending.v, out,
                               pending.lse, groups, pending.seq, pending.head_dim,
                               pending.scale, pending.in_layout, out_layout);
    } else if (pending.kind == 2) {
        launch_attention_warp_forward(pending.q, pending.k, pending.v, out,
                                      groups, pending.seq, pending.head_dim,
                                      pending.scale, backend->stream,
                                      pending.in_layout, out_layout);
    } else {
        launch_attention_small_forward(pending.q, pending.k, pending.v, nullptr,
                                       out, groups, pending.seq,
                                       pending.head_dim, pending.scale, false,
                                       true, backend->stream, pending.in_layout,
                                       out_layout);
    }
}

// Returns whether `column_partials` (when given) was filled.
bool run_attention_backward(CudaBackend *backend,
                            const PendingAttentionBackward &pending, float *dq,
                            float *dk, float *dv, bool add_q, bool add_k,
                            bool add_v, HeadLayout grad_layout,
                            float *column_partials = nullptr) {
    OpScope scope(backend, "multi_head_attention_backward", pending.bytes,
                  pending.flops);
    const size_t groups = pending.batch * pending.heads;
    bool partials_written = column_partials != nullptr;
    if (pending.kind == 3) {
        float *dots = scratch<float>(backend, backend->rows_scratch,
                                     groups * pending.seq);
        long_attention_backward(
            backend, pending.q, pending.k, pending.v, pending.out, pending.dout,
            pending.lse, dq, dk, dv, dots, groups, pending.seq,
            pending.head_dim, pending.scale, add_q, add_k, add_v,
            pending.in_layout, pending.out_layout, pending.dout_layout,
            grad_layout, column_partials, &partials_written);
    } else if (pending.kind == 2) {
        launch_attention_warp_backward(
            pending.q, pending.k, pending.v, pending.out, pending.dout, dq, dk,
            dv, groups, pending.seq, pending.head_dim, pending.scale, add_q,
            add_k, add_v, backend->stream, pending.in_layout,
            pending.out_layout, pending.dout_layout, grad_layout,
            column_partials);
    } else {
        launch_attention_small_backward(
            pending.q, pending.k, pending.v, nullptr, pending.out,
            pending.dout, dq, dk, dv, groups, pending.seq, pending.head_dim,
            pending.scale, add_q, add_k, add_v, true, backend->stream,
            pending.in_layout, pending.out_layout, pending.dout_layout,
            grad_layout);
        partials_written = false;
    }
    return partials_written;
}

// Held-back attention kernels, in their plain form: results go to the
// head-major tensors the host named.
void flush_attention(CudaBackend *backend) {
    if (backend->pending_attention.active) {
        const PendingAttention pending = backend->pending_attention;
        backend->pending_attention.active = false;
        float *o = view(backend, pending.output_host, Access::Overwrite);
        if (o) {
            run_attention(backend, pending, o, HeadLayout());
        }
    }
    if (backend->pending_attention_backward.active) {
        const PendingAttentionBackward pending =
            backend->pending_attention_backward;
        backend->pending_attention_backward.active = false;
        bool add_q = true, add_k = true, add_v = true;
        float *dq = accumulate_view(backend, pending.dq_host, &add_q);
        float *dk = accumulate_view(backend, pending.dk_host, &add_k);
        float *dv = accumulate_view(backend, pending.dv_host, &add_v);
        if (dq && dk && dv) {
            run_attention_backward(backend, pending, dq, dk, dv, add_q, add_k,
                                   add_v, HeadLayout());
        }
    }
}

// A buffer of at least `floats` floats from a free list, or a new one.
SumBuffer acquire_sum_buffer(CudaBackend *backend, std::vector<SumBuffer> &list,
                             size_t floats, bool zeroed) {
    SumBuffer buffer;
    for (size_t i = 0; i < list.size(); ++i) {
        if (list[i].floats >= floats) {
            buffer = list[i];
            list.erase(list.begin() + long(i));
            break;
        }
    }
    if (!buffer.memory) {
        const size_t grown = floats + floats / 2;
        void *memory = nullptr;
        check(cudaMalloc(&memory, grown * sizeof(float)), "cudaMalloc");
        buffer.memory = static_cast<float *>(memory);
        buffer.floats = grown;
        buffer.clean = false;
    }
    if (zeroed && !buffer.clean) {
        check(cudaMemsetAsync(buffer.memory, 0, buffer.floats * sizeof(float),
                              backend->stream),
              "cudaMemsetAsync");
        buffer.clean = true;
    }
    return buffer;
}

void retire_sum_buffer(std::vector<SumBuffer> &list, SumBuffer buffer) {
    if (buffer.memory) {
        list.push_back(buffer);
    }
}

// The current partial-rows buffer, at least `floats` long (contents
// undefined: its users overwrite or clear what they need).
float *partial_sums_buffer(CudaBackend *backend, size_t floats) {
    if (backend->partial_sums.floats < floats) {
        retire_sum_buffer(backend->free_partial, backend->partial_sums);
        backend->partial_sums =
            acquire_sum_buffer(backend, backend->free_partial, floats, false);
    }
    return backend->partial_sums.memory;
}

// A zeroed buffer of `cols` floats for a producer to add column sums into, or
// nullptr if the width is not worth it.
float *column_memo_begin(CudaBackend *backend, size_t cols) {
    backend->column_memo.valid = false;
    if (cols == 0 || cols > 16384) {
        return nullptr;
    }
    SumBuffer &running = backend->running_sums;
    if (running.floats < cols) {
        retire_sum_buffer(backend->free_running, running);
        running = acquire_sum_buffer(backend, backend->free_running, cols, true);
    } else if (!running.clean) {
        check(cudaMemsetAsync(running.memory, 0, running.floats * sizeof(float),
                              backend->stream),
              "cudaMemsetAsync");
    }
    running.clean = false;   // the producer is about to add into it
    return running.memory;
}

// Call after the producer's OpScope has closed.
void column_memo_commit(CudaBackend *backend, const float *data, size_t rows,
                        size_t cols, const float *partials = nullptr,
                        size_t partial_rows = 0) {
    ColumnSumMemo &memo = backend->column_memo;
    memo.partials = partials;
    memo.partial_rows = partial_rows;
    memo.valid = true;
    memo.data = data;
    memo.rows = rows;
    memo.cols = cols;
    memo.epoch = backend->epoch;
    memo.uploads = coherence_stats().host_to_device_copies;
}

bool column_memo_matches(CudaBackend *backend, const float *data, size_t rows,
                         size_t cols) {
    const ColumnSumMemo &memo = backend->column_memo;
    return memo.valid && memo.data == data && memo.rows == rows &&
           memo.cols == cols && memo.epoch == backend->epoch &&
           memo.uploads == coherence_stats().host_to_device_copies;
}

// Partial rows up to this many are folded by the batched launch (one block
// per 128 columns walks all of them); taller ones keep their own launch.
constexpr size_t kDeferredSumRows = 512;

// One launch for all the bias gradients that are waiting to be folded out of
// their column sums, then what each of them owes the gradient exchange.
void flush_column_sums(CudaBackend *backend) {
    if (backend->pending_sums.empty()) {
        return;
    }
    std::vector<PendingColumnSum> waiting;
    waiting.swap(backend->pending_sums);
    for (size_t first = 0; first < waiting.size(); first += kColumnSumBatch) {
        const size_t count = std::min(waiting.size() - first, size_t(kColumnSumBatch));
        ColumnSumJob jobs[kColumnSumBatch];
        double bytes = 0.0;
        for (size_t i = 0; i < count; ++i) {
            const PendingColumnSum &item = waiting[first + i];
            jobs[i].source = item.source.memory;
            jobs[i].destination = item.destination;
            jobs[i].rows = unsigned(item.rows);
            jobs[i].cols = unsigned(item.cols);
            jobs[i].add = item.add ? 1 : 0;
            jobs[i].clear = item.running ? 1 : 0;
            bytes += 4.0 * double(item.rows + 1) * double(item.cols);
        }
        OpScope scope(backend, "bias_add_backward", bytes, 0.0);
        launch_column_sums_batch(jobs, int(count), backend->stream);
    }
    for (const PendingColumnSum &item : waiting) {
        dp_gradient_produced(backend->dp, item.host_gradient, item.destination,
                             item.count);
        SumBuffer buffer = item.source;
        buffer.clean = item.running;   // the launch cleared a running row
        retire_sum_buffer(item.running ? backend->free_running : backend->free_partial,
                          buffer);
    }
}

// destination += source where destination is a pending zero fill: make it an
// alias of the source.  False when that is not the situation (or the source
// cannot be aliased), in which case nothing has changed.
bool alias_if_zero(CudaBackend *backend, const void *destination,
                   const void *source) {
    return coherent_is_zero_pending(destination) &&
           coherent_define_alias(destination, source, backend->stream);
}

// ---------------------------------------------------------------- op slots

int op_gemm(void *context, const vitb200_tensor *left,
            const vitb200_tensor *right, vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({left->data, right->data, output->data}) ||
        !fits_int(left->rows) || !fits_int(left->cols) ||
        !fits_int(right->cols)) {
        return -1;
    }
    const float *x = view(backend, left->data, Access::Read);
    const float *w = view(backend, right->data, Access::Read);
    float *y = view(backend, output->data, Access::Overwrite);
    // Not launched yet: the next op or two may join its epilogue.  The output
    // is already device-owned, so a host access to it faults and flushes.
    PendingGemm &pending = backend->pending;
    pending = PendingGemm();
    pending.active = true;
    pending.x = x;
    pending.w = w;
    pending.y = y;
    pending.y_host = output->data;
    pending.m = int(left->rows);
    pending.k = int(left->cols);
    pending.n = int(right->cols);
    pending.bytes = 4.0 * (double(left->rows) * left->cols +
                           double(right->rows) * right->cols +
                           double(output->rows) * output->cols);
    pending.flops = 2.0 * double(left->rows) * left->cols * right->cols;
    return 0;
}

int op_gemm_backward(void *context, vitb200_tensor *left, vitb200_tensor *right,
                     const vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    flush_pending(backend, true);
    if (!ours({left->data, left->grad, right->data, right->grad,
               output->grad}) ||
        !fits_int(left->rows) || !fits_int(left->cols) ||
        !fits_int(right->cols)) {
        return -1;
    }
    const float *x = view(backend, left->data, Access::Read);
    const float *w = view(backend, right->data, Access::Read);
    const float *dy = view(backend, output->grad, Access::Read);
    float *dw = view(backend, right->grad, Access::ReadWrite);
    const int m = int(left->rows), k = int(left->cols), n = int(right->cols);
    const double weight_bytes = 4.0 * (double(m) * k + double(m) * n +
                                       2.0 * double(k) * n);
    const double half_flops = 2.0 * double(m) * k * n;
    // The input gradient waits for one op when it would be the first thing
    // written into a zeroed buffer by a tensor-core product: a GELU backward
    // pass that follows takes it over (see op_gelu_backward).
    static const bool hold_back = getenv("VITB200_NO_GELU_BACKWARD_FUSION") == nullptr;
    if (hold_back && coherent_is_zero_pending(left->grad) &&
        prefer_tensor_cores(VITB200_PRECISION_AUTO, double(m) * k * n) &&
        k % 4 == 0 && n % 4 == 0) {
        {
            OpScope scope(backend, "gemm_backward", weight_bytes, half_flops);
            gemm_backward_weights(x, dy, dw, m, k, n, VITB200_PRECISION_AUTO,
                                  backend->stream);
        }
        PendingInputGradient &held = backend->pending_input_gradient;
        held.active = true;
        held.dx_host = left->grad;
        held.w_host = right->data;
        held.dy_host = output->grad;
        held.m = m;
        held.k = k;
        held.n = n;
        dp_gradient_produced(backend->dp, right->grad, dw, numel(right));
        return 0;
    }
    bool dx_add = true;
    float *dx = accumulate_view(backend, left->grad, &dx_add);
    // One scope per launch, here and where the input half is held back.
    {
        OpScope scope(backend, "gemm_backward",
                      4.0 * (double(m) * n + double(k) * n +
                             (dx_add ? 2.0 : 1.0) * double(m) * k),
                      half_flops);
        gemm_backward_input(w, dy, dx, m, k, n, VITB200_PRECISION_AUTO, dx_add,
                            backend->stream);
    }
    {
        OpScope scope(backend, "gemm_backward", weight_bytes, half_flops);
        gemm_backward_weights(x, dy, dw, m, k, n, VITB200_PRECISION_AUTO,
                              backend->stream);
    }
    dp_gradient_produced(backend->dp, right->grad, dw, numel(right));
    return 0;
}

int op_residual(void *context, const vitb200_tensor *left,
                const vitb200_tensor *right, vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    if (!ours({left->data, right->data, output->data})) {
        flush_pending(backend);
        return -1;
    }
    PendingGemm &pending = backend->pending;
    const bool left_is_product = left->data == pending.y_host;
    const bool right_is_product = right->data == pending.y_host;
    // Folding the residual add into the epilogue is implemented in the kernel
    // but not used: four epilogue warps cannot keep enough residual loads in
    // flight, and the fused launch measured slower (0.134 ms) than product +
    // streaming add (0.027 + 0.03 ms) at [102400,128]x[128,128].
    constexpr bool kFuseResidual = false;
    if (kFuseResidual && pending.active && left_is_product != right_is_product &&
        !pending.epilogue.gelu_out && !pending.epilogue.residual_out &&
        output->data != pending.y_host &&
        numel(output) == size_t(pending.m) * pending.n) {
        const vitb200_tensor *other = left_is_product ? right : left;
        const float *residual = view(backend, other->data, Access::Read);
        float *sum = view(backend, output->data, Access::Overwrite);
        if (pending.active) {   // an upload above may have flushed it
            pending.epilogue.residual = residual;
            pending.epilogue.residual_out = sum;
            pending.bytes += 8.0 * double(numel(output));
            backend->fused_epilogues += 1;
            flush_pending(backend);
            return 0;
        }
    }
    flush_pending(backend);
    const float *a = view(backend, left->data, Access::Read);
    const float *b = view(backend, right->data, Access::Read);
    float *out = view(backend, output->data, Access::Overwrite);
    // Not launched yet: a layer norm of the sum usually follows and adds the
    // two itself.  (The output is device-owned, so a host access flushes.)
    PendingResidual &held = backend->pending_residual;
    held.active = true;
    held.a = a;
    held.b = b;
    held.sum = out;
    held.sum_host = output->data;
    held.count = numel(output);
    return 0;
}

int op_residual_backward(void *context, vitb200_tensor *left,
                         vitb200_tensor *right, const vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    const ColumnSumMemo memo = backend->column_memo;
    flush_pending(backend, true);
    // One pass updates both branches, which needs them to be distinct.
    if (!ours({left->grad, right->grad, output->grad}) ||
        left->grad == right->grad) {
        return -1;
    }
    // Never parameter gradients in this model; a gradient exchange is told if
    // they ever are (it counts writers to know when a gradient is complete).
    dp_gradient_touched(backend->dp, left->grad);
    dp_gradient_touched(backend->dp, right->grad);
    bool add_a = true, add_b = true;
    const float *g = view(backend, output->grad, Access::Read);
    // A branch gradient that is still a pending zero fill simply becomes the
    // output gradient: declare it an alias instead of copying.
    const bool alias_a = alias_if_zero(backend, left->grad, output->grad);
    const bool alias_b = alias_if_zero(backend, right->grad, output->grad);
    if (alias_a && alias_b) {
        backend->column_memo = memo;   // nothing was written
        return 0;
    }
    if (alias_a || alias_b) {
        bool add = true;
        float *rest = accumulate_view(backend, alias_a ? right->grad : left->grad,
                                      &add);
        OpScope scope(backend, "residual_backward", 12.0 * double(numel(output)),
                      0.0);
        launch_accumulate(rest, g, numel(output), add, backend->stream);
        return 0;
    }
    float *a = accumulate_view(backend, left->grad, &add_a);
    float *b = accumulate_view(backend, right->grad, &add_b);
    {
        OpScope scope(backend, "residual_backward", 20.0 * double(numel(output)),
                      0.0);
        launch_accumulate2(a, b, g, numel(output), add_a, add_b,
                           backend->stream);
    }
    return 0;
}

int op_accumulate_gradient(void *context, vitb200_tensor *destination,
                           const vitb200_tensor *source) {
    CudaBackend *backend = self(context);
    const ColumnSumMemo memo = backend->column_memo;
    flush_pending(backend, true);
    if (!ours({destination->grad, source->grad}) ||
        destination->grad == source->grad) {
        return -1;
    }
    dp_gradient_touched(backend->dp, destination->grad);
    bool add = true;
    const float *src = view(backend, source->grad, Access::Read);
    if (alias_if_zero(backend, destination->grad, source->grad)) {
        backend->column_memo = memo;   // nothing was written
        return 0;
    }
    float *dst = accumulate_view(backend, destination->grad, &add);
    {
        OpScope scope(backend, "accumulate_gradient", 12.0 * double(numel(destination)),
                      0.0);
        launch_accumulate(dst, src, numel(destination), add, backend->stream);
    }
    return 0;
}

int op_bias_add(void *context, const vitb200_tensor *input,
                const vitb200_tensor *bias, vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    if (!ours({input->data, bias->data, output->data})) {
        flush_pending(backend);
        return -1;
    }
    const float *b = view(backend, bias->data, Access::Read);
    PendingGemm &pending = backend->pending;
    if (pending.active && input->data == pending.y_host &&
        output->data == pending.y_host && !pending.epilogue.bias &&
        !pending.epilogue.gelu_out && !pending.epilogue.residual_out &&
        input->cols == size_t(pending.n) && input->rows == size_t(pending.m)) {
        pending.epilogue.bias = b;
        backend->fused_epilogues += 1;
        return 0;   // stays pending: a GELU or a residual add may follow
    }
    flush_pending(backend);
    const bool in_place = input->data == output->data;
    const float *in =
        view(backend, input->data, in_place ? Access::ReadWrite : Access::Read);
    float *out = in_place ? const_cast<float *>(in)
                          : view(backend, output->data, Access::Overwrite);
    {
        OpScope scope(backend, "bias_add", 8.0 * double(numel(input)),
                      0.0);
        launch_bias_add(in, b, out, input->rows, input->cols, backend->stream);
    }
    return 0;
}

int op_bias_add_backward(void *context, const vitb200_tensor *output,
                         vitb200_tensor *bias_grad) {
    CudaBackend *backend = self(context);
    const ColumnSumMemo memo = backend->column_memo;
    flush_pending(backend, true);
    backend->column_memo = memo;   // checked against the launch count below
    if (!ours({output->grad, bias_grad->grad})) {
        return -1;
    }
    const float *dy = view(backend, output->grad, Access::Read);
    if (column_memo_matches(backend, dy, output->rows, output->cols)) {
        // The kernel that produced these values summed their columns too.
        const ColumnSumMemo used = backend->column_memo;
        backend->column_memo.valid = false;
        backend->memo_hits += 1;
        const bool running = used.partial_rows == 0;
        SumBuffer &current = running ? backend->running_sums : backend->partial_sums;
        // Folding the sums into the gradient is held back so that several
        // biases share one launch (flush_column_sums).  An earlier reduction
        // into the same gradient goes first.
        for (const PendingColumnSum &waiting : backend->pending_sums) {
            if (waiting.host_gradient == bias_grad->grad) {
                flush_column_sums(backend);
                break;
            }
        }
        static const bool batched = getenv("VITB200_NO_BATCHED_BIAS_SUMS") == nullptr;
        if (batched && output->cols % 4 == 0 && used.partial_rows <= kDeferredSumRows &&
            current.memory && (running || used.partials == current.memory)) {
            PendingColumnSum job;
            job.running = running;
            job.source = current;
            current = SumBuffer{};   // the next producer takes another buffer
            job.rows = running ? 1 : used.partial_rows;
            job.cols = output->cols;
            job.add = true;
            job.destination = accumulate_view(backend, bias_grad->grad, &job.add);
            job.host_gradient = bias_grad->grad;
            job.count = numel(bias_grad);
            backend->pending_sums.push_back(job);
            if (backend->pending_sums.size() >= size_t(kColumnSumBatch)) {
                flush_column_sums(backend);
            }
            return 0;
        }
        float *db = nullptr;
        if (!running) {
            db = view(backend, bias_grad->grad, Access::ReadWrite);
            OpScope scope(backend, "bias_add_backward",
                          4.0 * double(used.partial_rows * output->cols), 0.0);
            launch_column_sums(used.partials, db, used.partial_rows,
                               output->cols, output->cols, backend->stream);
        } else {
            bool add = true;
            db = accumulate_view(backend, bias_grad->grad, &add);
            OpScope scope(backend, "bias_add_backward", 8.0 * double(output->cols),
                          0.0);
            launch_take_column_sums(db, current.memory, output->cols, add,
                                    backend->stream);
            current.clean = true;   // the kernel leaves zeros behind
        }
        dp_gradient_produced(backend->dp, bias_grad->grad, db, numel(bias_grad));
        return 0;
    }
    float *db = view(backend, bias_grad->grad, Access::ReadWrite);
    {
        OpScope scope(backend, "bias_add_backward", 4.0 * double(numel(output)),
                      0.0);
        launch_column_sums(dy, db, output->rows, output->cols, output->cols,
                           backend->stream);
    }
    dp_gradient_produced(backend->dp, bias_grad->grad, db, numel(bias_grad));
    return 0;
}

int op_layer_norm(void *context, const vitb200_tensor *input,
                  const vitb200_tensor *gamma, const vitb200_tensor *beta,
                  float epsilon, vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    // The residual add that produced the input may still be held back.
    PendingResidual held = backend->pending_residual;
    const bool fuse = held.active && held.sum_host == input->data &&
                      held.count == numel(input) &&
                      layer_norm_takes_addend(input->cols) &&
                      ours({input->data, gamma->data, beta->data, output->data}) &&
                      input->data != output->data;
    if (fuse) {
        backend->pending_residual.active = false;
    }
    flush_pending(backend);
    if (!ours({input->data, gamma->data, beta->data, output->data}) ||
        input->data == output->data) {
        return -1;
    }
    const float *g = view(backend, gamma->data, Access::Read);
    const float *b = view(backend, beta->data, Access::Read);
    float *y = view(backend, output->data, Access::Overwrite);
    if (fuse) {
        backend->fused_residuals += 1;
        // Two reads (the addends), two writes (their sum, the normalised
        // rows): what the fused pass has to move, not the 12 + 8 B/elt of the
        // two ops it stands for.
        OpScope scope(backend, "layer_norm", 16.0 * double(numel(input)), 0.0);
        launch_layer_norm(held.a, g, b, epsilon, y, input->rows, input->cols,
                          backend->stream, held.b, held.sum);
        return 0;
    }
    const float *x = view(backend, input->data, Access::Read);
    {
        OpScope scope(backend, "layer_norm", 8.0 * double(numel(input)),
                      0.0);
        launch_layer_norm(x, g, b, epsilon, y, input->rows, input->cols,
                          backend->stream);
    }
    return 0;
}

int op_layer_norm_backward(void *context, const vitb200_tensor *input,
                           const vitb200_tensor *gamma, float epsilon,
                           const vitb200_tensor *output,
                           vitb200_tensor *input_grad,
                           vitb200_tensor *gamma_grad,
                           vitb200_tensor *beta_grad) {
    CudaBackend *backend = self(context);
    flush_pending(backend, true);
    if (!ours({input->data, gamma->data, output->grad, input_grad->grad,
               gamma_grad->grad, beta_grad->grad}) ||
        output->grad == input_grad->grad) {
        return -1;
    }
    const float *x = view(backend, input->data, Access::Read);
    const float *g = view(backend, gamma->data, Access::Read);
    const float *dy = view(backend, output->grad, Access::Read);
    // dx = base + increment: base is dx itself, the source that dx is still
    // an alias of, or absent when dx is a pending zero fill.
    const float *base = nullptr;
    float *dx = device_view_accumulate_based(input_grad->grad, backend->stream,
                                             &base);
    float *dg = view(backend, gamma_grad->grad, Access::ReadWrite);
    float *db = view(backend, beta_grad->grad, Access::ReadWrite);
    // dx is what the two bias gradients of the preceding linear layers are
    // the column sums of (reference src/vit.c:548-551, 567-571).
    float *sums = column_memo_begin(backend, input->cols);
    {
        OpScope scope(backend, "layer_norm_backward", 16.0 * double(numel(input)),
                      0.0);
        launch_layer_norm_backward(x, g, epsilon, dy, dx, dg, db, input->rows,
                                   input->cols, base, sums, backend->stream);
    }
    if (sums) {
        column_memo_commit(backend, dx, input->rows, input->cols);
    }
    dp_gradient_produced(backend->dp, gamma_grad->grad, dg, numel(gamma_grad));
    dp_gradient_produced(backend->dp, beta_grad->grad, db, numel(beta_grad));
    return 0;
}

int op_gelu(void *context, const vitb200_tensor *input,
            vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    if (!ours({input->data, output->data}) || input->data == output->data) {
        flush_pending(backend);
        return -1;
    }
    PendingGemm &pending = backend->pending;
    if (pending.active && input->data == pending.y_host &&
        !pending.epilogue.gelu_out && !pending.epilogue.residual_out &&
        numel(input) == size_t(pending.m) * pending.n) {
        float *activated = view(backend, output->data, Access::Overwrite);
        if (pending.active) {
            pending.epilogue.gelu_out = activated;
            pending.bytes += 4.0 * double(numel(output));
            backend->fused_epilogues += 1;
            flush_pending(backend);
            return 0;
        }
    }
    flush_pending(backend);
    const float *in = view(backend, input->data, Access::Read);
    float *out = view(backend, output->data, Access::Overwrite);
    {
        OpScope scope(backend, "gelu", 8.0 * double(numel(input)),
                      0.0);
        launch_gelu(in, out, numel(input), backend->stream);
    }
    return 0;
}

// A gradient skipped by the fused product + GELU backward kernel, computed
// after all because somebody reads it: dX = dY W^T.
void materialise_input_gradient(const void *arguments, float *output,
                                float *const *sources, cudaStream_t stream) {
    InputGradientShape shape;
    memcpy(&shape, arguments, sizeof(shape));
    gemm_backward_input(sources[1], sources[0], output, shape.m, shape.k,
                        shape.n, VITB200_PRECISION_AUTO, false, stream);
}

// gelu_backward right after the gemm_backward that would have produced its
// incoming gradient: one kernel computes d(hidden) = (dY W^T) * gelu'(hidden)
// and the column sums the bias gradient needs; the gradient in between is
// declared (dY W^T, should anybody read it) but not stored.  Returns false,
// with the held-back product still pending, when the situation is another.
bool gelu_backward_through_product(CudaBackend *backend,
                                   const vitb200_tensor *input,
                                   const vitb200_tensor *output) {
    const PendingInputGradient held = backend->pending_input_gradient;
    if (!held.active || output->grad != held.dx_host ||
        input->rows != size_t(held.m) || input->cols != size_t(held.k) ||
        !coherent_is_zero_pending(input->grad) ||
        !coherent_is_zero_pending(held.dx_host)) {
        return false;
    }
    // The skipped gradient is defined in terms of dY and W, which must be
    // plain device-resident buffers (dY is usually an alias: use its source).
    const void *sources[2] = {coherent_alias_root(held.dy_host), held.w_host};
    if (!sources[0] || sources[0] == sources[1]) {
        return false;
    }
    const float *w = view(backend, held.w_host, Access::Read);
    const float *dy = view(backend, held.dy_host, Access::Read);
    const float *h = view(backend, input->data, Access::Read);
    if (!gemm_backward_input_gelu_supported(w, dy, h, nullptr, held.m, held.k,
                                            held.n, VITB200_PRECISION_AUTO)) {
        return false;
    }
    const InputGradientShape shape = {held.m, held.k, held.n};
    if (!coherent_define_lazy(held.dx_host, sources, 2,
                              materialise_input_gradient, &shape, sizeof(shape),
                              backend->stream)) {
        return false;
    }
    backend->pending_input_gradient.active = false;
    flush_pending(backend, true);
    bool add = true;
    float *dh = accumulate_view(backend, input->grad, &add);   // add == false
    float *sums = partial_sums_buffer(backend,
                                      size_t(kGemmPartialRows) * input->cols);
    {
        OpScope scope(backend, "gemm_backward",
                      4.0 * (double(held.m) * held.n + double(held.k) * held.n +
                             2.0 * double(held.m) * held.k),
                      2.0 * double(held.m) * held.k * held.n);
        if (gemm_backward_input_gelu(w, dy, h, dh, sums, held.m, held.k, held.n,
                                     VITB200_PRECISION_AUTO,
                                     backend->stream) != 0) {
            fprintf(stderr, "vitb200: fused product + GELU backward failed to launch\n");
            abort();
        }
    }
    backend->fused_epilogues += 1;
    column_memo_commit(backend, dh, input->rows, input->cols, sums,
                       kGemmPartialRows);
    return true;
}

int op_gelu_backward(void *context, const vitb200_tensor *input,
                     const vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    if (backend->pending_input_gradient.active &&
        ours({input->data, input->grad, output->grad}) &&
        gelu_backward_through_product(backend, input, output)) {
        return 0;
    }
    flush_pending(backend, true);
    if (!ours({input->data, input->grad, output->grad})) {
        return -1;
    }
    dp_gradient_touched(backend->dp, input->grad);
    const float *x = view(backend, input->data, Access::Read);
    const float *dy = view(backend, output->grad, Access::Read);
    bool add = true;
    float *dx = accumulate_view(backend, input->grad, &add);
    float *sums = nullptr;
    size_t partial_rows = 0;
    if (gelu_backward_sums_supported(input->cols)) {
        partial_rows = gelu_backward_sums_blocks(input->rows, input->cols);
        sums = partial_sums_buffer(backend, partial_rows * input->cols);
    }
    {
        OpScope scope(backend, "gelu_backward", 16.0 * double(numel(input)),
                      0.0);
        if (sums) {
            launch_gelu_backward_sums(x, dy, dx, sums, input->rows, input->cols,
                                      add, backend->stream);
        } else {
            launch_gelu_backward(x, dy, dx, numel(input), add, backend->stream);
        }
    }
    if (sums) {
        column_memo_commit(backend, dx, input->rows, input->cols, sums,
                           partial_rows);
    }
    return 0;
}

constexpr size_t kMaxHeadDim = 128;

// Short sequences on the FP32 path: the probability matrix is half of the
// forward pass's traffic and the backward pass can rebuild it from Q and K in
// shared memory, so it is not written at all.  The host still owns a tensor
// for it; that tensor is declared to be softmax(scale Q K^T) and is computed
// only if somebody reads it.  On the same path the head-major copies of the
// projections and of their gradients are not made either (see HeadView).
//
// Returns 0 when the path does not apply, 1 for the FP32 whole-group kernels
// (seq <= 128), 2 for the tensor-core whole-group kernels (seq <= 64) and 3
// for the tensor-core streaming kernels (any length); tensor cores (TF32
// operands) are chosen like a matrix product's precision: forced by the
// policy, otherwise by the amount of work.
int short_attention_kind(size_t groups, size_t seq, size_t head_dim) {
    const int policy = gemm_default_precision();
    const double work = double(groups) * double(seq) * double(seq) * double(head_dim);
    if (policy != VITB200_PRECISION_FP32 && prefer_tensor_cores(policy, work)) {
        if (attention_warp_supported(seq, head_dim)) {
            return 2;
        }
        if (attention_stream_supported(head_dim)) {
            return 3;
        }
    }
    if (policy != VITB200_PRECISION_TF32 &&
        attention_small_supported(seq, head_dim)) {
        return 1;
    }
    return 0;
}

// Arguments of a pending head view: the output is columns
// [col0, col0 + d_model) of a token-major [batch*seq, row_floats] matrix,
// regrouped per head (what split_heads writes for one of Q, K, V, and what
// merge_heads_backward writes).
struct HeadView {
    size_t batch, seq, d_model, heads, row_floats, col0;
};

void materialise_head_view(const void *arguments, float *output,
                           float *const *sources, cudaStream_t stream) {
    HeadView d;
    memcpy(&d, arguments, sizeof(d));
    launch_head_view(sources[0], output, d.batch, d.seq, d.d_model, d.heads,
                     d.row_floats, d.col0, stream);
}

bool define_head_view(CudaBackend *backend, const void *output,
                      const void *matrix, size_t batch, size_t seq,
                      size_t d_model, size_t heads, size_t row_floats,
                      size_t col0) {
    const HeadView definition = {batch, seq, d_model, heads, row_floats, col0};
    const void *sources[1] = {matrix};
    return coherent_define_lazy(output, sources, 1, materialise_head_view,
                                &definition, sizeof(definition),
                                backend->stream);
}

// An attention operand: where its values can be read right now.
struct HeadOperand {
    const float *pointer = nullptr;
    HeadLayout layout;
    const void *matrix_host = nullptr;   // set when read through a head view
    size_t col0 = 0;
};

// If `host` is a pending head view with the geometry the attention call
// expects, points the operand at the matrix underneath; the view itself stays
// pending.
bool through_head_view(const void *host, size_t batch, size_t heads, size_t seq,
                       size_t head_dim, HeadOperand *operand) {
    HeadView d;
    const float *matrix = nullptr;
    const void *matrix_host = nullptr;
    if (!coherent_lazy_source(host, materialise_head_view, &d, sizeof(d),
                              &matrix, &matrix_host) ||
        d.batch != batch || d.heads != heads || d.seq != seq ||
        d.d_model != heads * head_dim || d.row_floats % 4 != 0 ||
        d.col0 % 4 != 0 || !fits_int(d.row_floats)) {
        return false;
    }
    operand->pointer = matrix + d.col0;
    operand->layout.ld = int(d.row_floats);
    operand->layout.heads = int(heads);
    operand->matrix_host = matrix_host;
    operand->col0 = d.col0;
    return true;
}

// Operand for reading: through a pending head view when there is one,
// otherwise the tensor itself (computing whatever defines it).
HeadOperand read_operand(CudaBackend *backend, const void *host, size_t batch,
                         size_t heads, size_t seq, size_t head_dim,
                         bool allow_view) {
    HeadOperand operand;
    if (!allow_view ||
        !through_head_view(host, batch, heads, seq, head_dim, &operand)) {
        operand = HeadOperand();
        operand.pointer = view(backend, host, Access::Read);
    }
    return operand;
}

bool same_layout(const HeadLayout &a, const HeadLayout &b) {
    return a.ld == b.ld && a.heads == b.heads;
}

int op_split_heads(void *context, const vitb200_tensor *projected,
                   vitb200_tensor *query, vitb200_tensor *key,
                   vitb200_tensor *value, size_t batch, size_t seq,
                   size_t d_model, size_t heads) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({projected->data, query->data, key->data, value->data})) {
        return -1;
    }
    const float *p = view(backend, projected->data, Access::Read);
    if (heads > 0 &&
        short_attention_kind(batch * heads, seq, d_model / heads) != 0 &&
        define_head_view(backend, query->data, projected->data, batch, seq,
                         d_model, heads, 3 * d_model, 0) &&
        define_head_view(backend, key->data, projected->data, batch, seq,
                         d_model, heads, 3 * d_model, d_model) &&
        define_head_view(backend, value->data, projected->data, batch, seq,
                         d_model, heads, 3 * d_model, 2 * d_model)) {
        return 0;
    }
    float *q = view(backend, query->data, Access::Overwrite);
    float *k = view(backend, key->data, Access::Overwrite);
    float *v = view(backend, value->data, Access::Overwrite);
    {
        OpScope scope(backend, "split_heads", 8.0 * double(numel(projected)),
                      0.0);
        launch_split_heads(p, q, k, v, batch, seq, d_model, heads, backend->stream);
    }
    return 0;
}

int op_split_heads_backward(void *context, vitb200_tensor *projected,
                            const vitb200_tensor *query,
                            const vitb200_tensor *key,
                            const vitb200_tensor *value, size_t batch,
                            size_t seq, size_t d_model, size_t heads) {
    CudaBackend *backend = self(context);
    if (!ours({projected->grad, query->grad, key->grad, value->grad})) {
        flush_pending(backend, true);
        return -1;
    }
    // The attention backward pass that produces the three gradients is still
    // held back and nothing else has been added to them or to the projected
    // gradient: let it write the projected gradient directly and make the
    // three tensors views of that.
    PendingAttentionBackward &held = backend->pending_attention_backward;
    if (held.active && held.dq_host == query->grad &&
        held.dk_host == key->grad && held.dv_host == value->grad &&
        held.batch == batch && held.heads == heads && held.seq == seq &&
        held.head_dim * heads == d_model && fits_int(3 * d_model) &&
        coherent_is_zero_pending(query->grad) &&
        coherent_is_zero_pending(key->grad) &&
        coherent_is_zero_pending(value->grad) &&
        coherent_is_zero_pending(projected->grad)) {
        const PendingAttentionBackward pending = held;
        held.active = false;
        flush_pending(backend, true);
        float *p = view(backend, projected->grad, Access::Overwrite);
        HeadLayout grad_layout;
        grad_layout.ld = int(3 * d_model);
        grad_layout.heads = int(heads);
        // The tensor-core kernel also leaves per-sample column sums of what it
        // writes: the QKV bias gradient the host asks for next
        // (reference src/vit.c:588-591) then sums [batch, 3d] instead of
        // [batch * seq, 3d].
        // (Whole-group kernels: one row per sample.  tcgen05 kernels: one row
        // per CTA of their persistent grid.)
        const bool from_tc = pending.kind == 3 &&
                             tc_attention_wanted(seq, pending.head_dim);
        const size_t partial_rows =
            pending.kind == 2 ? batch : (from_tc ? attention_tc_partial_rows() : 0);
        float *partials = partial_rows
            ? partial_sums_buffer(backend, partial_rows * 3 * d_model)
            : nullptr;
        if (!run_attention_backward(backend, pending, p, p + d_model,
                                    p + 2 * d_model, false, false, false,
                                    grad_layout, partials)) {
            partials = nullptr;
        }
        const vitb200_tensor *parts[3] = {query, key, value};
        for (size_t which = 0; which < 3; ++which) {
            if (!define_head_view(backend, parts[which]->grad, projected->grad,
                                  batch, seq, d_model, heads, 3 * d_model,
                                  which * d_model)) {
                float *part =
                    view(backend, parts[which]->grad, Access::Overwrite);
                launch_head_view(p, part, batch, seq, d_model, heads,
                                 3 * d_model, which * d_model,
                                 backend->stream);
            }
        }
        backend->fused_head_layouts += 1;
        if (partials) {
            column_memo_commit(backend, p, batch * seq, 3 * d_model, partials,
                               partial_rows);
        }
        return 0;
    }
    flush_pending(backend, true);
    bool add = true;
    float *p = accumulate_view(backend, projected->grad, &add);
    const float *q = view(backend, query->grad, Access::Read);
    const float *k = view(backend, key->grad, Access::Read);
    const float *v = view(backend, value->grad, Access::Read);
    {
        OpScope scope(backend, "split_heads_backward", 12.0 * double(numel(projected)),
                      0.0);
        launch_split_heads_backward(p, q, k, v, batch, seq, d_model, heads,
                                    add, backend->stream);
    }
    return 0;
}

int op_merge_heads(void *context, const vitb200_tensor *attended,
                   vitb200_tensor *merged, size_t batch, size_t seq,
                   size_t d_model, size_t heads) {
    CudaBackend *backend = self(context);
    if (!ours({attended->data, merged->data})) {
        flush_pending(backend);
        return -1;
    }
    PendingAttention &held = backend->pending_attention;
    if (held.active && held.output_host == attended->data &&
        held.batch == batch && held.heads == heads && held.seq == seq &&
        held.head_dim * heads == d_model && fits_int(d_model)) {
        const PendingAttention pending = held;
        held.active = false;
        flush_pending(backend);
        float *m = view(backend, merged->data, Access::Overwrite);
        HeadLayout out_layout;
        out_layout.ld = int(d_model);
        out_layout.heads = int(heads);
        run_attention(backend, pending, m, out_layout);
        if (!define_head_view(backend, attended->data, merged->data, batch, seq,
                              d_model, heads, d_model, 0)) {
            float *a = view(backend, attended->data, Access::Overwrite);
            launch_head_view(m, a, batch, seq, d_model, heads, d_model, 0,
                             backend->stream);
        }
        backend->fused_head_layouts += 1;
        return 0;
    }
    flush_pending(backend);
    const float *a = view(backend, attended->data, Access::Read);
    float *m = view(backend, merged->data, Access::Overwrite);
    {
        OpScope scope(backend, "merge_heads", 8.0 * double(numel(merged)),
                      0.0);
        launch_merge_heads(a, m, batch, seq, d_model, heads, backend->stream);
    }
    return 0;
}

int op_merge_heads_backward(void *context, vitb200_tensor *attended,
                            const vitb200_tensor *merged, size_t batch,
                            size_t seq, size_t d_model, size_t heads) {
    CudaBackend *backend = self(context);
    flush_pending(backend, true);
    if (!ours({attended->grad, merged->grad})) {
        return -1;
    }
    const float *m = view(backend, merged->grad, Access::Read);
    // Nothing has been added to the head-major gradient yet: it simply is
    // the merged gradient regrouped, which attention_backward can read in
    // place.
    if (heads > 0 &&
        short_attention_kind(batch * heads, seq, d_model / heads) != 0 &&
        coherent_is_zero_pending(attended->grad) &&
        define_head_view(backend, attended->grad, merged->grad, batch, seq,
                         d_model, heads, d_model, 0)) {
        return 0;
    }
    bool add = true;
    float *a = accumulate_view(backend, attended->grad, &add);
    {
        OpScope scope(backend, "merge_heads_backward", 12.0 * double(numel(merged)),
                      0.0);
        launch_merge_heads_backward(a, m, batch, seq, d_model, heads, add,
                                    backend->stream);
    }
    return 0;
}

// Arguments of a pending probability matrix (see op_attention).  With one
// source the queries and keys are read through head views of that matrix
// (column offsets q_col0 / k_col0, row stride ld); with two sources they are
// the head-major Q and K tensors.
struct ProbabilityDefinition {
    size_t groups, seq, head_dim;
    float scale;
    int tensor_cores;   // which forward kernel defines the values
    int ld, heads;
    size_t q_col0, k_col0;
};

// Produces P = softmax(scale Q K^T) for a definition that somebody finally
// reads.  The kernel's V input is irrelevant when only P is written, K stands
// in for it.
void materialise_probabilities(const void *arguments, float *output,
                               float *const *sources, cudaStream_t stream) {
    ProbabilityDefinition d;
    memcpy(&d, arguments, sizeof(d));
    if (d.ld && !attention_small_supported(d.seq, d.head_dim)) {
        // Long sequences read through head views: regroup Q and K into
        // temporary head-major buffers for the kernel that writes P.  Only a
        // host that asks for P ever gets here, so the allocation is made (and
        // released) on the spot.
        const size_t elements = d.groups * d.seq * d.head_dim;
        const size_t batch = d.groups / size_t(d.heads);
        const size_t d_model = size_t(d.heads) * d.head_dim;
        float *regrouped = nullptr;
        check(cudaMalloc(&regrouped, 2 * elements * sizeof(float)), "cudaMalloc");
        launch_head_view(sources[0], regrouped, batch, d.seq, d_model, d.heads,
                         size_t(d.ld), d.q_col0, stream);
        launch_head_view(sources[0], regrouped + elements, batch, d.seq, d_model,
                         d.heads, size_t(d.ld), d.k_col0, stream);
        launch_attention_mma_forward(regrouped, regrouped + elements,
                                     regrouped + elements, output, nullptr,
                                     d.groups, d.seq, d.head_dim, d.scale,
                                     stream);
        check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        check(cudaFree(regrouped), "cudaFree");
        return;
    }
    if (d.ld) {
        HeadLayout layout;
        layout.ld = d.ld;
        layout.heads = d.heads;
        launch_attention_small_forward(
            sources[0] + d.q_col0, sources[0] + d.k_col0, sources[0] + d.k_col0,
            output, nullptr, d.groups, d.seq, d.head_dim, d.scale, true, false,
            stream, layout);
        return;
    }
    if (d.tensor_cores) {
        launch_attention_mma_forward(sources[0], sources[1], sources[1], output,
                                     nullptr, d.groups, d.seq, d.head_dim,
                                     d.scale, stream);
        return;
    }
    launch_attention_small_forward(sources[0], sources[1], sources[1], output,
                                   nullptr, d.groups, d.seq, d.head_dim,
                                   d.scale, true, false, stream);
}

int op_attention(void *context, const vitb200_tensor *query,
                 const vitb200_tensor *key, const vitb200_tensor *value,
                 size_t batch, size_t heads, size_t seq, float scale,
                 vitb200_tensor *probabilities, vitb200_tensor *output) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({query->data, key->data, value->data, probabilities->data,
               output->data}) ||
        query->cols > kMaxHeadDim || value->cols != query->cols ||
        !fits_int(seq) || !fits_int(batch * heads)) {
        return -1;
    }
    const size_t groups = batch * heads;
    const size_t head_dim = query->cols;
    const double flops = 4.0 * double(numel(probabilities)) * double(head_dim);
    const int kind = short_attention_kind(groups, seq, head_dim);
    if (kind != 0) {
        HeadOperand q, k, v;
        const bool through =
            through_head_view(query->data, batch, heads, seq, head_dim, &q) &&
            through_head_view(key->data, batch, heads, seq, head_dim, &k) &&
            through_head_view(value->data, batch, heads, seq, head_dim, &v) &&
            q.matrix_host && q.matrix_host == k.matrix_host &&
            same_layout(q.layout, k.layout) && same_layout(q.layout, v.layout);
        bool defined = false;
        if (through) {
            const ProbabilityDefinition definition = {
                groups, seq, head_dim, scale, 0, q.layout.ld, q.layout.heads,
                q.col0, k.col0};
            const void *sources[1] = {q.matrix_host};
            defined = coherent_define_lazy(probabilities->data, sources, 1,
                                           materialise_probabilities,
                                           &definition, sizeof(definition),
                                           backend->stream);
        }
        if (!defined) {
            q = read_operand(backend, query->data, batch, heads, seq, head_dim, false);
            k = read_operand(backend, key->data, batch, heads, seq, head_dim, false);
            v = read_operand(backend, value->data, batch, heads, seq, head_dim, false);
            const ProbabilityDefinition definition = {
                groups, seq, head_dim, scale,
                attention_small_supported(seq, head_dim) ? 0 : 1, 0, 1, 0, 0};
            const void *sources[2] = {query->data, key->data};
            defined = coherent_define_lazy(probabilities->data, sources, 2,
                                           materialise_probabilities,
                                           &definition, sizeof(definition),
                                           backend->stream);
        }
        if (defined) {
            PendingAttention &pending = backend->pending_attention;
            pending.active = true;
            pending.kind = kind;
            pending.lse = nullptr;
            if (kind == 3) {
                pending.lse = scratch<float>(
                    backend, backend->lse_buffers[probabilities->data],
                    groups * seq);
                backend->lse_streamed[probabilities->data] = true;
            }
            pending.q = q.pointer;
            pending.k = k.pointer;
            pending.v = v.pointer;
            pending.in_layout = q.layout;
            pending.output_host = output->data;
            pending.batch = batch;
            pending.heads = heads;
            pending.seq = seq;
            pending.head_dim = head_dim;
            pending.scale = scale;
            pending.bytes = 16.0 * double(numel(query));
            pending.flops = flops;
            return 0;
        }
    }
    const float *q = view(backend, query->data, Access::Read);
    const float *k = view(backend, key->data, Access::Read);
    const float *v = view(backend, value->data, Access::Read);
    float *o = view(backend, output->data, Access::Overwrite);
    // Long sequences on tensor cores: flash attention.  One sweep, P never
    // written; the row log-sum-exp is kept for the backward pass and P itself
    // stays a pending definition.
    const double work = double(groups) * seq * seq * head_dim;
    if (!attention_small_supported(seq, head_dim) &&
        attention_mma_supported(head_dim) &&
        prefer_tensor_cores(VITB200_PRECISION_AUTO, work)) {
        const ProbabilityDefinition definition = {groups, seq, head_dim,
                                                  scale, 1, 0, 1, 0, 0};
        const void *sources[2] = {query->data, key->data};
        Scratch &buffer = backend->lse_buffers[probabilities->data];
        float *lse = scratch<float>(backend, buffer, groups * seq);
        if (coherent_define_lazy(probabilities->data, sources, 2,
                                 materialise_probabilities, &definition,
                                 sizeof(definition), backend->stream)) {
            OpScope scope(backend, "multi_head_attention",
                          16.0 * double(numel(query)), flops);
            // The register-resident streaming kernels where they exist
            // (head_dim 16, 32, 64); the two families keep different
            // log-sum-exp conventions, remembered per tensor.
            if (long_attention_forward(backend, q, k, v, o, lse, groups, seq,
                                       head_dim, scale)) {
                backend->lse_streamed[probabilities->data] = true;
                return 0;
            }
            backend->lse_streamed[probabilities->data] = false;
            if (launch_attention_mma_flash_forward(q, k, v, o, lse, groups, seq,
                                                   head_dim, scale,
                                                   backend->stream)) {
                return 0;
            }
        }
    }
    float *p = view(backend, probabilities->data, Access::Overwrite);
    {
        OpScope scope(backend, "multi_head_attention", 4.0 * (4.0 * double(numel(query)) + double(numel(probabilities))),
                      flops);
        launch_attention_forward(q, k, v, p, o, groups, seq, head_dim,
                                 scale, VITB200_PRECISION_AUTO,
                                 backend->stream);
    }
    return 0;
}

int op_attention_backward(void *context, const vitb200_tensor *query,
                          const vitb200_tensor *key,
                          const vitb200_tensor *value, size_t batch,
                          size_t heads, size_t seq, float scale,
                          const vitb200_tensor *probabilities,
                          const vitb200_tensor *output,
                          vitb200_tensor *query_grad, vitb200_tensor *key_grad,
                          vitb200_tensor *value_grad) {
    CudaBackend *backend = self(context);
    flush_pending(backend, true);
    if (!ours({query->data, key->data, value->data, probabilities->data,
               output->data, output->grad, query_grad->grad, key_grad->grad,
               value_grad->grad}) ||
        query->cols > kMaxHeadDim || value->cols != query->cols ||
        !fits_int(seq) || !fits_int(batch * heads)) {
        return -1;
    }
    const size_t groups = batch * heads;
    const size_t head_dim = query->cols;
    const bool pending_p = coherent_is_lazy(probabilities->data);
    const int kind = short_attention_kind(groups, seq, head_dim);
    // The streaming kernels rebuild P from the log-sum-exp their own forward
    // pass saved.
    const float *streamed_lse = nullptr;
    if (pending_p && kind == 3) {
        auto found = backend->lse_buffers.find(probabilities->data);
        auto streamed = backend->lse_streamed.find(probabilities->data);
        if (found != backend->lse_buffers.end() &&
            found->second.bytes >= groups * seq * sizeof(float) &&
            streamed != backend->lse_streamed.end() && streamed->second) {
            streamed_lse = static_cast<const float *>(found->second.memory);
        }
    }
    const bool recompute =
        pending_p && kind != 0 && (kind != 3 || streamed_lse != nullptr);
    const double bytes = 4.0 * (11.0 * double(numel(query)) +
                                (recompute ? 0.0 : double(numel(probabilities))));
    const double flops = 8.0 * double(numel(probabilities)) * double(head_dim);
    if (recompute) {
        // Short sequences: P is rebuilt in shared memory; every operand that
        // is a pending head view is read in place.  The launch is held back
        // for op_split_heads_backward.
        HeadOperand q, k, v;
        const bool through =
            through_head_view(query->data, batch, heads, seq, head_dim, &q) &&
            through_head_view(key->data, batch, heads, seq, head_dim, &k) &&
            through_head_view(value->data, batch, heads, seq, head_dim, &v) &&
            same_layout(q.layout, k.layout) && same_layout(q.layout, v.layout);
        if (!through) {
            q = read_operand(backend, query->data, batch, heads, seq, head_dim, false);
            k = read_operand(backend, key->data, batch, heads, seq, head_dim, false);
            v = read_operand(backend, value->data, batch, heads, seq, head_dim, false);
        }
        const HeadOperand o = read_operand(backend, output->data, batch, heads,
                                           seq, head_dim, true);
        const HeadOperand go = read_operand(backend, output->grad, batch, heads,
                                            seq, head_dim, true);
        PendingAttentionBackward &pending = backend->pending_attention_backward;
        pending.active = true;
        pending.kind = kind;
        pending.lse = streamed_lse;
        pending.q = q.pointer;
        pending.k = k.pointer;
        pending.v = v.pointer;
        pending.out = o.pointer;
        pending.dout = go.pointer;
        pending.in_layout = q.layout;
        pending.out_layout = o.layout;
        pending.dout_layout = go.layout;
        pending.dq_host = query_grad->grad;
        pending.dk_host = key_grad->grad;
        pending.dv_host = value_grad->grad;
        pending.batch = batch;
        pending.heads = heads;
        pending.seq = seq;
        pending.head_dim = head_dim;
        pending.scale = scale;
        pending.bytes = bytes;
        pending.flops = flops;
        return 0;
    }
    float *dots = scratch<float>(backend, backend->rows_scratch, groups * seq);
    const float *q = view(backend, query->data, Access::Read);
    const float *k = view(backend, key->data, Access::Read);
    const float *v = view(backend, value->data, Access::Read);
    const float *lse = nullptr;
    if (pending_p) {
        auto found = backend->lse_buffers.find(probabilities->data);
        if (found != backend->lse_buffers.end() &&
            found->second.bytes >= groups * seq * sizeof(float)) {
            lse = static_cast<const float *>(found->second.memory);
        }
    }
    const float *p =
        lse ? nullptr : view(backend, probabilities->data, Access::Read);
    const float *o = view(backend, output->data, Access::Read);
    const float *go = view(backend, output->grad, Access::Read);
    bool add_q = true, add_k = true, add_v = true;
    float *dq = accumulate_view(backend, query_grad->grad, &add_q);
    float *dk = accumulate_view(backend, key_grad->grad, &add_k);
    float *dv = accumulate_view(backend, value_grad->grad, &add_v);
    {
        OpScope scope(backend, "multi_head_attention_backward", bytes, flops);
        if (lse && backend->lse_streamed[probabilities->data]) {
            long_attention_backward(backend, q, k, v, o, go, lse, dq, dk, dv,
                                    dots, groups, seq, head_dim, scale, add_q,
                                    add_k, add_v);
        } else if (lse) {
            launch_attention_mma_backward(q, k, v, nullptr, lse, o, go, dq, dk,
                                          dv, dots, groups, seq, head_dim,
                                          scale, add_q, add_k, add_v,
                                          backend->stream);
        } else {
            launch_attention_backward(q, k, v, p, o, go, dq, dk, dv, dots,
                                      groups, seq, head_dim, scale, add_q,
                                      add_k, add_v, VITB200_PRECISION_AUTO,
                                      backend->stream);
        }
    }
    return 0;
}

int op_zero_gradient(void *context, vitb200_tensor *tensor) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({tensor->grad})) {
        return -1;
    }
    // Nothing is written here: the buffer is declared zero, the first kernel
    // that adds into it stores instead, and a fill is issued only if somebody
    // reads the zeros first.
    coherent_mark_zero(tensor->grad, backend->stream);
    return 0;
}

// Largest gradient buffer that the batched zero fill covers.  Above it the
// fill's own traffic outweighs the launch it saves, and a product that is the
// first writer would rather skip the read (see coherent_mark_zero).
constexpr size_t kBatchedZeroBytes = size_t(1) << 20;

int op_zero_gradients(void *context, vitb200_tensor *const *tensors,
                      size_t count) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    for (size_t i = 0; i < count; ++i) {
        if (!coherent_owns(tensors[i]->grad)) {
            return -1;
        }
    }
    std::vector<const void *> gradients(count);
    for (size_t i = 0; i < count; ++i) {
        coherent_mark_zero(tensors[i]->grad, backend->stream);
        gradients[i] = tensors[i]->grad;
    }
    // The small ones (biases, layer-norm parameters, narrow weight matrices)
    // are accumulated into by kernels that need the zeros in memory; writing
    // them all now is one launch instead of a memset node before each.
    static const bool batched = getenv("VITB200_NO_BATCHED_ZERO_FILL") == nullptr;
    if (batched && count > 1) {
        if (coherent_zero_fill_batch(gradients.data(), count, kBatchedZeroBytes,
                                     backend->stream)) {
            ++g_kernel_launches;
        }
    }
    return 0;
}

int op_extract_patches(void *context, const vitb200_tensor *images,
                       vitb200_tensor *patches, size_t channels, size_t height,
                       size_t width, size_t patch) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({images->data, patches->data})) {
        return -1;
    }
    const float *in = view(backend, images->data, Access::Read);
    float *out = view(backend, patches->data, Access::Overwrite);
    {
        OpScope scope(backend, "extract_patches", 8.0 * double(numel(patches)),
                      0.0);
        launch_extract_patches(in, out, images->rows, channels, height, width,
                               patch, backend->stream);
    }
    return 0;
}

int op_token_embedding(void *context, const vitb200_tensor *patch_tokens,
                       const vitb200_tensor *cls, const vitb200_tensor *pos,
                       vitb200_tensor *tokens, size_t batch) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({patch_tokens->data, cls->data, pos->data, tokens->data})) {
        return -1;
    }
    const float *p = view(backend, patch_tokens->data, Access::Read);
    const float *c = view(backend, cls->data, Access::Read);
    const float *e = view(backend, pos->data, Access::Read);
    float *t = view(backend, tokens->data, Access::Overwrite);
    {
        OpScope scope(backend, "token_embedding", 8.0 * double(numel(tokens)),
                      0.0);
        launch_token_embedding(p, c, e, t, batch, pos->rows, tokens->cols,
                               backend->stream);
    }
    return 0;
}

int op_token_embedding_backward(void *context, vitb200_tensor *patch_tokens,
                                vitb200_tensor *cls, vitb200_tensor *pos,
                                const vitb200_tensor *tokens, size_t batch) {
    CudaBackend *backend = self(context);
    flush_pending(backend, true);
    if (!ours({patch_tokens->grad, cls->grad, pos->grad, tokens->grad})) {
        return -1;
    }
    bool add_patch = true;
    float *p = accumulate_view(backend, patch_tokens->grad, &add_patch);
    float *c = view(backend, cls->grad, Access::ReadWrite);
    float *e = view(backend, pos->grad, Access::ReadWrite);
    const float *t = view(backend, tokens->grad, Access::Read);
    {
        OpScope scope(backend, "token_embedding_backward", 12.0 * double(numel(tokens)),
                      0.0);
        launch_token_embedding_backward(p, c, e, t, batch, pos->rows, tokens->cols,
                                        add_patch, backend->stream);
    }
    dp_gradient_produced(backend->dp, cls->grad, c, numel(cls));
    dp_gradient_produced(backend->dp, pos->grad, e, numel(pos));
    return 0;
}

int op_gather_rows(void *context, const vitb200_tensor *source,
                   vitb200_tensor *destination, size_t row_stride) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({source->data, destination->data})) {
        return -1;
    }
    const float *s = view(backend, source->data, Access::Read);
    float *d = view(backend, destination->data, Access::Overwrite);
    {
        OpScope scope(backend, "gather_rows", 8.0 * double(numel(destination)),
                      0.0);
        launch_gather_rows(s, d, destination->rows, destination->cols, row_stride,
                           backend->stream);
    }
    return 0;
}

int op_gather_rows_backward(void *context, vitb200_tensor *source,
                            const vitb200_tensor *destination,
                            size_t row_stride) {
    CudaBackend *backend = self(context);
    flush_pending(backend, true);
    if (!ours({source->grad, destination->grad})) {
        return -1;
    }
    dp_gradient_touched(backend->dp, source->grad);
    float *s = view(backend, source->grad, Access::ReadWrite);
    const float *d = view(backend, destination->grad, Access::Read);
    {
        OpScope scope(backend, "gather_rows_backward", 12.0 * double(numel(destination)),
                      0.0);
        launch_gather_rows_backward(s, d, destination->rows, destination->cols,
                                    row_stride, backend->stream);
    }
    return 0;
}

int op_softmax_cross_entropy(void *context, const vitb200_tensor *logits,
                             const vitb200_tensor *targets,
                             const vitb200_tensor *class_weights,
                             float label_smoothing, vitb200_tensor *loss,
                             vitb200_tensor *logits_grad) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({logits->data, targets->data, loss->data, logits_grad->grad}) ||
        (class_weights && !coherent_owns(class_weights->data))) {
        return -1;
    }
    float *row_losses =
        scratch<float>(backend, backend->rows_scratch, logits->rows);
    const float *z = view(backend, logits->data, Access::Read);
    const float *t = view(backend, targets->data, Access::Read);
    const float *w = class_weights
        ? view(backend, class_weights->data, Access::Read)
        : nullptr;
    float *l = view(backend, loss->data, Access::Overwrite);
    float *g = view(backend, logits_grad->grad, Access::ReadWrite);
    {
        OpScope scope(backend, "softmax_cross_entropy", 16.0 * double(numel(logits)),
                      0.0);
        launch_softmax_cross_entropy(z, t, w, label_smoothing, l, g, row_losses,
                                     logits->rows, logits->cols, backend->stream);
    }
    if (backend->deferred_synchronize) {
        // The host reads the loss at the end of the step: send it on its way
        // now, so that the read waits for the forward pass only.
        coherent_prefetch_host(loss->data, backend->stream);
    }
    return 0;
}

// Copies `bytes` from host memory into a device buffer through the pinned
// ring, without waiting for earlier work on the stream.
void upload_small(CudaBackend *backend, void *device, const void *host,
                  size_t bytes) {
    const int slot = backend->staging_next;
    backend->staging_next = (slot + 1) % kStagingSlots;
    check(cudaEventSynchronize(backend->staging_done[slot]),
          "cudaEventSynchronize");
    memcpy(backend->staging[slot], host, bytes);
    check(cudaMemcpyAsync(device, backend->staging[slot], bytes,
                          cudaMemcpyHostToDevice, backend->stream),
          "cudaMemcpyAsync");
    check(cudaEventRecord(backend->staging_done[slot], backend->stream),
          "cudaEventRecord");
}

struct SliceTable {
    const ParameterSlice *device = nullptr;
    unsigned slices = 0;
    unsigned blocks = 0;
    double elements = 0.0;
};

// with_moments = false builds a gradient-only table (for clipping alone).
int build_slice_table(CudaBackend *backend,
                      vitb200_parameter *const *parameters,
                      const float *weight_decays, size_t count, float beta1,
                      float beta2, bool with_moments, SliceTable *table) {
    if (count == 0 || count * sizeof(ParameterSlice) > kStagingBytes) {
        return -1;
    }
    for (size_t i = 0; i < count; ++i) {
        const vitb200_parameter *p = parameters[i];
        if (!ours({p->value.grad}) ||
            (with_moments && !ours({p->value.data, p->m, p->v}))) {
            return -1;
        }
    }
    std::vector<ParameterSlice> slices(count);
    unsigned long long blocks = 0;
    for (size_t i = 0; i < count; ++i) {
        vitb200_parameter *p = parameters[i];
        ParameterSlice &slice = slices[i];
        slice.value = with_moments
            ? view(backend, p->value.data, Access::ReadWrite) : nullptr;
        slice.grad = view(backend, p->value.grad, Access::ReadWrite);
        slice.m = with_moments ? view(backend, p->m, Access::ReadWrite) : nullptr;
        slice.v = with_moments ? view(backend, p->v, Access::ReadWrite) : nullptr;
        slice.count = numel(&p->value);
        slice.first_block = blocks;
        slice.weight_decay = weight_decays ? weight_decays[i] : 0.0f;
        // The host has already advanced `step` (reference src/ops.c:1140-1142).
        slice.correction1 = 1.0f - powf(beta1, float(p->step));
        slice.correction2 = 1.0f - powf(beta2, float(p->step));
        slice.pad = 0.0f;
        blocks += (slice.count + kSliceBlockElements - 1) / kSliceBlockElements;
    }
    if (blocks == 0 || blocks > unsigned(INT_MAX)) {
        return -1;
    }
    ParameterSlice *device =
        scratch<ParameterSlice>(backend, backend->slice_table, count);
    upload_small(backend, device, slices.data(),
                 count * sizeof(ParameterSlice));
    table->device = device;
    table->slices = unsigned(count);
    table->blocks = unsigned(blocks);
    for (const ParameterSlice &slice : slices) {
        table->elements += double(slice.count);
    }
    return 0;
}

int op_clip_gradient_norm(void *context, vitb200_parameter *const *parameters,
                          size_t count, float max_norm) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    SliceTable table;
    if (build_slice_table(backend, parameters, nullptr, count, 0.0f, 0.0f,
                          false, &table) != 0) {
        return -1;
    }
    float *partials =
        scratch<float>(backend, backend->norm_partials, table.blocks);
    float *scale = scratch<float>(backend, backend->clip_scale, 1);
    OpScope scope(backend, "clip_gradient_norm", 12.0 * table.elements, 0.0);
    launch_gradient_clip_scale(table.device, table.slices, table.blocks,
                               max_norm, 1.0f, partials, scale,
                               backend->stream);
    launch_scale_gradients(table.device, table.slices, table.blocks, scale,
                           backend->stream);
    return 0;
}

int op_adamw_step(void *context, vitb200_parameter *parameter, float lr,
                  float beta1, float beta2, float epsilon, float weight_decay,
                  float correction1, float correction2) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    if (!ours({parameter->value.data, parameter->value.grad, parameter->m,
               parameter->v})) {
        return -1;
    }
    float *w = view(backend, parameter->value.data, Access::ReadWrite);
    float *g = view(backend, parameter->value.grad, Access::ReadWrite);
    float *m = view(backend, parameter->m, Access::ReadWrite);
    float *v = view(backend, parameter->v, Access::ReadWrite);
    {
        OpScope scope(backend, "adamw_step", 28.0 * double(numel(&parameter->value)),
                      0.0);
        launch_adamw_single(w, g, m, v, numel(&parameter->value), lr, beta1, beta2,
                            epsilon, weight_decay, correction1, correction2,
                            backend->stream);
    }
    return 0;
}

int op_adamw_step_parameters(void *context,
                             vitb200_parameter *const *parameters,
                             const float *weight_decays, size_t count, float lr,
                             float beta1, float beta2, float epsilon,
                             float max_gradient_norm) {
    CudaBackend *backend = self(context);
    flush_pending(backend);
    for (size_t i = 0; i < count; ++i) {
        if (!ours({parameters[i]->value.data, parameters[i]->value.grad,
                   parameters[i]->m, parameters[i]->v})) {
            return -1;
        }
    }
    // Data parallel: finish the gradient exchange first; the summed gradients
    // are turned into their mean by the scale the update multiplies by.  (The
    // exchange may move the gradients' device buffers, so it comes before the
    // table of pointers the kernels work from.)
    float inverse_world = 1.0f;
    if (backend->dp && dp_status(backend->dp) != 0) {
        return -1;   // the exchange has failed: nothing sensible to apply
    }
    if (backend->dp && dp_world(backend->dp) > 1) {
        std::vector<const void *> host_grads(count);
        std::vector<float *> device_grads(count);
        std::vector<size_t> counts(count);
        for (size_t i = 0; i < count; ++i) {
            host_grads[i] = parameters[i]->value.grad;
            device_grads[i] =
                view(backend, parameters[i]->value.grad, Access::ReadWrite);
            counts[i] = numel(&parameters[i]->value);
        }
        inverse_world = dp_before_optimizer(backend->dp, host_grads.data(),
                                            device_grads.data(), counts.data(),
                                            count);
    }
    SliceTable table;
    if (build_slice_table(backend, parameters, weight_decays, count, beta1,
                          beta2, true, &table) != 0) {
        return -1;
    }
    // Gradient accumulation: the gradients are sums over micro-batches as well.
    inverse_world *= backend->accumulation_inverse;
    const bool needs_scale = max_gradient_norm > 0.0f || inverse_world != 1.0f;
    const float *scale = nullptr;
    float *partials = nullptr, *scale_out = nullptr;
    if (needs_scale) {
        partials = scratch<float>(backend, backend->norm_partials, table.blocks);
        scale_out = scratch<float>(backend, backend->clip_scale, 1);
    }
    OpScope scope(backend, "adamw_step_parameters",
                  (needs_scale ? 32.0 : 28.0) * table.elements, 0.0);
    if (needs_scale) {
        launch_gradient_clip_scale(
            table.device, table.slices, table.blocks,
            max_gradient_norm > 0.0f ? max_gradient_norm : FLT_MAX,
            inverse_world, partials, scale_out, backend->stream);
        scale = scale_out;
    }
    launch_adamw(table.device, table.slices, table.blocks, scale, lr, beta1,
                 beta2, epsilon, backend->stream);
    return 0;
}

// With deferred synchronisation the slot only launches what was held back:
// nothing the host can observe depends on the wait, because every host access
// to memory the device owns faults and waits for exactly what it needs
// (coherence.cu), and the step's loss is prefetched.  The host then prepares
// the next step (zeroing, the copy of the next batch into the input tensor)
// while the device is still in the backward pass of this one.
void op_synchronize(void *context) {
    CudaBackend *backend = self(context);
    if (backend->deferred_synchronize) {
        flush_pending(backend);
        if (const int code = gemm_tc_status()) {
            fprintf(stderr,
                    "vitb200: a tensor-core kernel gave up waiting (code %d)\n",
                    code);
            abort();
        }
        return;
    }
    settle_timers(backend);
}

// Every op slot goes through this wrapper, which counts the calls the slot
// declined (non-zero return: the host synchronises and runs its own CPU loop,
// reference src/ops.c:61-64).  A training or evaluation step that is meant to
// run on the device must leave the count unchanged.
template <auto Slot>
struct Counted;
template <typename... Arguments, int (*Slot)(void *, Arguments...)>
struct Counted<Slot> {
    static int call(void *context, Arguments... arguments) {
        const int status = Slot(context, arguments...);
        if (status != 0) {
            self(context)->declined_ops += 1;
        }
        return status;
    }
};
#define COUNTED(slot) Counted<slot>::call

vitb200_op_table make_table(CudaBackend *backend) {
    vitb200_op_table table = {};
    table.context = backend;
    table.gemm = COUNTED(op_gemm);
    table.gemm_backward = COUNTED(op_gemm_backward);
    table.residual = COUNTED(op_residual);
    table.residual_backward = COUNTED(op_residual_backward);
    table.accumulate_gradient = COUNTED(op_accumulate_gradient);
    table.bias_add = COUNTED(op_bias_add);
    table.bias_add_backward = COUNTED(op_bias_add_backward);
    table.layer_norm = COUNTED(op_layer_norm);
    table.layer_norm_backward = COUNTED(op_layer_norm_backward);
    table.gelu = COUNTED(op_gelu);
    table.gelu_backward = COUNTED(op_gelu_backward);
    table.split_heads = COUNTED(op_split_heads);
    table.split_heads_backward = COUNTED(op_split_heads_backward);
    table.merge_heads = COUNTED(op_merge_heads);
    table.merge_heads_backward = COUNTED(op_merge_heads_backward);
    table.multi_head_attention = COUNTED(op_attention);
    table.multi_head_attention_backward = COUNTED(op_attention_backward);
    table.zero_gradient = COUNTED(op_zero_gradient);
    table.extract_patches = COUNTED(op_extract_patches);
    table.token_embedding = COUNTED(op_token_embedding);
    table.token_embedding_backward = COUNTED(op_token_embedding_backward);
    table.gather_rows = COUNTED(op_gather_rows);
    table.gather_rows_backward = COUNTED(op_gather_rows_backward);
    table.softmax_cross_entropy = COUNTED(op_softmax_cross_entropy);
    table.clip_gradient_norm = COUNTED(op_clip_gradient_norm);
    table.adamw_step = COUNTED(op_adamw_step);
    table.zero_gradients = COUNTED(op_zero_gradients);
    table.adamw_step_parameters = COUNTED(op_adamw_step_parameters);
    table.synchronize = op_synchronize;
    return table;
}

int pick_device(int device_count) {
    const char *explicit_device = getenv("VITB200_DEVICE");
    const char *from_rank = getenv("VITB200_DEVICE_FROM_RANK");
    const char *local_rank = getenv("LOCAL_RANK");
    int device = 0;
    if (explicit_device) {
        device = atoi(explicit_device);
    } else if (from_rank && atoi(from_rank) != 0 && local_rank) {
        device = atoi(local_rank);
    }
    return device >= 0 && device < device_count ? device : -1;
}

cudaStream_t as_stream(void *stream) {
    return static_cast<cudaStream_t>(stream);
}

}  // namespace

// ------------------------------------------------------------------ part 1

extern "C" int cuda_backend_create(CudaBackend **backend) {
    if (!backend) {
        return -1;
    }
    *backend = nullptr;
    int device_count = 0;
    if (cudaGetDeviceCount(&device_count) != cudaSuccess || device_count == 0) {
        cudaGetLastError();
        return 1;
    }
    const int device = pick_device(device_count);
    cudaDeviceProp properties = {};
    if (device < 0 || cudaSetDevice(device) != cudaSuccess ||
        cudaGetDeviceProperties(&properties, device) != cudaSuccess) {
        cudaGetLastError();
        return 1;
    }
    if (properties.major != 10) {
        fprintf(stderr,
                "vitb200: device %d is sm_%d%d; this library carries sm_100a "
                "code only\n",
                device, properties.major, properties.minor);
        return 1;
    }
    CudaBackend *result = new CudaBackend();
    result->device = device;
    if (cudaStreamCreateWithFlags(&result->stream, cudaStreamNonBlocking) !=
        cudaSuccess) {
        delete result;
        return -1;
    }
    bool ok = cudaEventCreate(&result->timer_begin) == cudaSuccess &&
              cudaEventCreate(&result->timer_end) == cudaSuccess &&
              cudaEventCreate(&result->span_begin) == cudaSuccess &&
              cudaEventCreate(&result->span_end) == cudaSuccess;
    for (int i = 0; ok && i < kStagingSlots; ++i) {
        ok = cudaHostAlloc(reinterpret_cast<void **>(&result->staging[i]),
                           kStagingBytes, cudaHostAllocDefault) == cudaSuccess &&
             cudaEventCreateWithFlags(&result->staging_done[i],
                                      cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) {
        cuda_backend_free(result);
        return -1;
    }
    coherence_set_stream(result->stream, flush_hook);
    coherence_set_release_hook(release_hook);
    g_flush_backend = result;
    *backend = result;
    return 0;
}

extern "C" void cuda_backend_free(CudaBackend *backend) {
    if (!backend) {
        return;
    }
    cuda_backend_disable_device_execution(backend);
    if (backend->stream) {
        settle_timers(backend);
    }
    dp_destroy(backend->dp);
    backend->dp = nullptr;
    for (auto &entry : backend->lse_buffers) {
        free_scratch(entry.second);
    }
    backend->lse_buffers.clear();
    free_scratch(backend->rows_scratch);
    free_scratch(backend->norm_partials);
    free_scratch(backend->clip_scale);
    free_scratch(backend->slice_table);
    backend->free_running.push_back(backend->running_sums);
    backend->free_partial.push_back(backend->partial_sums);
    for (std::vector<SumBuffer> *list : {&backend->free_running, &backend->free_partial}) {
        for (const SumBuffer &buffer : *list) {
            if (buffer.memory) {
                cudaFree(buffer.memory);
            }
        }
        list->clear();
    }
    free_scratch(backend->augment_source);
    free_scratch(backend->augment_destination);
    free_scratch(backend->augment_table);
    free_scratch(backend->augment_means);
    if (backend->augment_host_table) {
        cudaFreeHost(backend->augment_host_table);
    }
    if (backend->augment_table_read) {
        cudaEventDestroy(backend->augment_table_read);
    }
    for (int i = 0; i < kStagingSlots; ++i) {
        if (backend->staging[i]) {
            cudaFreeHost(backend->staging[i]);
        }
        if (backend->staging_done[i]) {
            cudaEventDestroy(backend->staging_done[i]);
        }
    }
    if (backend->timer_begin) {
        cudaEventDestroy(backend->timer_begin);
    }
    if (backend->timer_end) {
        cudaEventDestroy(backend->timer_end);
    }
    if (backend->span_begin) {
        cudaEventDestroy(backend->span_begin);
    }
    if (backend->span_end) {
        cudaEventDestroy(backend->span_end);
    }
    for (cudaEvent_t event : backend->free_events) {
        cudaEventDestroy(event);
    }
    // Tensors that outlive the backend are copied back on the legacy default
    // stream from here on.
    coherence_set_stream(nullptr, nullptr);
    coherence_set_release_hook(nullptr);
    if (g_flush_backend == backend) {
        g_flush_backend = nullptr;
    }
    if (backend->stream) {
        cudaStreamDestroy(backend->stream);
    }
    delete backend;
}

extern "C" int cuda_backend_available(const CudaBackend *backend) {
    return backend && backend->stream ? 1 : 0;
}

extern "C" int cuda_backend_enable_device_execution(CudaBackend *backend) {
    if (!cuda_backend_available(backend)) {
        return -1;
    }
    backend->set_table = ops_set_device_backend;
    backend->set_allocator = tensor_set_allocator;
    if (!backend->set_table) {
        backend->set_table = reinterpret_cast<void (*)(const vitb200_op_table *)>(
            dlsym(RTLD_DEFAULT, "ops_set_device_backend"));
    }
    if (!backend->set_allocator) {
        backend->set_allocator = reinterpret_cast<void (*)(
            vitb200_allocate_fn, vitb200_release_fn, void *)>(
            dlsym(RTLD_DEFAULT, "tensor_set_allocator"));
    }
    if (!backend->set_table || !backend->set_allocator) {
        fprintf(stderr,
                "vitb200: host functions ops_set_device_backend / "
                "tensor_set_allocator not found in this process\n");
        return -1;
    }
    check(cudaSetDevice(backend->device), "cudaSetDevice");
    coherence_install_fault_handler();
    coherence_set_stream(backend->stream, flush_hook);
    coherence_set_release_hook(release_hook);
    g_flush_backend = backend;
    backend->table = make_table(backend);
    backend->set_table(&backend->table);
    backend->set_allocator(coherent_allocate, coherent_release, backend);
    backend->enabled = 1;
    return 0;
}

extern "C" void cuda_backend_disable_device_execution(CudaBackend *backend) {
    if (!backend || !backend->enabled) {
        return;
    }
    settle_timers(backend);
    // ops_set_device_backend synchronises the outgoing table first
    // (reference src/ops.c:66-74).
    backend->set_table(nullptr);
    backend->set_allocator(nullptr, nullptr, nullptr);
    backend->enabled = 0;
}

extern "C" void vitb200_zero_fill_counters(size_t *memsets, size_t *batched,
                                           size_t *prefetched_reads) {
    const CoherenceStats s = coherence_stats();
    if (memsets) *memsets = s.zero_fills_materialised;
    if (batched) *batched = s.zero_fills_batched;
    if (prefetched_reads) *prefetched_reads = s.prefetched_reads;
}

extern "C" unsigned long long vitb200_kernel_launches(void) {
    return g_kernel_launches;
}

extern "C" void vitb200_memory_counters(size_t *live_allocations,
                                        size_t *mirror_bytes,
                                        size_t *device_bytes,
                                        size_t *h2d_copies, size_t *h2d_bytes,
                                        size_t *d2h_copies, size_t *d2h_bytes,
                                        size_t *faults) {
    const CoherenceStats s = coherence_stats();
    if (live_allocations) *live_allocations = s.live_allocations;
    if (mirror_bytes) *mirror_bytes = s.mirror_bytes;
    if (device_bytes) *device_bytes = s.device_bytes;
    if (h2d_copies) *h2d_copies = s.host_to_device_copies;
    if (h2d_bytes) *h2d_bytes = s.host_to_device_bytes;
    if (d2h_copies) *d2h_copies = s.device_to_host_copies;
    if (d2h_bytes) *d2h_bytes = s.device_to_host_bytes;
    if (faults) *faults = s.faults_served;
}

extern "C" void vitb200_elision_counters(size_t *zero_fills_elided,
                                         size_t *zero_fills_materialised,
                                         size_t *lazy_defined,
                                         size_t *lazy_materialised,
                                         size_t *lazy_dropped) {
    const CoherenceStats s = coherence_stats();
    if (zero_fills_elided) *zero_fills_elided = s.zero_fills_elided;
    if (zero_fills_materialised) *zero_fills_materialised = s.zero_fills_materialised;
    if (lazy_defined) *lazy_defined = s.lazy_defined;
    if (lazy_materialised) *lazy_materialised = s.lazy_materialised;
    if (lazy_dropped) *lazy_dropped = s.lazy_dropped;
}

namespace {

static_assert(VITB200_GEMM_PARTIAL_ROWS == kGemmPartialRows,
              "the public header states the partial row count");
static_assert(sizeof(vitb200_augmentation) == sizeof(AugmentationSettings),
              "public and internal augmentation settings must match");

// Device view of an augmentation operand: tensor memory from our allocator is
// used where it is, anything else goes through a staging buffer.
const float *augment_input(CudaBackend *backend, const float *source,
                           size_t count) {
    if (coherent_owns(source)) {
        return view(backend, source, Access::Read);
    }
    float *staged = scratch<float>(backend, backend->augment_source, count);
    check(cudaMemcpyAsync(staged, source, count * sizeof(float),
                          cudaMemcpyHostToDevice, backend->stream),
          "cudaMemcpyAsync(host to device)");
    return staged;
}

float *augment_output(CudaBackend *backend, float *destination, size_t count,
                      bool *staged) {
    *staged = !coherent_owns(destination);
    if (!*staged) {
        return view(backend, destination, Access::Overwrite);
    }
    return scratch<float>(backend, backend->augment_destination, count);
}

// Copies a staged result back and waits, so that a plain host buffer holds it
// when the call returns.
void augment_finish(CudaBackend *backend, float *destination,
                    const float *device, size_t count, bool staged) {
    if (staged) {
        check(cudaMemcpyAsync(destination, device, count * sizeof(float),
                              cudaMemcpyDeviceToHost, backend->stream),
              "cudaMemcpyAsync(device to host)");
        check(cudaStreamSynchronize(backend->stream), "cudaStreamSynchronize");
    }
}

}  // namespace

extern "C" int vitb200_data_augmentation_enabled(
    const vitb200_augmentation *augmentation) {
    return augmentation &&
           augmentation_enabled(
               *reinterpret_cast<const AugmentationSettings *>(augmentation));
}

extern "C" int vitb200_data_augmentation_apply(
    CudaBackend *backend, const vitb200_augmentation *augmentation,
    uint64_t *random_state, const float *source, float *destination,
    size_t batch, size_t channels, size_t height, size_t width) {
    const AugmentationSettings *settings =
        reinterpret_cast<const AugmentationSettings *>(augmentation);
    if (!cuda_backend_available(backend) ||
        !augmentation_arguments_valid(settings, random_state, source,
                                      destination, batch, channels, height,
                                      width) ||
        !fits_int(height * width) || !fits_int(channels)) {
        return -1;
    }
    flush_pending(backend);
    // The per-sample table is written on the host into pinned memory that the
    // previous call's upload may still be reading.
    const size_t table_bytes = batch * sizeof(AugmentationSample);
    if (!backend->augment_table_read) {
        check(cudaEventCreateWithFlags(&backend->augment_table_read,
                                       cudaEventDisableTiming),
              "cudaEventCreate");
    } else {
        check(cudaEventSynchronize(backend->augment_table_read),
              "cudaEventSynchronize");
    }
    if (backend->augment_host_bytes < table_bytes) {
        if (backend->augment_host_table) {
            cudaFreeHost(backend->augment_host_table);
        }
        check(cudaHostAlloc(&backend->augment_host_table, table_bytes * 2,
                            cudaHostAllocDefault),
              "cudaHostAlloc");
        backend->augment_host_bytes = table_bytes * 2;
    }
    AugmentationSample *host_table =
        static_cast<AugmentationSample *>(backend->augment_host_table);
    augmentation_plan(*settings, random_state, batch, channels, height, width,
                      host_table);
    const size_t count = batch * channels * height * width;
    AugmentationSample *table = scratch<AugmentationSample>(
        backend, backend->augment_table, batch);
    float *means = scratch<float>(backend, backend->augment_means,
                                  batch * channels);
    check(cudaMemcpyAsync(table, host_table, table_bytes,
                          cudaMemcpyHostToDevice, backend->stream),
          "cudaMemcpyAsync(host to device)");
    check(cudaEventRecord(backend->augment_table_read, backend->stream),
          "cudaEventRecord");
    const float *in = nullptr;
    float *out = nullptr;
    bool staged = false;
    if (source == destination) {
        // In place (only without a geometric transform, checked above).
        if (coherent_owns(destination)) {
            out = view(backend, destination, Access::ReadWrite);
        } else {
            out = const_cast<float *>(augment_input(backend, source, count));
            staged = true;
        }
        in = out;
    } else {
        in = augment_input(backend, source, count);
        out = augment_output(backend, destination, count, &staged);
    }
    {
        OpScope scope(backend, "data_augmentation", 8.0 * double(count), 0.0);
        launch_augmentation(*settings, table, in, out, means, batch, channels,
                            height, width, backend->stream);
    }
    augment_finish(backend, destination, out, count, staged);
    return 0;
}

extern "C" int vitb200_data_augmentation_translate(
    CudaBackend *backend, const float *source, float *destination, size_t batch,
    size_t channels, size_t height, size_t width, float shift_y,
    float shift_x) {
    // Checks of the reference, src/augmentation.c:235-238.
    if (!cuda_backend_available(backend) || !source || !destination ||
        source == destination || batch == 0 || channels == 0 || height == 0 ||
        width == 0 || !fits_int(height * width) || !fits_int(channels)) {
        return -1;
    }
    flush_pending(backend);
    const size_t count = batch * channels * height * width;
    const float *in = augment_input(backend, source, count);
    bool staged = false;
    float *out = augment_output(backend, destination, count, &staged);
    {
        OpScope scope(backend, "data_augmentation", 8.0 * double(count), 0.0);
        launch_augmentation_translate(in, out, batch, channels, height, width,
                                      shift_y, shift_x, backend->stream);
    }
    augment_finish(backend, destination, out, count, staged);
    return 0;
}

// ------------------------------------------------------------ dataset

// Samples on the device as 8- or 16-bit integers, the order table next to
// them; labels and the order's master copy stay on the host, where the
// shuffle draws and the label upload happen.
struct vitb200_dataset {
    CudaBackend *backend = nullptr;
    size_t samples = 0, height = 0, width = 0;
    bool wide = false;
    void *pixels = nullptr;
    uint16_t *max_values = nullptr;
    uint32_t *order = nullptr;
    bool order_on_device = false;   // false: identity, or a shuffle not yet uploaded
    bool shuffled = false;
    std::vector<uint32_t> host_order;
    std::vector<size_t> labels;
    float mean = 0.0f, inverse_std = 1.0f;
    Scratch staging;
};

namespace {

int dataset_create(CudaBackend *backend, ParsedDataset &parsed,
                   vitb200_dataset **out) {
    vitb200_dataset *dataset = new vitb200_dataset();
    dataset->backend = backend;
    dataset->samples = parsed.samples();
    dataset->height = parsed.height;
    dataset->width = parsed.width;
    dataset_statistics(parsed, &dataset->mean, &dataset->inverse_std);
    for (uint16_t max_value : parsed.max_values) {
        dataset->wide = dataset->wide || max_value >= 256;
    }
    // A binary file may hold bytes above its own maximum; they still fit.
    const size_t count = parsed.pixels.size();
    check(cudaSetDevice(backend->device), "cudaSetDevice");
    if (dataset->wide) {
        check(cudaMalloc(&dataset->pixels, count * sizeof(uint16_t)), "cudaMalloc");
        check(cudaMemcpy(dataset->pixels, parsed.pixels.data(),
                         count * sizeof(uint16_t), cudaMemcpyHostToDevice),
              "cudaMemcpy");
    } else {
        std::vector<uint8_t> narrow(count);
        for (size_t i = 0; i < count; ++i) {
            narrow[i] = uint8_t(parsed.pixels[i]);
        }
        check(cudaMalloc(&dataset->pixels, count ? count : 1), "cudaMalloc");
        check(cudaMemcpy(dataset->pixels, narrow.data(), count,
                         cudaMemcpyHostToDevice),
              "cudaMemcpy");
    }
    check(cudaMalloc(&dataset->max_values, dataset->samples * sizeof(uint16_t)),
          "cudaMalloc");
    check(cudaMemcpy(dataset->max_values, parsed.max_values.data(),
                     dataset->samples * sizeof(uint16_t), cudaMemcpyHostToDevice),
          "cudaMemcpy");
    check(cudaMalloc(&dataset->order, dataset->samples * sizeof(uint32_t)),
          "cudaMalloc");
    dataset->host_order.resize(dataset->samples);
    for (size_t i = 0; i < dataset->samples; ++i) {
        dataset->host_order[i] = uint32_t(i);
    }
    dataset->labels.swap(parsed.labels);
    *out = dataset;
    return 0;
}

}  // namespace

extern "C" int vitb200_dataset_load_pgm_csv(CudaBackend *backend,
                                            const char *manifest_path,
                                            vitb200_dataset **dataset) {
    if (dataset) {
        *dataset = nullptr;
    }
    ParsedDataset parsed;
    if (!dataset || !cuda_backend_available(backend) ||
        dataset_parse_pgm_csv(manifest_path, &parsed) != 0 ||
        parsed.samples() > UINT_MAX) {
        return -1;
    }
    return dataset_create(backend, parsed, dataset);
}

extern "C" int vitb200_dataset_from_integers(
    CudaBackend *backend, const unsigned short *pixels,
    const unsigned short *max_values, const size_t *labels, size_t sample_count,
    size_t height, size_t width, vitb200_dataset **dataset) {
    if (dataset) {
        *dataset = nullptr;
    }
    if (!dataset || !cuda_backend_available(backend) || !pixels || !labels ||
        sample_count == 0 || height == 0 || width == 0 ||
        sample_count > UINT_MAX) {
        return -1;
    }
    ParsedDataset parsed;
    parsed.height = height;
    parsed.width = width;
    parsed.pixels.assign(pixels, pixels + sample_count * height * width);
    parsed.labels.assign(labels, labels + sample_count);
    parsed.max_values.assign(sample_count, uint16_t(255));
    for (size_t i = 0; max_values && i < sample_count; ++i) {
        if (max_values[i] == 0) {
            return -1;
        }
        parsed.max_values[i] = max_values[i];
    }
    return dataset_create(backend, parsed, dataset);
}

extern "C" void vitb200_dataset_free(vitb200_dataset *dataset) {
    if (!dataset) {
        return;
    }
    cudaStreamSynchronize(dataset->backend->stream);
    cudaFree(dataset->pixels);
    cudaFree(dataset->max_values);
    cudaFree(dataset->order);
    free_scratch(dataset->staging);
    delete dataset;
}

extern "C" size_t vitb200_dataset_sample_count(const vitb200_dataset *dataset) {
    return dataset ? dataset->samples : 0;
}

extern "C" size_t vitb200_dataset_height(const vitb200_dataset *dataset) {
    return dataset ? dataset->height : 0;
}

extern "C" size_t vitb200_dataset_width(const vitb200_dataset *dataset) {
    return dataset ? dataset->width : 0;
}

extern "C" size_t vitb200_dataset_channels(const vitb200_dataset *dataset) {
    return dataset ? 1 : 0;
}

extern "C" int vitb200_dataset_statistics(const vitb200_dataset *dataset,
                                          float *mean,
                                          float *inverse_standard_deviation) {
    if (!dataset || !mean || !inverse_standard_deviation) {
        return -1;
    }
    *mean = dataset->mean;
    *inverse_standard_deviation = dataset->inverse_std;
    return 0;
}

extern "C" int vitb200_dataset_shuffle(vitb200_dataset *dataset,
                                       unsigned long *state) {
    if (!dataset || !state) {
        return -1;
    }
    dataset_shuffle(dataset->host_order, state);
    dataset->shuffled = true;
    dataset->order_on_device = false;
    return 0;
}

extern "C" int vitb200_dataset_batch(vitb200_dataset *dataset, size_t offset,
                                     size_t batch, float mean,
                                     float inverse_standard_deviation,
                                     float *images, size_t *labels) {
    if (!dataset || !images || batch == 0 || offset > dataset->samples ||
        batch > dataset->samples - offset ||
        !cuda_backend_available(dataset->backend)) {
        return -1;
    }
    CudaBackend *backend = dataset->backend;
    flush_pending(backend);
    if (dataset->shuffled && !dataset->order_on_device) {
        // Pageable source: the copy is staged before the call returns, and it
        // is ordered behind the batches that still read the old table.
        check(cudaMemcpyAsync(dataset->order, dataset->host_order.data(),
                              dataset->samples * sizeof(uint32_t),
                              cudaMemcpyHostToDevice, backend->stream),
              "cudaMemcpyAsync(host to device)");
        dataset->order_on_device = true;
    }
    const size_t image_size = dataset->height * dataset->width;
    const size_t count = batch * image_size;
    const bool staged = !coherent_owns(images);
    float *out = staged ? scratch<float>(backend, dataset->staging, count)
                        : view(backend, images, Access::Overwrite);
    {
        OpScope scope(backend, "dataset_batch",
                      double(count) * (4.0 + (dataset->wide ? 2.0 : 1.0)), 0.0);
        launch_dataset_batch(dataset->pixels, dataset->wide, dataset->max_values,
                             dataset->shuffled ? dataset->order : nullptr,
                             offset, batch, image_size, mean,
                             inverse_standard_deviation, out, backend->stream);
    }
    if (staged) {
        check(cudaMemcpyAsync(images, out, count * sizeof(float),
                              cudaMemcpyDeviceToHost, backend->stream),
              "cudaMemcpyAsync(device to host)");
        check(cudaStreamSynchronize(backend->stream), "cudaStreamSynchronize");
    }
    for (size_t i = 0; labels && i < batch; ++i) {
        labels[i] = dataset->labels[dataset->host_order[offset + i]];
    }
    return 0;
}

extern "C" int vitb200_dataset_parse_pgm_csv(
    const char *manifest_path, unsigned short **pixels,
    unsigned short **max_values, size_t **labels, size_t *sample_count,
    size_t *height, size_t *width) {
    ParsedDataset parsed;
    if (!pixels || !max_values || !labels || !sample_count || !height ||
        !width || dataset_parse_pgm_csv(manifest_path, &parsed) != 0) {
        return -1;
    }
    *pixels = static_cast<unsigned short *>(
        malloc(parsed.pixels.size() * sizeof(unsigned short)));
    *max_values = static_cast<unsigned short *>(
        malloc(parsed.samples() * sizeof(unsigned short)));
    *labels = static_cast<size_t *>(malloc(parsed.samples() * sizeof(size_t)));
    if (!*pixels || !*max_values || !*labels) {
        free(*pixels);
        free(*max_values);
        free(*labels);
        return -1;
    }
    memcpy(*pixels, parsed.pixels.data(),
           parsed.pixels.size() * sizeof(unsigned short));
    memcpy(*max_values, parsed.max_values.data(),
           parsed.samples() * sizeof(unsigned short));
    memcpy(*labels, parsed.labels.data(), parsed.samples() * sizeof(size_t));
    *sample_count = parsed.samples();
    *height = parsed.height;
    *width = parsed.width;
    return 0;
}

extern "C" int vitb200_dataset_pixel_statistics(
    const unsigned short *pixels, const unsigned short *max_values,
    size_t sample_count, size_t image_size, float *mean,
    float *inverse_standard_deviation) {
    if (!pixels || !mean || !inverse_standard_deviation || sample_count == 0 ||
        image_size == 0) {
        return -1;
    }
    ParsedDataset parsed;
    parsed.height = image_size;
    parsed.width = 1;
    parsed.pixels.assign(pixels, pixels + sample_count * image_size);
    parsed.labels.assign(sample_count, 0);
    parsed.max_values.assign(sample_count, uint16_t(255));
    for (size_t i = 0; max_values && i < sample_count; ++i) {
        parsed.max_values[i] = max_values[i];
    }
    dataset_statistics(parsed, mean, inverse_standard_deviation);
    return 0;
}

extern "C" void vitb200_dataset_shuffle_order(unsigned int *order, size_t count,
                                              unsigned long *state) {
    if (!order || !state) {
        return;
    }
    std::vector<uint32_t> table(order, order + count);
    dataset_shuffle(table, state);
    memcpy(order, table.data(), count * sizeof(uint32_t));
}

extern "C" void vitb200_fusion_counters(const CudaBackend *backend,
                                        unsigned long long *epilogues,
                                        unsigned long long *head_layouts,
                                        unsigned long long *bias_gradients) {
    if (epilogues) *epilogues = backend ? backend->fused_epilogues : 0;
    if (head_layouts) *head_layouts = backend ? backend->fused_head_layouts : 0;
    if (bias_gradients) *bias_gradients = backend ? backend->memo_hits : 0;
}

extern "C" unsigned long long vitb200_declined_ops(const CudaBackend *backend) {
    return backend ? backend->declined_ops : 0;
}

extern "C" void vitb200_kernel_path_counters(
    const CudaBackend *backend, unsigned long long *tensor_core_products,
    unsigned long long *wide_tile_products, unsigned long long *fma_products,
    unsigned long long *tensor_core_attention,
    unsigned long long *streaming_attention) {
    unsigned long long tc = 0, wide = 0, fma = 0;
    gemm_path_counters(&tc, &wide, &fma);
    if (tensor_core_products) *tensor_core_products = tc;
    if (wide_tile_products) *wide_tile_products = wide;
    if (fma_products) *fma_products = fma;
    if (tensor_core_attention) {
        *tensor_core_attention = backend ? backend->tc_attention_launches : 0;
    }
    if (streaming_attention) {
        *streaming_attention = backend ? backend->streaming_attention_launches : 0;
    }
}

static CheckpointCounters g_last_checkpoint = {};

extern "C" int vitb200_checkpoint_save(CudaBackend *backend, const char *path,
                                       const void *config, size_t config_bytes,
                                       vitb200_parameter *const *parameters,
                                       size_t count) {
    if (!cuda_backend_available(backend)) {
        return -1;
    }
    flush_pending(backend);
    g_last_checkpoint = CheckpointCounters{};
    return checkpoint_save(path, config, config_bytes, parameters, count,
                           backend->stream, &g_last_checkpoint);
}

extern "C" int vitb200_checkpoint_load(CudaBackend *backend, const char *path,
                                       const void *config, size_t config_bytes,
                                       vitb200_parameter *const *parameters,
                                       size_t count) {
    if (!cuda_backend_available(backend)) {
        return -1;
    }
    flush_pending(backend);
    settle_timers(backend);
    return checkpoint_load(path, config, config_bytes, parameters, count,
                           backend->stream);
}

extern "C" void vitb200_checkpoint_counters(size_t *bytes_from_device,
                                            size_t *bytes_from_host_memory) {
    if (bytes_from_device) *bytes_from_device = g_last_checkpoint.from_device;
    if (bytes_from_host_memory) *bytes_from_host_memory = g_last_checkpoint.from_mirrors;
}

extern "C" int vitb200_make_host_coherent(const void *tensor_memory) {
    return coherent_make_host_owned(tensor_memory);
}

extern "C" int vitb200_timer_begin(CudaBackend *backend) {
    if (!cuda_backend_available(backend)) {
        return -1;
    }
    return cudaEventRecord(backend->timer_begin, backend->stream) == cudaSuccess
        ? 0 : -1;
}

extern "C" float vitb200_timer_end(CudaBackend *backend) {
    if (!cuda_backend_available(backend) ||
        cudaEventRecord(backend->timer_end, backend->stream) != cudaSuccess ||
        cudaEventSynchronize(backend->timer_end) != cudaSuccess) {
        return -1.0f;
    }
    float ms = -1.0f;
    cudaEventElapsedTime(&ms, backend->timer_begin, backend->timer_end);
    return ms;
}

extern "C" int vitb200_dp_unique_id(void *out128) {
    return dp_unique_id(out128);
}

extern "C" int vitb200_dp_init(CudaBackend *backend, int rank, int world,
                               const void *id128) {
    if (!cuda_backend_available(backend) || backend->dp) {
        return -1;
    }
    check(cudaSetDevice(backend->device), "cudaSetDevice");
    backend->dp = dp_create(rank, world, id128, backend->stream);
    return backend->dp ? 0 : -1;
}

extern "C" void vitb200_dp_shutdown(CudaBackend *backend) {
    if (backend && backend->dp) {
        settle_timers(backend);
        dp_destroy(backend->dp);
        backend->dp = nullptr;
    }
}

extern "C" void vitb200_dp_counters(CudaBackend *backend,
                                    unsigned long long *all_reduce_calls,
                                    unsigned long long *overlapped_tensors,
                                    unsigned long long *late_tensors,
                                    unsigned long long *bytes) {
    dp_counters(backend ? backend->dp : nullptr, all_reduce_calls,
                overlapped_tensors, late_tensors, bytes);
}

extern "C" int vitb200_dp_status(CudaBackend *backend) {
    return dp_status(backend ? backend->dp : nullptr);
}

extern "C" unsigned long long vitb200_dp_flat_ranges(CudaBackend *backend) {
    return dp_flat_ranges(backend ? backend->dp : nullptr);
}

extern "C" int vitb200_set_gradient_accumulation(CudaBackend *backend,
                                                 int micro_batches) {
    if (!cuda_backend_available(backend) || micro_batches < 1) {
        return -1;
    }
    const float inverse = 1.0f / float(micro_batches);
    if (inverse != backend->accumulation_inverse) {
        backend->accumulation_inverse = inverse;
        dp_forget_schedule(backend->dp);
    }
    return 0;
}

extern "C" void vitb200_set_gemm_precision(int precision) {
    gemm_set_default_precision(precision);
}

extern "C" int vitb200_tensor_core_status(void) {
    return gemm_tc_status();
}

extern "C" double vitb200_device_busy_ms(CudaBackend *backend, int reset) {
    if (!cuda_backend_available(backend)) {
        return -1.0;
    }
    settle_timers(backend);
    const double ms = backend->busy_ms;
    if (reset) {
        backend->busy_ms = 0.0;
    }
    return ms;
}

int poll_exchange() {
    CudaBackend *backend = g_flush_backend;
    return backend && backend->dp && dp_world(backend->dp) > 1
               ? dp_poll(backend->dp) : 0;
}

extern "C" int vitb200_set_deferred_synchronize(CudaBackend *backend, int on) {
    if (!cuda_backend_available(backend)) {
        return -1;
    }
    settle_timers(backend);
    const int before = backend->deferred_synchronize ? 1 : 0;
    backend->deferred_synchronize = on != 0;
    coherent_set_wait_poll(on ? poll_exchange : nullptr);
    coherent_set_overlapped_uploads(on != 0);
    return before;
}

extern "C" void vitb200_profile_enable(CudaBackend *backend, int on) {
    if (!cuda_backend_available(backend)) {
        return;
    }
    settle_timers(backend);
    backend->profiling = on != 0;
    if (on) {
        backend->op_stats.clear();
    }
}

extern "C" size_t vitb200_profile_entries(CudaBackend *backend) {
    if (!cuda_backend_available(backend)) {
        return 0;
    }
    settle_timers(backend);
    return backend->op_stats.size();
}

extern "C" int vitb200_profile_entry(CudaBackend *backend, size_t index,
                                     const char **name,
                                     unsigned long long *calls,
                                     double *milliseconds, double *bytes,
                                     double *flops) {
    if (!cuda_backend_available(backend) || index >= backend->op_stats.size()) {
        return -1;
    }
    const OpStat &stat = backend->op_stats[index];
    if (name) *name = stat.name;
    if (calls) *calls = stat.calls;
    if (milliseconds) *milliseconds = stat.ms;
    if (bytes) *bytes = stat.bytes;
    if (flops) *flops = stat.flops;
    return 0;
}

// ------------------------------------------------------------------ part 2

extern "C" int vitb200_k_gemm(const float *x, const float *w, float *y,
                              size_t m, size_t k, size_t n, int precision,
                              void *stream) {
    if (!fits_int(m) || !fits_int(k) || !fits_int(n)) {
        return -1;
    }
    return gemm_forward(x, w, y, int(m), int(k), int(n), precision,
                        as_stream(stream));
}

extern "C" int vitb200_k_gemm_fused(const float *x, const float *w, float *y,
                                    const float *bias, float *gelu_out,
                                    const float *residual, float *residual_out,
                                    size_t m, size_t k, size_t n, int precision,
                                    void *stream) {
    if (!fits_int(m) || !fits_int(k) || !fits_int(n) ||
        (gelu_out && residual_out) || (!residual != !residual_out)) {
        return -1;
    }
    GemmEpilogue epilogue;
    epilogue.bias = bias;
    epilogue.gelu_out = gelu_out;
    epilogue.residual = residual;
    epilogue.residual_out = residual_out;
    return gemm_forward_fused(x, w, y, int(m), int(k), int(n), epilogue,
                              precision, as_stream(stream));
}

extern "C" int vitb200_k_gemm_backward(const float *x, const float *w,
                                       const float *dy, float *dx, float *dw,
                                       size_t m, size_t k, size_t n,
                                       int precision, void *stream) {
    if (!fits_int(m) || !fits_int(k) || !fits_int(n)) {
        return -1;
    }
    return gemm_backward(x, w, dy, dx, dw, int(m), int(k), int(n), precision,
                         true, as_stream(stream));
}

extern "C" int vitb200_k_gemm_backward_gelu(const float *w, const float *dy,
                                            const float *gelu_input,
                                            float *d_gelu_input,
                                            float *column_partials, size_t m,
                                            size_t k, size_t n, int precision,
                                            void *stream) {
    if (!fits_int(m) || !fits_int(k) || !fits_int(n)) {
        return -1;
    }
    return gemm_backward_input_gelu(w, dy, gelu_input, d_gelu_input,
                                    column_partials, int(m), int(k), int(n),
                                    precision, as_stream(stream));
}

extern "C" int vitb200_k_bias_add(const float *in, const float *bias,
                                  float *out, size_t rows, size_t cols,
                                  void *stream) {
    launch_bias_add(in, bias, out, rows, cols, as_stream(stream));
    return 0;
}

extern "C" int vitb200_k_column_sums(const float *in, float *out, size_t rows,
                                     size_t cols, void *stream) {
    launch_column_sums(in, out, rows, cols, cols, as_stream(stream));
    return 0;
}

extern "C" int vitb200_k_layer_norm(const float *x, const float *gamma,
                                    const float *beta, float epsilon, float *y,
                                    size_t rows, size_t cols, void *stream) {
    launch_layer_norm(x, gamma, beta, epsilon, y, rows, cols,
                      as_stream(stream));
    return 0;
}

extern "C" int vitb200_k_layer_norm_backward(const float *x, const float *gamma,
                                             float epsilon, const float *dy,
                                             float *dx, float *dgamma,
                                             float *dbeta, size_t rows,
                                             size_t cols, void *stream) {
    launch_layer_norm_backward(x, gamma, epsilon, dy, dx, dgamma, dbeta, rows,
                               cols, dx, nullptr, as_stream(stream));
    return 0;
}

extern "C" int vitb200_k_gelu(const float *in, float *out, size_t n,
                              void *stream) {
    launch_gelu(in, out, n, as_stream(stream));
    return 0;
}

extern "C" int vitb200_k_gelu_backward(const float *x, const float *dy,
                                       float *dx, size_t n, void *stream) {
    launch_gelu_backward(x, dy, dx, n, true, as_stream(stream));
    return 0;
}

extern "C" int vitb200_k_attention(const float *q, const float *k,
                                   const float *v, float *probabilities,
                                   float *out, size_t groups, size_t seq,
                                   size_t head_dim, float scale, int precision,
                                   void *stream) {
    if (head_dim > kMaxHeadDim || !fits_int(seq) || !fits_int(groups)) {
        return -1;
    }
    if (!probabilities) {
        // P is not wanted: the whole-group kernels that keep it on chip.
        const double work = double(groups) * seq * seq * head_dim;
        if (precision != VITB200_PRECISION_FP32 &&
            attention_warp_supported(seq, head_dim) &&
            prefer_tensor_cores(precision, work)) {
            return launch_attention_warp_forward(q, k, v, out, groups, seq,
                                                 head_dim, scale,
                                                 as_stream(stream)) ? 0 : -1;
        }
        if (precision != VITB200_PRECISION_TF32 &&
            attention_small_supported(seq, head_dim)) {
            return launch_attention_small_forward(q, k, v, nullptr, out, groups,
                                                  seq, head_dim, scale, false,
                                                  true, as_stream(stream)) ? 0 : -1;
        }
        return -1;
    }
    if (precision == VITB200_PRECISION_TF32 &&
        !attention_mma_supported(head_dim)) {
        return -1;
    }
    launch_attention_forward(q, k, v, probabilities, out, groups, seq, head_dim,
                             scale, precision, as_stream(stream));
    return 0;
}

extern "C" int vitb200_k_attention_stream(const float *q, const float *k,
                                          const float *v, float *out,
                                          float *lse, size_t groups, size_t seq,
                                          size_t head_dim, float scale,
                                          void *stream) {
    if (!fits_int(seq) || !fits_int(groups)) {
        return -1;
    }
    return launch_attention_stream_forward(q, k, v, out, lse, groups, seq,
                                           head_dim, scale, as_stream(stream))
        ? 0 : -1;
}

extern "C" int vitb200_k_attention_stream_backward(
    const float *q, const float *k, const float *v, const float *out,
    const float *dout, const float *lse, float *dq, float *dk, float *dv,
    float *row_dots, size_t groups, size_t seq, size_t head_dim, float scale,
    void *stream) {
    if (!fits_int(seq) || !fits_int(groups)) {
        return -1;
    }
    return launch_attention_stream_backward(q, k, v, out, dout, lse, dq, dk, dv,
                                            row_dots, groups, seq, head_dim,
                                            scale, true, true, true,
                                            as_stream(stream))
        ? 0 : -1;
}

// ld == 0: head-major tensors ([groups*seq, head_dim]).  Otherwise every
// operand is a block of `heads * head_dim` columns inside a token-major matrix
// whose rows are `ld` floats apart (the pointers name the first column), as
// the Q, K, V blocks of the projection and the merged attention output are.
static HeadLayout abi_layout(size_t ld, size_t heads) {
    HeadLayout layout;
    if (ld != 0) {
        layout.ld = int(ld);
        layout.heads = int(heads);
    }
    return layout;
}

extern "C" int vitb200_k_attention_tc(const float *q, const float *k,
                                      const float *v, float *out, float *lse,
                                      size_t groups, size_t seq, size_t head_dim,
                                      float scale, size_t in_ld, size_t out_ld,
                                      size_t heads, void *stream) {
    if (!fits_int(seq) || !fits_int(groups) || !fits_int(heads) ||
        in_ld > size_t(INT_MAX) || out_ld > size_t(INT_MAX)) {
        return -1;
    }
    return launch_attention_tc_forward(q, k, v, out, lse, groups, seq, head_dim,
                                       scale, as_stream(stream),
                                       abi_layout(in_ld, heads),
                                       abi_layout(out_ld, heads))
        ? 0 : -1;
}

extern "C" int vitb200_k_attention_tc_backward(
    const float *q, const float *k, const float *v, const float *out,
    const float *dout, const float *lse, float *dq, float *dk, float *dv,
    float *row_dots, size_t groups, size_t seq, size_t head_dim, float scale,
    int accumulate, size_t in_ld, size_t out_ld, size_t grad_ld, size_t heads,
    void *stream) {
    if (!fits_int(seq) || !fits_int(groups) || !fits_int(heads) ||
        in_ld > size_t(INT_MAX) || out_ld > size_t(INT_MAX) ||
        grad_ld > size_t(INT_MAX)) {
        return -1;
    }
    const bool add = accumulate != 0;
    return launch_attention_tc_backward(
               q, k, v, out, dout, lse, dq, dk, dv, row_dots, groups, seq,
               head_dim, scale, add, add, add, as_stream(stream),
               abi_layout(in_ld, heads), abi_layout(out_ld, heads),
               abi_layout(out_ld, heads), abi_layout(grad_ld, heads))
        ? 0 : -1;
}

extern "C" int vitb200_k_attention_backward(
    const float *q, const float *k, const float *v, const float *probabilities,
    const float *out, const float *dout, float *dq, float *dk, float *dv,
    float *row_dots, size_t groups, size_t seq, size_t head_dim, float scale,
    int precision, void *stream) {
    if (head_dim > kMaxHeadDim || !fits_int(seq) || !fits_int(groups)) {
        return -1;
    }
    if (!probabilities) {
        const double work = double(groups) * seq * seq * head_dim;
        if (precision != VITB200_PRECISION_FP32 &&
            attention_warp_supported(seq, head_dim) &&
            prefer_tensor_cores(precision, work)) {
            return launch_attention_warp_backward(
                       q, k, v, out, dout, dq, dk, dv, groups, seq, head_dim,
                       scale, true, true, true, as_stream(stream)) ? 0 : -1;
        }
        if (precision != VITB200_PRECISION_TF32 &&
            attention_small_supported(seq, head_dim)) {
            return launch_attention_small_backward(
                       q, k, v, nullptr, out, dout, dq, dk, dv, groups, seq,
                       head_dim, scale, true, true, true, true,
                       as_stream(stream)) ? 0 : -1;
        }
        return -1;
    }
    launch_attention_backward(q, k, v, probabilities, out, dout, dq, dk, dv,
                              row_dots, groups, seq, head_dim, scale, true,
                              true, true, precision, as_stream(stream));
    return 0;
}

extern "C" int vitb200_k_softmax_cross_entropy(
    const float *logits, const float *targets, const float *class_weights,
    float label_smoothing, float *loss, float *logits_grad, float *row_losses,
    size_t rows, size_t cols, void *stream) {
    launch_softmax_cross_entropy(logits, targets, class_weights,
                                 label_smoothing, loss, logits_grad, row_losses,
                                 rows, cols, as_stream(stream));
    return 0;
}

extern "C" int vitb200_attention_tile_index(int head_dim, int row, int col) {
    return row < 0 || row >= 64 || col < 0 || col >= head_dim
        ? -1 : attention_tile_index(head_dim, row, col);
}

extern "C" int vitb200_attention_lane_column(int head_dim, int t, int e) {
    return t < 0 || t >= 4 || e < 0 || e >= head_dim / 4
        ? -1 : attention_lane_column(head_dim, t, e);
}

extern "C" int vitb200_k_softmax_cross_entropy_static(
    const float *logits, const float *targets, const float *class_weights,
    float label_smoothing, float *loss, float *logits_grad, size_t rows,
    size_t cols, void *stream) {
    return launch_softmax_cross_entropy_static(logits, targets, class_weights,
                                               label_smoothing, loss,
                                               logits_grad, rows, cols,
                                               as_stream(stream));
}
