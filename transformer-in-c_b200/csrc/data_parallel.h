// Data-parallel gradient exchange: one process per GPU, batch sharded by
// sample, parameters replicated, one sum-all-reduce of every parameter gradient
// per step (NCCL over NVLink / NVSwitch), overlapped with the backward pass.
//
// The host program is unaware of it.  It keeps calling the op table; the
// backend learns which gradient buffers belong to parameters from the
// optimiser call (`adamw_step_parameters` lists them) and counts the ops that
// write each one between two optimiser calls (one per micro-batch); once that
// count has repeated it starts reducing a gradient as soon as the last op that
// adds to it has been enqueued:
//
//   compute stream   ... dW GEMM | record event ........ | wait comm | clip + AdamW
//   comm stream                  | wait event, all-reduce bucket ... |
//
// Gradients are summed; the 1/world factor is folded into the clip scale the
// optimiser kernel already multiplies by, so no extra pass touches them.
//
// The first optimiser call learns the parameter list, the second the order in
// which the gradients become complete; their device buffers then move, in
// that order, into one allocation, and from the third step on contiguous
// ranges of it (at least 4 MiB, the last one whatever is left) are
// all-reduced as soon as their last gradient is complete: a handful of NCCL
// calls per step, the final one issued when the last weight gradient of the
// backward pass has been enqueued.  VITB200_DP_FLAT=0 keeps the per-tensor
// exchange of the first two steps for good.
// NCCL is loaded with dlopen when data parallelism is switched on, so single
// GPU users need no NCCL at all.
#pragma once

#include <cstddef>
#include <cuda_runtime.h>

namespace vitb200 {

struct DataParallel;

// Fills 128 bytes with a fresh NCCL unique id (rank 0 calls this and sends the
// bytes to the other ranks by any means).  0 on success.
int dp_unique_id(void *out128);

// Collective over all ranks.  Returns nullptr on failure.
DataParallel *dp_create(int rank, int world, const void *id128,
                        cudaStream_t compute_stream);
void dp_destroy(DataParallel *dp);
int dp_world(const DataParallel *dp);

// Asks NCCL whether the communicator has failed asynchronously (a peer died,
// a transport error).  On the first error the communicator is aborted, which
// ends its kernels, and the error code is kept: dp_status() returns it from
// then on and the optimiser slot declines.  Cheap; called at every
// synchronise.  Returns the kept code (0 = healthy).
int dp_poll(DataParallel *dp);
int dp_status(const DataParallel *dp);

// Called after the op that wrote `device_grad` (the gradient whose host mirror
// is `host_grad`, `count` floats) has been enqueued on the compute stream.
// Does nothing for buffers that are not known parameter gradients.
void dp_gradient_produced(DataParallel *dp, const void *host_grad,
                          float *device_grad, size_t count);

// Called by ops that add into a gradient buffer without being one of the
// counted producers above (residual_backward, accumulate_gradient,
// gather_rows_backward, gelu_backward).  Does nothing for buffers that are not
// known parameter gradients (this model's never are).  A parameter gradient
// written this way is from then on exchanged at the optimiser call, when all
// its writers are certain to have run; if its exchange had already started
// the process is stopped, because the sum on the wire lacks this write.
void dp_gradient_touched(DataParallel *dp, const void *host_grad);

// Called by the optimiser slot with the full parameter list, before the norm
// and update kernels are enqueued: reduces whatever has not been reduced yet,
// makes the compute stream wait for the exchange, and remembers the list for
// the next step.  Returns 1/world.
float dp_before_optimizer(DataParallel *dp, const void *const *host_grads,
                          float *const *device_grads, const size_t *counts,
                          size_t parameters);

// Forgets how many ops write each gradient per step; the next two steps are
// exchanged at the optimiser call while the counts are learnt again.  To be
// called when the number of micro-batches per optimiser step changes.
void dp_forget_schedule(DataParallel *dp);

// A tensor is about to be released: if it is one of the known parameter
// gradients, the schedule (and the arena the gradients were moved into) is
// dropped and learnt again from the next optimiser call on.
void dp_tensor_released(DataParallel *dp, const void *host_pointer);

// Counters for tests and the bench line.
void dp_counters(const DataParallel *dp, unsigned long long *all_reduce_calls,
                 unsigned long long *overlapped_tensors,
                 unsigned long long *late_tensors, unsigned long long *bytes);

// Contiguous ranges all-reduced out of the gradient arena so far.
unsigned long long dp_flat_ranges(const DataParallel *dp);

}  // namespace vitb200
