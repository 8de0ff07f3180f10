// Host-visible tensor memory backed by explicit device allocations.
//
// The host program dereferences tensor memory directly (weight initialisation,
// input upload, loss read-back, CPU fallbacks, gradient checks), while every
// kernel works on plain cudaMalloc'd buffers.  Each allocation handed to the
// host is an anonymous private mapping (the "mirror"); a device buffer of the
// same size is created the first time a kernel needs it.  Exactly one side is
// authoritative at a time and page protection on the mirror tells us when the
// host touches a mirror whose current contents live on the device:
//
//   HOST    mirror read+write, device copy stale or absent
//   SHARED  mirror read-only, both copies identical
//   DEVICE  mirror inaccessible, device copy authoritative
//
// A host access that the protection forbids raises SIGSEGV; the handler drains
// the stream, copies the allocation back if needed, relaxes the protection and
// returns, so the faulting instruction simply re-executes.  In steady-state
// training only the images, the labels and the four loss bytes ever move.
#pragma once

#include <cstddef>
#include <cuda_runtime.h>

namespace vitb200 {

enum class Access { Read, ReadWrite, Overwrite };

struct CoherenceStats {
    size_t live_allocations;
    size_t mirror_bytes;
    size_t device_bytes;
    size_t host_to_device_copies;
    size_t host_to_device_bytes;
    size_t device_to_host_copies;
    size_t device_to_host_bytes;
    size_t faults_served;
    size_t zero_fills_elided;
    size_t zero_fills_materialised;
    size_t zero_fills_batched;   // materialised for free after a batched fill
    size_t prefetched_reads;     // host reads served from a prefetched copy
    size_t lazy_defined;
    size_t lazy_materialised;
    size_t lazy_dropped;
    size_t alias_reads;
    size_t sources_copied;   // in-place updates moved to a copy (readers pending)
};

// Allocator pair installed through tensor_set_allocator
// (reference src/autodiff.c:11-17).  Both ignore `context`: tensors may be
// released after the backend object that was current at allocation time has
// been destroyed (reference examples/organ_smnist.c:996-997).
void *coherent_allocate(void *context, size_t bytes);
void coherent_release(void *context, void *memory);

// True when `host_pointer` is the base address of a live mirror.
bool coherent_owns(const void *host_pointer);

// Device pointer for a mirror base address, after making the device copy valid
// for `access` on `stream`.  Returns nullptr for memory we did not allocate.
float *device_view(const void *host_pointer, Access access, cudaStream_t stream);

// Declares the buffer to be all zeros without touching memory ("zero
// pending").  The fill is materialised only if somebody reads the buffer
// before overwriting it; an accumulating kernel that asks through
// device_view_accumulate is told to store instead of add.  Returns false for
// memory we did not allocate.
bool coherent_mark_zero(const void *host_pointer, cudaStream_t stream);

// One kernel launch that writes the zeros of every listed buffer whose
// contents are a pending zero fill, which already has device memory and which
// holds at most `max_bytes`.  The fills stay pending (a kernel that overwrites
// the buffer still skips the read), but materialising one later is free.  For
// the many small gradients that are accumulated into: one launch per step
// instead of one memset node in front of every accumulating kernel.  Returns
// the number of buffers cleared.
size_t coherent_zero_fill_batch(const void *const *host_pointers, size_t count,
                                size_t max_bytes, cudaStream_t stream);

// Device pointer for a buffer the caller is about to add into.  *was_zero is
// set when the buffer's current contents are a pending zero fill, in which
// case the caller must overwrite every element (value = 0 + increment) and the
// pending fill is dropped.
float *device_view_accumulate(const void *host_pointer, cudaStream_t stream,
                              bool *was_zero);

// Lazily defined buffers.  `output` is declared to hold function(sources)
// without computing it.  The value is produced (by calling `function` on the
// stream) the first time anybody, device op or host, reads the buffer, and is
// never produced if the buffer is overwritten first.  Sources stay readable:
// if one is about to be overwritten while definitions are pending, its old
// device buffer is handed to them and the source continues in a fresh one, so
// no copy is made either way.  Any number of definitions may read one source;
// a source must itself hold computed values on the device.
typedef void (*LazyMaterialise)(const void *arguments, float *output,
                                float *const *sources, cudaStream_t stream);
bool coherent_define_lazy(const void *output_host,
                          const void *const *source_hosts, int sources,
                          LazyMaterialise function, const void *arguments,
                          size_t argument_bytes, cudaStream_t stream);
bool coherent_is_lazy(const void *host_pointer);
// Declares `output` to be a copy of `source` (same size) without copying.
// Readers (Access::Read) of the output are handed the source's buffer; the
// copy is made only if the output is modified in place or read by the host.
bool coherent_define_alias(const void *output_host, const void *source_host,
                           cudaStream_t stream);
// For an update output = output + increment written as a three-operand
// kernel: returns the buffer to write and sets *base to the buffer holding the
// current contents (the same pointer, an alias's source, or nullptr when the
// contents are a pending zero fill).  Every element must be written.
float *device_view_accumulate_based(const void *host_pointer,
                                    cudaStream_t stream, const float **base);
// For an output pending under `function` with one source: copies the
// definition's arguments out and returns the device pointer that currently
// holds the source's values, so that a consumer can read through the
// definition instead of having it computed.  The pointer is valid for work
// enqueued on the stream before the next call into this layer.  *source_host
// is the source's host address, or nullptr when the source has moved on and
// the definition reads a kept copy of its old contents.
bool coherent_lazy_source(const void *output_host, LazyMaterialise function,
                          void *arguments, size_t argument_bytes,
                          const float **source, const void **source_host);
// The buffer whose values `host_pointer` currently stands for: itself, or the
// source when it is an alias.  nullptr for an alias whose source has moved on
// (the alias then reads a kept copy that has no address of its own).
const void *coherent_alias_root(const void *host_pointer);
// Starts copying the buffer's device contents (as of everything enqueued on
// `stream` so far) to page-locked staging memory on a stream of its own.  A
// host read that follows waits for that copy only, not for the work enqueued
// after this call; a device write to the buffer in between cancels it.  For
// buffers of at most 4096 bytes that the device owns; false otherwise.
bool coherent_prefetch_host(const void *host_pointer, cudaStream_t stream);
// Called every ~1000 spins while a host access waits for the device; a
// non-zero answer ends the spinning (the wait then blocks in the driver).
void coherent_set_wait_poll(int (*poll)(void));
// Uploads of large page-locked inputs that are rewritten again and again (the
// image batch) go through a copy stream and a second device buffer from now
// on, so that they overlap whatever the compute stream is still busy with.
void coherent_set_overlapped_uploads(bool on);
// True while the buffer is a pending zero fill (see coherent_mark_zero).
bool coherent_is_zero_pending(const void *host_pointer);

// Makes the mirror readable and writable by the host again (copying back if
// the device holds the current contents).  Needed before handing a mirror to a
// system call such as fread/fwrite, which reports EFAULT instead of faulting.
int coherent_make_host_owned(const void *host_pointer);

// Makes every mirror that overlaps [pointer, pointer + bytes) valid for a
// host-side read (host_writes = false) or read-write access that cannot take
// a page fault, i.e. a system call.  Returns the number of mirrors touched; 0
// for memory we did not allocate (decided without looking at the registry, so
// this may be called from any thread for foreign memory).
int coherent_prepare_host_io(const void *pointer, size_t bytes,
                             bool host_writes);

// Where the current contents of a mirror can be read without changing who
// owns them: the device buffer (pending zero fills and definitions are
// computed first, on `stream`), or nullptr when the mirror itself is current
// (or the memory is not ours).  The pointer is valid for work enqueued on the
// stream before the next call into this layer.
const float *coherent_current_device(const void *host_pointer,
                                     cudaStream_t stream);

// Device memory owned by the caller in which buffers may be placed
// (coherent_place_device_buffer): this layer never pools or frees it.
// add = false withdraws a range registered earlier (by its base address).
void coherent_external_range(const void *base, size_t bytes, bool add);
// Bytes a device buffer for this mirror occupies (the page-rounded size of the
// allocation); 0 for memory we did not allocate.
size_t coherent_device_bytes(const void *host_pointer);
// Moves a mirror's device buffer to `device` (inside a registered external
// range, coherent_device_bytes() large), carrying current device contents
// along on `stream`; the old buffer is recycled.  device = nullptr moves a
// buffer that lives in external memory back into memory of this layer's own.
// False (nothing changed) for memory we did not allocate and for buffers that
// are lazily defined or read by pending definitions.
bool coherent_place_device_buffer(const void *host_pointer, float *device,
                                  cudaStream_t stream);

// Called by the backend so the fault handler can drain work before copying.
void coherence_set_stream(cudaStream_t stream, void (*flush)(void));
// Called with the host address of every allocation that is released, so that
// the backend can drop what it keeps per tensor.
void coherence_set_release_hook(void (*released)(const void *));
void coherence_install_fault_handler();
CoherenceStats coherence_stats();

}  // namespace vitb200
