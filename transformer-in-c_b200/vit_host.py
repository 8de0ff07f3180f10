"""ctypes bindings for driving the ViT host code with the B200 backend.

Two shared libraries are involved:

* the *host* library: the reference's unmodified ops.c / vit.c / autodiff.c
  compiled together with host/vit_host.c (flat entry points over its structs).
  Its path is supplied by the caller; this package does not know where it is.
* ``libvitb200.so`` (next to this file): the backend.  It exports the five
  ``cuda_backend_*`` functions of the reference's include/cuda_backend.h and
  plugs itself into the host library through ops_set_device_backend /
  tensor_set_allocator when enabled.

There is no CPU fallback in here: if the backend library is missing or no
B200 is visible, `Backend()` raises.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
BACKEND_LIBRARY = os.path.join(_HERE, "libvitb200.so")

_size_t = ctypes.c_size_t
_float_p = ctypes.POINTER(ctypes.c_float)


class Augmentation(ctypes.Structure):
    """vitb200_augmentation: the reference's DataAugmentation, field for field
    (include/augmentation.h:7-19)."""
    _fields_ = [(name, ctypes.c_float) for name in (
        "max_shift_pixels", "max_rotation_degrees", "max_scale_delta",
        "max_brightness_delta", "max_contrast_delta",
        "noise_standard_deviation", "erasing_probability",
        "erasing_max_side_fraction", "erasing_value", "minimum_value",
        "maximum_value")]


def load_host_library(path, visible_to_backend=True):
    """Loads a host library and declares the flat entry points.  The copy that
    drives the backend is loaded with RTLD_GLOBAL, so that the backend finds
    its ops_set_device_backend / tensor_set_allocator; a copy that serves as
    the CPU checker is loaded with local scope (visible_to_backend=False) and
    never gets a backend installed."""
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL if visible_to_backend
                      else ctypes.RTLD_LOCAL)
    lib.vithost_create.restype = ctypes.c_void_p
    lib.vithost_create.argtypes = [_size_t] * 9 + [ctypes.c_uint64]
    lib.vithost_destroy.argtypes = [ctypes.c_void_p]
    lib.vithost_destroy.restype = None
    lib.vithost_parameter_count.restype = _size_t
    lib.vithost_parameter_count.argtypes = [ctypes.c_void_p]
    lib.vithost_parameter_name.restype = ctypes.c_char_p
    lib.vithost_parameter_name.argtypes = [ctypes.c_void_p, _size_t]
    lib.vithost_parameter_view.restype = _size_t
    lib.vithost_parameter_view.argtypes = [
        ctypes.c_void_p, _size_t, ctypes.c_int, ctypes.POINTER(_float_p),
        ctypes.POINTER(_size_t), ctypes.POINTER(_size_t)]
    lib.vithost_parameter_step.restype = _size_t
    lib.vithost_parameter_step.argtypes = [ctypes.c_void_p, _size_t]
    lib.vithost_gradients.restype = ctypes.c_int
    lib.vithost_gradients.argtypes = [
        ctypes.c_void_p, _float_p, ctypes.POINTER(_size_t), _float_p,
        ctypes.c_float, _float_p]
    lib.vithost_train_step.restype = ctypes.c_int
    lib.vithost_train_step.argtypes = [
        ctypes.c_void_p, _float_p, ctypes.POINTER(_size_t), ctypes.c_float,
        ctypes.c_float, _float_p, ctypes.c_float, _float_p]
    lib.vithost_train_step_accumulated.restype = ctypes.c_int
    lib.vithost_train_step_accumulated.argtypes = [
        ctypes.c_void_p, _float_p, ctypes.POINTER(_size_t), _size_t,
        ctypes.c_float, ctypes.c_float, _float_p, ctypes.c_float, ctypes.c_int,
        _float_p]
    lib.vithost_forward.restype = ctypes.c_int
    lib.vithost_forward.argtypes = [ctypes.c_void_p, _float_p, _float_p]
    lib.vithost_set_parameter.restype = ctypes.c_int
    lib.vithost_set_parameter.argtypes = [ctypes.c_void_p, _size_t, _float_p]
    lib.vithost_block_tensor.restype = _size_t
    lib.vithost_block_tensor.argtypes = [
        ctypes.c_void_p, _size_t, ctypes.c_char_p, ctypes.c_int,
        ctypes.POINTER(_float_p), ctypes.POINTER(_size_t),
        ctypes.POINTER(_size_t)]
    lib.vithost_evaluate.restype = ctypes.c_int
    lib.vithost_evaluate.argtypes = [
        ctypes.c_void_p, _float_p, ctypes.POINTER(_size_t), _size_t, _float_p,
        _float_p, ctypes.POINTER(ctypes.c_double)]
    lib.vithost_predict.restype = ctypes.c_int
    lib.vithost_predict.argtypes = [ctypes.c_void_p, _float_p, _size_t, _float_p]
    lib.vithost_images_tensor.restype = ctypes.c_void_p
    lib.vithost_images_tensor.argtypes = [ctypes.c_void_p]
    lib.ops_synchronize.restype = None
    return lib


def load_backend_library():
    if not os.path.exists(BACKEND_LIBRARY):
        raise RuntimeError(
            f"{BACKEND_LIBRARY} is missing: build it with "
            "`python transformer-in-c_b200/build.py` (there is no CPU fallback)")
    lib = ctypes.CDLL(BACKEND_LIBRARY, mode=ctypes.RTLD_GLOBAL)
    lib.cuda_backend_create.restype = ctypes.c_int
    lib.cuda_backend_create.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
    lib.cuda_backend_free.restype = None
    lib.cuda_backend_free.argtypes = [ctypes.c_void_p]
    lib.cuda_backend_available.restype = ctypes.c_int
    lib.cuda_backend_available.argtypes = [ctypes.c_void_p]
    lib.cuda_backend_enable_device_execution.restype = ctypes.c_int
    lib.cuda_backend_enable_device_execution.argtypes = [ctypes.c_void_p]
    lib.cuda_backend_disable_device_execution.restype = None
    lib.cuda_backend_disable_device_execution.argtypes = [ctypes.c_void_p]
    lib.vitb200_kernel_launches.restype = ctypes.c_ulonglong
    lib.vitb200_memory_counters.restype = None
    lib.vitb200_memory_counters.argtypes = [ctypes.POINTER(_size_t)] * 8
    lib.vitb200_data_augmentation_apply.restype = ctypes.c_int
    lib.vitb200_data_augmentation_apply.argtypes = [
        ctypes.c_void_p, ctypes.POINTER(Augmentation),
        ctypes.POINTER(ctypes.c_uint64), _float_p, _float_p, _size_t, _size_t,
        _size_t, _size_t]
    lib.vitb200_data_augmentation_translate.restype = ctypes.c_int
    lib.vitb200_data_augmentation_translate.argtypes = [
        ctypes.c_void_p, _float_p, _float_p, _size_t, _size_t, _size_t, _size_t,
        ctypes.c_float, ctypes.c_float]
    lib.vitb200_data_augmentation_enabled.restype = ctypes.c_int
    lib.vitb200_data_augmentation_enabled.argtypes = [
        ctypes.POINTER(Augmentation)]
    lib.vitb200_fusion_counters.restype = None
    lib.vitb200_fusion_counters.argtypes = [ctypes.c_void_p] + \
        [ctypes.POINTER(ctypes.c_ulonglong)] * 3
    lib.vitb200_elision_counters.restype = None
    lib.vitb200_elision_counters.argtypes = [ctypes.POINTER(_size_t)] * 5
    lib.vitb200_zero_fill_counters.restype = None
    lib.vitb200_zero_fill_counters.argtypes = [ctypes.POINTER(_size_t)] * 3
    lib.vitb200_set_deferred_synchronize.restype = ctypes.c_int
    lib.vitb200_set_deferred_synchronize.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.vitb200_timer_begin.restype = ctypes.c_int
    lib.vitb200_timer_begin.argtypes = [ctypes.c_void_p]
    lib.vitb200_timer_end.restype = ctypes.c_float
    lib.vitb200_timer_end.argtypes = [ctypes.c_void_p]
    lib.vitb200_dp_unique_id.restype = ctypes.c_int
    lib.vitb200_dp_unique_id.argtypes = [ctypes.c_void_p]
    lib.vitb200_dp_init.restype = ctypes.c_int
    lib.vitb200_dp_init.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_void_p]
    lib.vitb200_dp_shutdown.restype = None
    lib.vitb200_dp_shutdown.argtypes = [ctypes.c_void_p]
    lib.vitb200_dp_counters.restype = None
    lib.vitb200_dp_counters.argtypes = [ctypes.c_void_p] + \
        [ctypes.POINTER(ctypes.c_ulonglong)] * 4
    lib.vitb200_set_gradient_accumulation.restype = ctypes.c_int
    lib.vitb200_set_gradient_accumulation.argtypes = [ctypes.c_void_p,
                                                      ctypes.c_int]
    _ushort_p = ctypes.POINTER(ctypes.c_ushort)
    lib.vitb200_dataset_load_pgm_csv.restype = ctypes.c_int
    lib.vitb200_dataset_load_pgm_csv.argtypes = [
        ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.vitb200_dataset_from_integers.restype = ctypes.c_int
    lib.vitb200_dataset_from_integers.argtypes = [
        ctypes.c_void_p, _ushort_p, _ushort_p, ctypes.POINTER(_size_t), _size_t,
        _size_t, _size_t, ctypes.POINTER(ctypes.c_void_p)]
    lib.vitb200_dataset_free.restype = None
    lib.vitb200_dataset_free.argtypes = [ctypes.c_void_p]
    for name in ("sample_count", "height", "width", "channels"):
        getter = getattr(lib, "vitb200_dataset_" + name)
        getter.restype = _size_t
        getter.argtypes = [ctypes.c_void_p]
    lib.vitb200_dataset_statistics.restype = ctypes.c_int
    lib.vitb200_dataset_statistics.argtypes = [ctypes.c_void_p, _float_p, _float_p]
    lib.vitb200_dataset_shuffle.restype = ctypes.c_int
    lib.vitb200_dataset_shuffle.argtypes = [ctypes.c_void_p,
                                            ctypes.POINTER(ctypes.c_ulong)]
    lib.vitb200_dataset_batch.restype = ctypes.c_int
    lib.vitb200_dataset_batch.argtypes = [
        ctypes.c_void_p, _size_t, _size_t, ctypes.c_float, ctypes.c_float,
        ctypes.c_void_p, ctypes.POINTER(_size_t)]
    lib.vitb200_dataset_parse_pgm_csv.restype = ctypes.c_int
    lib.vitb200_dataset_parse_pgm_csv.argtypes = [
        ctypes.c_char_p, ctypes.POINTER(_ushort_p), ctypes.POINTER(_ushort_p),
        ctypes.POINTER(ctypes.POINTER(_size_t)), ctypes.POINTER(_size_t),
        ctypes.POINTER(_size_t), ctypes.POINTER(_size_t)]
    lib.vitb200_dataset_pixel_statistics.restype = ctypes.c_int
    lib.vitb200_dataset_pixel_statistics.argtypes = [
        _ushort_p, _ushort_p, _size_t, _size_t, _float_p, _float_p]
    lib.vitb200_dataset_shuffle_order.restype = None
    lib.vitb200_dataset_shuffle_order.argtypes = [
        ctypes.POINTER(ctypes.c_uint), _size_t, ctypes.POINTER(ctypes.c_ulong)]
    lib.vitb200_set_gemm_precision.restype = None
    lib.vitb200_set_gemm_precision.argtypes = [ctypes.c_int]
    lib.vitb200_tensor_core_status.restype = ctypes.c_int
    lib.vitb200_device_busy_ms.restype = ctypes.c_double
    lib.vitb200_device_busy_ms.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.vitb200_profile_enable.restype = None
    lib.vitb200_profile_enable.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.vitb200_profile_entries.restype = _size_t
    lib.vitb200_profile_entries.argtypes = [ctypes.c_void_p]
    lib.vitb200_profile_entry.restype = ctypes.c_int
    lib.vitb200_profile_entry.argtypes = [
        ctypes.c_void_p, _size_t, ctypes.POINTER(ctypes.c_char_p),
        ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_double),
        ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
    return lib


class Backend:
    """Owns one CudaBackend.  `enable()` / `disable()` mirror the reference's
    cuda_backend_enable_device_execution / _disable_device_execution."""

    def __init__(self):
        self.lib = load_backend_library()
        handle = ctypes.c_void_p()
        status = self.lib.cuda_backend_create(ctypes.byref(handle))
        if status != 0 or not self.lib.cuda_backend_available(handle):
            raise RuntimeError(
                f"cuda_backend_create returned {status}: no usable B200")
        self.handle = handle
        self.enabled = False

    def enable(self):
        if self.lib.cuda_backend_enable_device_execution(self.handle) != 0:
            raise RuntimeError("cuda_backend_enable_device_execution failed")
        self.enabled = True

    def disable(self):
        self.lib.cuda_backend_disable_device_execution(self.handle)
        self.enabled = False

    def close(self):
        if self.handle:
            self.lib.cuda_backend_free(self.handle)
            self.handle = None

    def kernel_launches(self):
        return int(self.lib.vitb200_kernel_launches())

    def memory_counters(self):
        values = [_size_t() for _ in range(8)]
        self.lib.vitb200_memory_counters(*[ctypes.byref(v) for v in values])
        names = ["live_allocations", "mirror_bytes", "device_bytes",
                 "h2d_copies", "h2d_bytes", "d2h_copies", "d2h_bytes", "faults"]
        return {n: int(v.value) for n, v in zip(names, values)}

    def dp_unique_id(self):
        """128 opaque bytes from rank 0, to be handed to every rank's dp_init."""
        buffer = ctypes.create_string_buffer(128)
        if self.lib.vitb200_dp_unique_id(buffer) != 0:
            raise RuntimeError("NCCL is not available (libnccl.so.2 not found)")
        return buffer.raw

    def dp_init(self, rank, world, unique_id):
        """Collective: joins this backend to a data-parallel group."""
        buffer = ctypes.create_string_buffer(bytes(unique_id), 128)
        if self.lib.vitb200_dp_init(self.handle, rank, world, buffer) != 0:
            raise RuntimeError("vitb200_dp_init failed")

    def dp_shutdown(self):
        self.lib.vitb200_dp_shutdown(self.handle)

    def dp_status(self):
        """0, or the error NCCL reported asynchronously for the exchange (it
        is polled at every synchronise; after an error the communicator has
        been aborted and the backend no longer exchanges anything)."""
        self.lib.vitb200_dp_status.restype = ctypes.c_int
        self.lib.vitb200_dp_status.argtypes = [ctypes.c_void_p]
        return int(self.lib.vitb200_dp_status(self.handle))

    def dp_counters(self):
        values = [ctypes.c_ulonglong() for _ in range(4)]
        self.lib.vitb200_dp_counters(self.handle,
                                     *[ctypes.byref(v) for v in values])
        names = ["all_reduce_calls", "overlapped_tensors", "late_tensors", "bytes"]
        counters = {n: int(v.value) for n, v in zip(names, values)}
        self.lib.vitb200_dp_flat_ranges.restype = ctypes.c_ulonglong
        self.lib.vitb200_dp_flat_ranges.argtypes = [ctypes.c_void_p]
        counters["flat_ranges"] = int(self.lib.vitb200_dp_flat_ranges(self.handle))
        return counters

    def set_gradient_accumulation(self, micro_batches):
        """The following optimiser steps consume gradients summed over this
        many forward/backward passes (VitHost.train_step_accumulated)."""
        if self.lib.vitb200_set_gradient_accumulation(
                self.handle, int(micro_batches)) != 0:
            raise ValueError("vitb200_set_gradient_accumulation failed")

    def set_gemm_precision(self, precision):
        """0 auto, 1 FP32 FMA, 2 TF32 tensor cores, -1 start-up default."""
        self.lib.vitb200_set_gemm_precision(int(precision))

    def tensor_core_status(self):
        return int(self.lib.vitb200_tensor_core_status())

    def elision_counters(self):
        values = [_size_t() for _ in range(5)]
        self.lib.vitb200_elision_counters(*[ctypes.byref(v) for v in values])
        names = ["zero_fills_elided", "zero_fills_materialised", "lazy_defined",
                 "lazy_materialised", "lazy_dropped"]
        return {n: int(v.value) for n, v in zip(names, values)}

    def zero_fill_counters(self):
        values = [_size_t() for _ in range(3)]
        self.lib.vitb200_zero_fill_counters(*[ctypes.byref(v) for v in values])
        return {n: int(v.value)
                for n, v in zip(["memsets", "batched", "prefetched_reads"], values)}

    def augment(self, settings, state, source, destination=None):
        """vitb200_data_augmentation_apply on host arrays.  `settings` maps the
        reference's DataAugmentation field names to numbers; source is
        [batch, channels, height, width] float32.  Returns
        (status, destination, new_state); destination=source (the same array)
        asks for in-place operation."""
        config = Augmentation(**{k: float(v) for k, v in settings.items()})
        source = np.ascontiguousarray(source, dtype=np.float32)
        if destination is None:
            destination = np.zeros_like(source)
        rng = ctypes.c_uint64(state)
        batch, channels, height, width = source.shape
        status = self.lib.vitb200_data_augmentation_apply(
            self.handle, ctypes.byref(config), ctypes.byref(rng),
            source.ctypes.data_as(_float_p), destination.ctypes.data_as(_float_p),
            batch, channels, height, width)
        return int(status), destination, int(rng.value)

    def translate(self, source, shift_y, shift_x):
        source = np.ascontiguousarray(source, dtype=np.float32)
        destination = np.zeros_like(source)
        batch, channels, height, width = source.shape
        status = self.lib.vitb200_data_augmentation_translate(
            self.handle, source.ctypes.data_as(_float_p),
            destination.ctypes.data_as(_float_p), batch, channels, height,
            width, ctypes.c_float(shift_y), ctypes.c_float(shift_x))
        return int(status), destination

    def fusion_counters(self):
        values = [ctypes.c_ulonglong() for _ in range(3)]
        self.lib.vitb200_fusion_counters(self.handle,
                                         *[ctypes.byref(v) for v in values])
        names = ["epilogues", "head_layouts", "bias_gradients"]
        return {n: int(v.value) for n, v in zip(names, values)}

    def declined_ops(self):
        """Op-table calls the backend declined (the host ran its CPU loop)."""
        self.lib.vitb200_declined_ops.restype = ctypes.c_ulonglong
        self.lib.vitb200_declined_ops.argtypes = [ctypes.c_void_p]
        return int(self.lib.vitb200_declined_ops(self.handle))

    def kernel_paths(self):
        values = [ctypes.c_ulonglong() for _ in range(5)]
        self.lib.vitb200_kernel_path_counters.restype = None
        self.lib.vitb200_kernel_path_counters.argtypes = \
            [ctypes.c_void_p] + [ctypes.POINTER(ctypes.c_ulonglong)] * 5
        self.lib.vitb200_kernel_path_counters(
            self.handle, *[ctypes.byref(v) for v in values])
        names = ["tensor_core_products", "wide_tile_products", "fma_products",
                 "tensor_core_attention", "streaming_attention"]
        return {n: int(v.value) for n, v in zip(names, values)}

    def set_deferred_synchronize(self, on):
        """The `synchronize` slot stops waiting for the device (host accesses
        still wait for what they read); returns the previous setting."""
        return int(self.lib.vitb200_set_deferred_synchronize(self.handle, int(on)))

    def device_busy_ms(self, reset=False):
        return float(self.lib.vitb200_device_busy_ms(self.handle, int(reset)))

    def profile(self, on):
        self.lib.vitb200_profile_enable(self.handle, int(on))

    def profile_entries(self):
        """[{name, calls, ms, bytes, flops}] accumulated since profile(True)."""
        entries = []
        for i in range(int(self.lib.vitb200_profile_entries(self.handle))):
            name = ctypes.c_char_p()
            calls = ctypes.c_ulonglong()
            ms, nbytes, flops = ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
            self.lib.vitb200_profile_entry(
                self.handle, i, ctypes.byref(name), ctypes.byref(calls),
                ctypes.byref(ms), ctypes.byref(nbytes), ctypes.byref(flops))
            entries.append({"name": name.value.decode(), "calls": int(calls.value),
                            "ms": ms.value, "bytes": nbytes.value,
                            "flops": flops.value})
        return entries

    def timer_begin(self):
        self.lib.vitb200_timer_begin(self.handle)

    def timer_end(self):
        return float(self.lib.vitb200_timer_end(self.handle))


def parse_pgm_csv(lib, manifest_path):
    """vitb200_dataset_parse_pgm_csv (no device): (status, pixels
    [samples, height, width] uint16, max_values, labels)."""
    pixels = ctypes.POINTER(ctypes.c_ushort)()
    maxima = ctypes.POINTER(ctypes.c_ushort)()
    labels = ctypes.POINTER(_size_t)()
    count, height, width = _size_t(), _size_t(), _size_t()
    status = lib.vitb200_dataset_parse_pgm_csv(
        os.fsencode(manifest_path), ctypes.byref(pixels), ctypes.byref(maxima),
        ctypes.byref(labels), ctypes.byref(count), ctypes.byref(height),
        ctypes.byref(width))
    if status != 0:
        return status, None, None, None
    n, h, w = int(count.value), int(height.value), int(width.value)
    out = (np.ctypeslib.as_array(pixels, shape=(n, h, w)).copy(),
           np.ctypeslib.as_array(maxima, shape=(n,)).copy(),
           np.ctypeslib.as_array(labels, shape=(n,)).copy())
    libc = ctypes.CDLL(None)
    libc.free.argtypes = [ctypes.c_void_p]
    for pointer in (pixels, maxima, labels):
        libc.free(ctypes.cast(pointer, ctypes.c_void_p))
    return 0, out[0], out[1], out[2]


class Dataset:
    """A vitb200_dataset: samples resident on the backend's device
    (include/vitb200_dataset.h)."""

    def __init__(self, backend, manifest_path=None, pixels=None, max_values=None,
                 labels=None):
        self.backend = backend
        self.lib = backend.lib
        handle = ctypes.c_void_p()
        if manifest_path is not None:
            status = self.lib.vitb200_dataset_load_pgm_csv(
                backend.handle, os.fsencode(manifest_path), ctypes.byref(handle))
        else:
            pixels = np.ascontiguousarray(pixels, dtype=np.uint16)
            labels = np.ascontiguousarray(labels, dtype=np.uintp)
            maxima = None
            if max_values is not None:
                maxima = np.ascontiguousarray(max_values, dtype=np.uint16)
            ushort_p = ctypes.POINTER(ctypes.c_ushort)
            status = self.lib.vitb200_dataset_from_integers(
                backend.handle, pixels.ctypes.data_as(ushort_p),
                maxima.ctypes.data_as(ushort_p) if maxima is not None else None,
                labels.ctypes.data_as(ctypes.POINTER(_size_t)), pixels.shape[0],
                pixels.shape[1], pixels.shape[2], ctypes.byref(handle))
        if status != 0 or not handle:
            raise RuntimeError("the dataset could not be loaded")
        self.handle = handle
        self.samples = int(self.lib.vitb200_dataset_sample_count(handle))
        self.height = int(self.lib.vitb200_dataset_height(handle))
        self.width = int(self.lib.vitb200_dataset_width(handle))

    def close(self):
        if self.handle:
            self.lib.vitb200_dataset_free(self.handle)
            self.handle = None

    def statistics(self):
        mean, inverse = ctypes.c_float(), ctypes.c_float()
        self.lib.vitb200_dataset_statistics(self.handle, ctypes.byref(mean),
                                            ctypes.byref(inverse))
        return float(mean.value), float(inverse.value)

    def shuffle(self, state):
        """Returns the generator state after the shuffle's draws."""
        value = ctypes.c_ulong(state)
        if self.lib.vitb200_dataset_shuffle(self.handle, ctypes.byref(value)) != 0:
            raise RuntimeError("vitb200_dataset_shuffle failed")
        return int(value.value)

    def batch(self, offset, batch, mean, inverse_std, destination=None):
        """(status, images, labels).  `destination`: None (a new host array), a
        float32 host array, or an integer address of tensor memory."""
        labels = np.empty(batch, np.uintp)
        if isinstance(destination, int):
            target, images = ctypes.c_void_p(destination), None
        else:
            images = destination if destination is not None else np.empty(
                (batch, self.height * self.width), np.float32)
            target = ctypes.c_void_p(images.ctypes.data)
        status = self.lib.vitb200_dataset_batch(
            self.handle, offset, batch, ctypes.c_float(mean),
            ctypes.c_float(inverse_std), target,
            labels.ctypes.data_as(ctypes.POINTER(_size_t)))
        return int(status), images, labels


class VitHost:
    """A model plus its activation cache, created through the reference's
    vit_model_init_seeded / vit_model_cache_init.  Tensors land on the device
    iff a backend is enabled at construction time (reference
    tests/test_device.c:141-170 relies on the same rule)."""

    def __init__(self, host_lib, config, batch, seed=42):
        self.lib = host_lib
        self.config = tuple(int(v) for v in config)
        self.batch = int(batch)
        self.handle = host_lib.vithost_create(*self.config, self.batch, seed)
        if not self.handle:
            raise RuntimeError("vithost_create failed")
        self.count = int(host_lib.vithost_parameter_count(self.handle))
        self.names = []
        layer = -1
        for i in range(self.count):
            name = host_lib.vithost_parameter_name(self.handle, i).decode()
            if name == "query_key_value":
                layer += 1
            per_layer = i >= 4 and i < self.count - 4
            self.names.append(f"{layer}.{name}" if per_layer else name)

    def close(self):
        if self.handle:
            self.lib.vithost_destroy(self.handle)
            self.handle = None

    def _view(self, index, what):
        data = _float_p()
        rows, cols = _size_t(), _size_t()
        count = self.lib.vithost_parameter_view(
            self.handle, index, what, ctypes.byref(data), ctypes.byref(rows),
            ctypes.byref(cols))
        array = np.ctypeslib.as_array(data, shape=(int(count),))
        return array.reshape(int(rows.value), int(cols.value))

    def parameters(self, what=0):
        """Copies of every parameter's value (0), gradient (1), first (2) or
        second (3) moment, keyed like oracle.vit_oracle.parameter_names."""
        return {name: self._view(i, what).copy()
                for i, name in enumerate(self.names)}

    def set_parameters(self, values):
        for i, name in enumerate(self.names):
            array = np.ascontiguousarray(values[name], dtype=np.float32)
            if self.lib.vithost_set_parameter(
                    self.handle, i, array.ctypes.data_as(_float_p)) != 0:
                raise RuntimeError(f"set_parameter({name}) failed")

    def steps(self):
        return [int(self.lib.vithost_parameter_step(self.handle, i))
                for i in range(self.count)]

    @staticmethod
    def _inputs(images, labels, class_weights):
        images = np.ascontiguousarray(images, dtype=np.float32)
        labels = np.ascontiguousarray(labels, dtype=np.uintp)
        weights = None
        if class_weights is not None:
            weights = np.ascontiguousarray(class_weights, dtype=np.float32)
        return images, labels, weights

    def gradients(self, images, labels, class_weights=None, label_smoothing=0.0):
        images, labels, weights = self._inputs(images, labels, class_weights)
        loss = ctypes.c_float()
        status = self.lib.vithost_gradients(
            self.handle, images.ctypes.data_as(_float_p),
            labels.ctypes.data_as(ctypes.POINTER(_size_t)),
            weights.ctypes.data_as(_float_p) if weights is not None else None,
            label_smoothing, ctypes.byref(loss))
        if status != 0:
            raise RuntimeError("vithost_gradients failed")
        return float(loss.value)

    def train_step(self, images, labels, lr, weight_decay, class_weights=None,
                   label_smoothing=0.0):
        images, labels, weights = self._inputs(images, labels, class_weights)
        return self.train_step_raw(images, labels, lr, weight_decay, weights,
                                   label_smoothing)

    def train_step_raw(self, images, labels, lr, weight_decay, weights,
                       label_smoothing):
        """Same as train_step for inputs that are already contiguous float32 /
        uintp arrays (no conversions inside a timed loop)."""
        loss = ctypes.c_float()
        status = self.lib.vithost_train_step(
            self.handle, images.ctypes.data_as(_float_p),
            labels.ctypes.data_as(ctypes.POINTER(_size_t)), lr, weight_decay,
            weights.ctypes.data_as(_float_p) if weights is not None else None,
            label_smoothing, ctypes.byref(loss))
        if status != 0:
            raise RuntimeError("vit_model_train_batch_smoothed failed")
        return float(loss.value)

    def train_step_accumulated(self, images, labels, micro_batches, lr,
                               weight_decay, weights=None, label_smoothing=0.0,
                               scale_on_host=False):
        """One optimiser step over `micro_batches` x batch images (contiguous
        float32 / uintp arrays).  On a device model the backend must have been
        told the count (Backend.set_gradient_accumulation); a CPU model passes
        scale_on_host=True instead."""
        loss = ctypes.c_float()
        status = self.lib.vithost_train_step_accumulated(
            self.handle, images.ctypes.data_as(_float_p),
            labels.ctypes.data_as(ctypes.POINTER(_size_t)), int(micro_batches),
            lr, weight_decay,
            weights.ctypes.data_as(_float_p) if weights is not None else None,
            label_smoothing, int(scale_on_host), ctypes.byref(loss))
        if status != 0:
            raise RuntimeError("vithost_train_step_accumulated failed")
        return float(loss.value)

    def images_tensor(self):
        """Host address of the cache's image tensor (tensor memory)."""
        return int(self.lib.vithost_images_tensor(self.handle))

    def forward_from_address(self, address):
        """vit_model_forward with the images read from `address` (for example
        images_tensor() after a device-side producer has filled it)."""
        logits = np.empty((self.batch, self.config[7]), np.float32)
        if self.lib.vithost_forward(self.handle,
                                    ctypes.cast(ctypes.c_void_p(address), _float_p),
                                    logits.ctypes.data_as(_float_p)) != 0:
            raise RuntimeError("vit_model_forward failed")
        return logits

    def forward(self, images):
        images = np.ascontiguousarray(images, dtype=np.float32)
        logits = np.empty((self.batch, self.config[7]), np.float32)
        if self.lib.vithost_forward(self.handle,
                                    images.ctypes.data_as(_float_p),
                                    logits.ctypes.data_as(_float_p)) != 0:
            raise RuntimeError("vit_model_forward failed")
        return logits

    def evaluate(self, images, labels):
        """vit_model_evaluate: (accuracy, average loss, samples per second)."""
        images = np.ascontiguousarray(images, dtype=np.float32)
        labels = np.ascontiguousarray(labels, dtype=np.uintp)
        accuracy, loss = ctypes.c_float(), ctypes.c_float()
        rate = ctypes.c_double()
        if self.lib.vithost_evaluate(
                self.handle, images.ctypes.data_as(_float_p),
                labels.ctypes.data_as(ctypes.POINTER(_size_t)), len(labels),
                ctypes.byref(accuracy), ctypes.byref(loss),
                ctypes.byref(rate)) != 0:
            raise RuntimeError("vit_model_evaluate failed")
        return float(accuracy.value), float(loss.value), float(rate.value)

    def predict(self, images):
        """vit_model_predict_probabilities: [samples, classes]."""
        images = np.ascontiguousarray(images, dtype=np.float32)
        count = images.shape[0]
        out = np.empty((count, self.config[7]), np.float32)
        if self.lib.vithost_predict(self.handle,
                                    images.ctypes.data_as(_float_p), count,
                                    out.ctypes.data_as(_float_p)) != 0:
            raise RuntimeError("vit_model_predict_probabilities failed")
        return out

    def block_tensor(self, layer, name, grad=False):
        data = _float_p()
        rows, cols = _size_t(), _size_t()
        count = self.lib.vithost_block_tensor(
            self.handle, layer, name.encode(), int(grad), ctypes.byref(data),
            ctypes.byref(rows), ctypes.byref(cols))
        if count == 0:
            raise KeyError(name)
        array = np.ctypeslib.as_array(data, shape=(int(count),))
        return array.reshape(int(rows.value), int(cols.value)).copy()


class ExchangeError(RuntimeError):
    """A rank of the data-parallel group is missing, late or gone."""


class ExchangeGroup:
    """Host-side failure detection around the gradient exchange.

    NCCL's collectives (and ncclCommInitRank itself) block until every rank
    takes part, so a rank that never starts, or leaves between two steps,
    would leave the others waiting inside a kernel on their GPUs.  Everything
    that can be learnt on the host is therefore checked on the host first,
    through a small key/value store every rank can reach (anything with the
    set / get / wait / check interface of torch.distributed's TCPStore or
    FileStore):

      rendezvous(make_id)   rank 0 publishes the 128 id bytes, every rank
                            announces itself, and nobody proceeds to
                            Backend.dp_init before all ranks have, within
                            `timeout` seconds; otherwise ExchangeError names
                            what is missing and no collective has been entered
      before_step(step)     each rank records the step it is about to launch
                            and checks, before launching anything, that no
                            rank has announced its departure and that every
                            rank has reached the previous step within
                            `timeout` seconds
      leave()               announces a departure; a rank calls it between
                            steps, with none of its kernels or collectives in
                            flight (after a synchronise)

    Nothing here touches a GPU."""

    def __init__(self, store, rank, world, timeout=30.0, prefix="vitb200"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout, self.prefix = float(timeout), prefix

    def _key(self, *parts):
        return "/".join([self.prefix, *[str(p) for p in parts]])

    def _wait(self, keys, what):
        import datetime
        try:
            self.store.wait(keys, datetime.timedelta(seconds=self.timeout))
        except Exception as error:   # the stores raise their own timeout types
            missing = [k for k in keys if not self.store.check([k])]
            raise ExchangeError(
                f"rank {self.rank}: {what} within {self.timeout:g} s "
                f"(missing: {', '.join(missing) or 'unknown'})") from error

    def rendezvous(self, make_id):
        if self.rank == 0:
            self.store.set(self._key("id"), bytes(make_id()))
        self._wait([self._key("id")], "rank 0 never published the exchange id")
        unique_id = bytes(self.store.get(self._key("id")))
        self.store.set(self._key("joined", self.rank), b"1")
        self._wait([self._key("joined", r) for r in range(self.world)],
                   "not every rank joined the exchange")
        return unique_id

    def leave(self):
        self.store.set(self._key("left", self.rank), b"1")

    def before_step(self, step):
        import time
        self.store.set(self._key("step", self.rank), str(int(step)).encode())
        deadline = time.monotonic() + self.timeout
        for peer in range(self.world):
            if peer == self.rank:
                continue
            while True:
                if self.store.check([self._key("left", peer)]):
                    raise ExchangeError(
                        f"rank {self.rank}: rank {peer} has left the exchange "
                        f"(noticed before step {step})")
                reached = -1
                if self.store.check([self._key("step", peer)]):
                    reached = int(bytes(self.store.get(self._key("step", peer))))
                if reached >= step - 1:
                    break
                if time.monotonic() > deadline:
                    raise ExchangeError(
                        f"rank {self.rank}: rank {peer} has not reached step "
                        f"{step - 1} within {self.timeout:g} s (last seen at "
                        f"step {reached})")
                time.sleep(0.01)


def synthetic_batch(batch, height, width, classes, seed):
    """Stand-in for an OrganSMNIST batch: uint8 pixels uniform in 0..255,
    scaled to [0,1] and standardised over the batch; labels uniform."""
    rng = np.random.RandomState(seed)
    pixels = rng.randint(0, 256, size=(batch, height * width)).astype(np.float32)
    pixels /= 255.0
    images = (pixels - pixels.mean()) / pixels.std()
    labels = rng.randint(0, classes, size=batch).astype(np.uintp)
    return images.astype(np.float32), labels
