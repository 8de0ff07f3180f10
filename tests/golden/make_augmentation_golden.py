"""Writes tests/golden/augmentation.npz from the reference's own compiled
data_augmentation_apply / data_augmentation_translate (oracle/_ref/libvithost.so,
built from the reference's src/augmentation.c by oracle/build_ref.py).

Run where the reference tree is available:
    python oracle/build_ref.py && python tests/golden/make_augmentation_golden.py
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(REPO, "oracle"))
import augmentation_oracle as ao  # noqa: E402


class DataAugmentation(ctypes.Structure):
    _fields_ = [(name, ctypes.c_float) for name in ao.FIELDS]


def reference_library():
    lib = ctypes.CDLL(os.path.join(REPO, "oracle", "_ref", "libvithost.so"))
    fp = ctypes.POINTER(ctypes.c_float)
    lib.data_augmentation_apply.restype = ctypes.c_int
    lib.data_augmentation_apply.argtypes = [
        ctypes.POINTER(DataAugmentation), ctypes.POINTER(ctypes.c_uint64), fp,
        fp, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t]
    lib.data_augmentation_translate.restype = ctypes.c_int
    lib.data_augmentation_translate.argtypes = [
        fp, fp, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t,
        ctypes.c_size_t, ctypes.c_float, ctypes.c_float]
    return lib


def reference_apply(lib, settings, state, source):
    """Returns (status, destination, new_state) from the reference's C code."""
    a = DataAugmentation(**{k: float(v) for k, v in settings.items()})
    source = np.ascontiguousarray(source, dtype=np.float32)
    out = np.zeros_like(source)
    rng = ctypes.c_uint64(state)
    fp = ctypes.POINTER(ctypes.c_float)
    batch, channels, height, width = source.shape
    status = lib.data_augmentation_apply(
        ctypes.byref(a), ctypes.byref(rng), source.ctypes.data_as(fp),
        out.ctypes.data_as(fp), batch, channels, height, width)
    return status, out, int(rng.value)


def reference_translate(lib, source, shift_y, shift_x):
    source = np.ascontiguousarray(source, dtype=np.float32)
    out = np.zeros_like(source)
    fp = ctypes.POINTER(ctypes.c_float)
    batch, channels, height, width = source.shape
    status = lib.data_augmentation_translate(
        source.ctypes.data_as(fp), out.ctypes.data_as(fp), batch, channels,
        height, width, shift_y, shift_x)
    return status, out


def settings(**overrides):
    base = dict.fromkeys(ao.FIELDS, 0.0)
    base.update(overrides)
    return base


# The trainer's defaults after normalisation with the OrganSMNIST statistics
# would scale brightness / noise by 1/std; plain [0, 1] pixels are used here.
TRAINER = settings(max_shift_pixels=2.0, max_rotation_degrees=10.0,
                   max_scale_delta=0.1, max_brightness_delta=0.05,
                   max_contrast_delta=0.1, noise_standard_deviation=0.01,
                   erasing_probability=0.25, erasing_max_side_fraction=0.4,
                   erasing_value=0.5, minimum_value=0.0, maximum_value=1.0)

CASES = {
    # name: (settings, state, (batch, channels, height, width))
    "trainer_28": (TRAINER, 1234, (6, 1, 28, 28)),
    "all_on_4x4": (settings(max_shift_pixels=1.0, max_rotation_degrees=15.0,
                            max_scale_delta=0.1, max_brightness_delta=0.1,
                            max_contrast_delta=0.2,
                            noise_standard_deviation=0.05,
                            erasing_probability=1.0,
                            erasing_max_side_fraction=0.5, erasing_value=0.5,
                            minimum_value=0.0, maximum_value=1.0),
                   1, (2, 1, 4, 4)),
    "geometry_only_rgb": (settings(max_shift_pixels=3.0,
                                   max_rotation_degrees=45.0,
                                   max_scale_delta=0.3), 99, (3, 3, 9, 13)),
    "intensity_noise_no_clamp": (settings(max_brightness_delta=0.2,
                                          max_contrast_delta=0.5,
                                          noise_standard_deviation=0.1),
                                 7, (4, 2, 5, 7)),
    "erasing_only": (settings(erasing_probability=0.6,
                              erasing_max_side_fraction=1.0,
                              erasing_value=-1.0), 2024, (16, 1, 8, 8)),
    "clamp_only_noise": (settings(noise_standard_deviation=0.5,
                                  minimum_value=0.25, maximum_value=0.75),
                         5, (2, 1, 6, 6)),
    "single_pixel": (settings(max_shift_pixels=1.0,
                              noise_standard_deviation=0.1,
                              erasing_probability=1.0,
                              erasing_max_side_fraction=0.0), 11, (3, 1, 1, 1)),
}


def case_source(name, shape):
    rng = np.random.RandomState(sum(map(ord, name)))
    return rng.randint(0, 256, size=shape).astype(np.float32) / np.float32(255.0)


def main():
    lib = reference_library()
    arrays = {}
    for name, (config, state, shape) in CASES.items():
        source = case_source(name, shape)
        status, out, new_state = reference_apply(lib, config, state, source)
        assert status == 0, name
        arrays[name + "/out"] = out
        arrays[name + "/state"] = np.array([new_state], dtype=np.uint64)
    source = case_source("translate", (2, 2, 7, 5))
    status, out = reference_translate(lib, source, 1.5, -0.75)
    assert status == 0
    arrays["translate/out"] = out
    path = os.path.join(HERE, "augmentation.npz")
    np.savez_compressed(path, **arrays)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
