"""Device augmentation (vitb200_data_augmentation_apply / _translate) against
the reference's compiled C code where it is present, the committed fixtures it
produced, and the numpy restatement at batch sizes the fixtures do not cover.

Everything except the Gaussian noise is bit-identical by construction (same
draws, same rounding of every operation; cos / sin of the rotation come from
the host's libm).  The noise passes through the device's logf and cosf, whose
last-bit differences can also move the rounding of pixel + noise by one unit
in the last place of the pixel; cases with noise are therefore compared to
NOISE_TOLERANCE of the noise amplitude plus one ulp of the largest pixel."""
import os

import numpy as np
import pytest

from conftest import REPO, load_module

pytestmark = pytest.mark.gpu

ao = load_module("augmentation_oracle", os.path.join(REPO, "oracle", "augmentation_oracle.py"))
golden_maker = load_module("make_augmentation_golden",
                           os.path.join(REPO, "tests", "golden", "make_augmentation_golden.py"))
GOLDEN = np.load(os.path.join(REPO, "tests", "golden", "augmentation.npz"))
HAVE_REFERENCE = os.path.exists(os.path.join(REPO, "oracle", "_ref", "libvithost.so"))
NOISE_TOLERANCE = 4e-6   # x noise standard deviation; libm differences only


def allowed_error(config, largest=1.0):
    sigma = float(config["noise_standard_deviation"])
    if sigma == 0.0:
        return 0.0
    return NOISE_TOLERANCE * sigma + float(np.spacing(np.float32(largest)))


@pytest.mark.parametrize("name", sorted(golden_maker.CASES))
def test_matches_reference_fixture(backend, name):
    config, state, shape = golden_maker.CASES[name]
    source = golden_maker.case_source(name, shape)
    status, out, new_state = backend.augment(config, state, source)
    assert status == 0
    assert new_state == int(GOLDEN[name + "/state"][0])
    expected = GOLDEN[name + "/out"]
    if allowed_error(config) == 0.0:
        assert np.array_equal(out, expected)
    else:
        np.testing.assert_allclose(out, expected, rtol=0,
                                   atol=allowed_error(config, np.abs(expected).max()))


def test_translate_is_bit_identical(backend):
    source = golden_maker.case_source("translate", (2, 2, 7, 5))
    status, out = backend.translate(source, 1.5, -0.75)
    assert status == 0
    assert np.array_equal(out, GOLDEN["translate/out"])
    assert backend.translate(source[:0], 0.0, 0.0)[0] == -1   # empty batch


@pytest.mark.skipif(not HAVE_REFERENCE, reason="reference build not present")
@pytest.mark.parametrize("batch,height,width,channels", [
    (2048, 28, 28, 1), (64, 64, 64, 1), (33, 17, 9, 3), (1, 28, 28, 1),
])
def test_matches_reference_at_training_sizes(backend, batch, height, width, channels):
    """The trainer's settings (examples/organ_smnist.c:142-151) at the bench
    batch: same draw count, every pixel within the noise tolerance, and the
    erased rectangles and clamped pixels exactly equal."""
    lib = golden_maker.reference_library()
    config = golden_maker.TRAINER
    rng = np.random.RandomState(batch + height)
    source = rng.randint(0, 256, size=(batch, channels, height, width)).astype(np.float32) / np.float32(255)
    state = 20240 + batch
    ref_status, expected, ref_state = golden_maker.reference_apply(lib, config, state, source)
    status, out, new_state = backend.augment(config, state, source)
    assert status == ref_status == 0
    assert new_state == ref_state
    np.testing.assert_allclose(out, expected, rtol=0,
                                   atol=allowed_error(config, np.abs(expected).max()))
    exact = (expected == config["erasing_value"]) | (expected == 0.0) | (expected == 1.0)
    assert np.array_equal(out[exact], expected[exact])
    # A second batch continues the same stream.
    _, expected2, ref_state2 = golden_maker.reference_apply(lib, config, ref_state, source)
    _, out2, new_state2 = backend.augment(config, new_state, source)
    assert new_state2 == ref_state2
    np.testing.assert_allclose(out2, expected2, rtol=0,
                               atol=allowed_error(config, np.abs(expected2).max()))


def test_without_noise_large_batch_is_bit_identical_to_the_oracle(backend):
    config = dict(golden_maker.TRAINER, noise_standard_deviation=0.0)
    source = np.random.RandomState(5).rand(257, 1, 28, 28).astype(np.float32)
    expected, expected_state = ao.apply(config, 77, source)
    status, out, new_state = backend.augment(config, 77, source)
    assert status == 0 and new_state == expected_state
    # numpy's cos / sin may differ from the host libm by an ulp in the rotation.
    np.testing.assert_allclose(out, expected, rtol=0, atol=2e-6)


def test_reference_unit_test_expectations(backend):
    """tests/test_vision.c:831-871 through the device entry points."""
    source = (np.arange(32, dtype=np.float32) % 16 / np.float32(15.0)).reshape(2, 1, 4, 4)
    identity = golden_maker.settings()
    status, out, state = backend.augment(identity, 1, source)
    assert status == 0 and state == 1 and np.array_equal(out, source)
    config, _, _ = golden_maker.CASES["all_on_4x4"]
    status, out, _ = backend.augment(config, 1, source)
    assert status == 0
    assert np.isfinite(out).all() and out.min() >= 0.0 and out.max() <= 1.0
    # In place with a geometric transform is refused, and nothing is drawn.
    status, _, state = backend.augment(config, 1, source, destination=source)
    assert status == -1 and state == 1


def test_in_place_without_geometry_and_invalid_settings(backend):
    config = golden_maker.settings(max_contrast_delta=0.3, max_brightness_delta=0.1,
                                   erasing_probability=0.5, erasing_max_side_fraction=0.5,
                                   erasing_value=0.25)
    source = np.random.RandomState(3).rand(9, 2, 6, 5).astype(np.float32)
    expected, expected_state = ao.apply(config, 31, source)
    buffer = source.copy()
    status, out, state = backend.augment(config, 31, buffer, destination=buffer)
    assert status == 0 and out is buffer and state == expected_state
    assert np.array_equal(buffer, expected)
    for bad in (dict(max_scale_delta=1.0), dict(max_contrast_delta=1.5),
                dict(erasing_probability=1.5), dict(noise_standard_deviation=-0.1),
                dict(max_shift_pixels=-1.0), dict(erasing_max_side_fraction=2.0)):
        status, _, state = backend.augment(golden_maker.settings(**bad), 5, source)
        assert status == -1 and state == 5


def test_tensor_memory_is_augmented_where_it_lives(vit_host_module, host_lib, backend):
    """Source and destination that were allocated through the backend (here the
    value and the gradient of a model parameter, 512 floats each) are used in
    place on the device: nothing is copied back until the host reads."""
    import ctypes
    vh = vit_host_module
    backend.enable()
    model = vh.VitHost(host_lib, (1, 28, 28, 4, 32, 4, 1, 11), 4)
    shape = (2, 1, 16, 16)
    source = np.random.RandomState(9).rand(*shape).astype(np.float32)
    float_p = ctypes.POINTER(ctypes.c_float)
    assert host_lib.vithost_set_parameter(model.handle, 0,
                                          source.ctypes.data_as(float_p)) == 0
    value = model._view(0, 0).ctypes.data_as(float_p)      # no host access
    gradient = model._view(0, 1).ctypes.data_as(float_p)
    config = dict(golden_maker.TRAINER, noise_standard_deviation=0.0)
    settings = vh.Augmentation(**{k: float(v) for k, v in config.items()})
    rng = ctypes.c_uint64(123)
    before = backend.memory_counters()
    status = backend.lib.vitb200_data_augmentation_apply(
        backend.handle, ctypes.byref(settings), ctypes.byref(rng), value,
        gradient, *shape)
    assert status == 0
    assert backend.memory_counters()["d2h_copies"] == before["d2h_copies"]
    out = model._view(0, 1).reshape(shape).copy()           # host read: faults in
    assert backend.memory_counters()["d2h_copies"] == before["d2h_copies"] + 1
    expected, expected_state = ao.apply(config, 123, source)
    assert int(rng.value) == expected_state
    np.testing.assert_allclose(out, expected, rtol=0, atol=2e-6)
    model.close()
    backend.disable()
