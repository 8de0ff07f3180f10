"""The numpy restatement of the reference's augmentation against fixtures made
by the reference's compiled C code (tests/golden/augmentation.npz, written by
tests/golden/make_augmentation_golden.py), plus the reference's own unit-test
expectations (tests/test_vision.c:831-871)."""
import os

import numpy as np
import pytest

from conftest import REPO, load_module

ao = load_module("augmentation_oracle", os.path.join(REPO, "oracle", "augmentation_oracle.py"))
golden_maker = load_module("make_augmentation_golden",
                           os.path.join(REPO, "tests", "golden", "make_augmentation_golden.py"))
GOLDEN = np.load(os.path.join(REPO, "tests", "golden", "augmentation.npz"))

# libm (cosf, sinf, logf) may differ by an ulp between numpy and glibc; the
# pixels are O(1), the noise a small multiple of that.
TOLERANCE = 2e-6


@pytest.mark.parametrize("name", sorted(golden_maker.CASES))
def test_oracle_matches_reference_fixture(name):
    config, state, shape = golden_maker.CASES[name]
    source = golden_maker.case_source(name, shape)
    out, new_state = ao.apply(config, state, source)
    assert new_state == int(GOLDEN[name + "/state"][0])   # same number of draws
    np.testing.assert_allclose(out, GOLDEN[name + "/out"], rtol=0, atol=TOLERANCE)


def test_translate_matches_reference_fixture():
    source = golden_maker.case_source("translate", (2, 2, 7, 5))
    np.testing.assert_allclose(ao.translate(source, 1.5, -0.75),
                               GOLDEN["translate/out"], rtol=0, atol=TOLERANCE)


def test_reference_unit_test_expectations():
    """tests/test_vision.c:831-871: a zeroed configuration is the identity and
    draws nothing; the full configuration keeps pixels finite and inside the
    clamp range; in-place use with a geometric transform is refused."""
    source = (np.arange(32, dtype=np.float32) % 16 / np.float32(15.0)).reshape(2, 1, 4, 4)
    identity = golden_maker.settings()
    assert not ao.enabled(identity)
    out, state = ao.apply(identity, 1, source)
    assert state == 1 and np.array_equal(out, source)
    config, _, _ = golden_maker.CASES["all_on_4x4"]
    assert ao.enabled(config)
    out, _ = ao.apply(config, 1, source)
    assert np.isfinite(out).all() and out.min() >= 0.0 and out.max() <= 1.0
    assert ao.valid(config, same_buffer=False)
    assert not ao.valid(config, same_buffer=True)


def test_draws_are_a_pure_function_of_the_start_state():
    """Draw k of a splitmix64 stream is mix(state + (k+1) * GOLDEN): the
    property the device kernels rely on to generate noise per pixel."""
    stream = ao.Stream(42)
    sequential = [stream.bits() for _ in range(50)]
    direct = [ao.mix((42 + (k + 1) * ao.GOLDEN) & ao.MASK) for k in range(50)]
    assert sequential == direct


@pytest.mark.skipif(not os.path.exists(os.path.join(REPO, "oracle", "_ref", "libvithost.so")),
                    reason="reference build not present")
def test_fixture_is_what_the_reference_produces_now():
    lib = golden_maker.reference_library()
    for name, (config, state, shape) in golden_maker.CASES.items():
        status, out, new_state = golden_maker.reference_apply(
            lib, config, state, golden_maker.case_source(name, shape))
        assert status == 0
        assert new_state == int(GOLDEN[name + "/state"][0])
        assert np.array_equal(out, GOLDEN[name + "/out"])
