"""Gradient accumulation, host side (CPU only): the accumulated step composed
from the reference's public pieces (vithost_train_step_accumulated) must be the
reference's own vit_model_train_batch_smoothed on the concatenated batch.

Each micro-batch loss is a mean over its rows (reference src/ops.c:1067-1070),
so K micro-batches of b images add up to K times the gradient of the mean over
K*b images; dividing by K before clip + AdamW gives the full-batch step.  The
only difference left is FP32 summation order (per micro-batch instead of over
the whole batch).
"""
import numpy as np
import pytest

CONFIG = (1, 28, 28, 4, 32, 4, 2, 11)
LR, WD, SMOOTHING = 1e-3, 0.05, 0.1


def key_bias_mask(name, array, d_model=32):
    keep = np.ones(array.shape[-1], bool)
    if name.endswith("query_key_value_bias"):
        keep[d_model:2 * d_model] = False  # exact gradient is zero: noise only
    return keep


@pytest.mark.parametrize("micro_batches,batch", [(1, 4), (2, 3), (4, 1)])
def test_accumulated_cpu_step_is_the_full_batch_step(vit_host_module, host_lib,
                                                     micro_batches, batch):
    vh = vit_host_module
    total = micro_batches * batch
    images, labels = vh.synthetic_batch(total, 28, 28, 11, 5)
    whole = vh.VitHost(host_lib, CONFIG, total)
    parts = vh.VitHost(host_lib, CONFIG, batch)
    for _ in range(3):
        expected = whole.train_step(images, labels, LR, WD, None, SMOOTHING)
        actual = parts.train_step_accumulated(
            images, labels, micro_batches, LR, WD, None, SMOOTHING,
            scale_on_host=True)
        assert abs(actual - expected) < 1e-5
    assert parts.steps() == whole.steps()
    reference = whole.parameters(0)
    for name, value in parts.parameters(0).items():
        keep = key_bias_mask(name, value)
        np.testing.assert_allclose(value[..., keep], reference[name][..., keep],
                                   rtol=0, atol=2e-5, err_msg=name)
    whole.close()
    parts.close()


def test_unscaled_sum_differs_from_the_mean(vit_host_module, host_lib):
    """Guards the test above: without the 1/K factor the step is a different
    one whenever the clip does not hide it (the norm stays below the bound
    here because the learning signal is small with label smoothing 0.9)."""
    vh = vit_host_module
    images, labels = vh.synthetic_batch(4, 28, 28, 11, 6)
    scaled = vh.VitHost(host_lib, CONFIG, 2)
    summed = vh.VitHost(host_lib, CONFIG, 2)
    scaled.train_step_accumulated(images, labels, 2, LR, WD, None, 0.9, True)
    summed.train_step_accumulated(images, labels, 2, LR, WD, None, 0.9, False)
    first = scaled.parameters(2)["head"]
    second = summed.parameters(2)["head"]
    assert np.abs(first - second).max() > 1e-6
    scaled.close()
    summed.close()
